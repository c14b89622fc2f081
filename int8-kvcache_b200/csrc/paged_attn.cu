// Paged decode attention for sm_100a over an INT8 (or bf16/fp16) block cache [num_blocks, BS, Hkv, D].
//
// Work decomposition.  The unit of work is one WARP serving one (sequence, KV head, KV split): it reads every
// 16-token tile of that head's K and V exactly once and serves all query heads of the GQA group from that single
// read (group <= 8 heads sit on the N=8 side of the tensor-core tile, so 7 heads cost 8/7 padding, not 16/7).  A
// CTA is four such warps working on consecutive items (with Hkv = 4: the four KV heads of the same pages), or a
// single warp when the grid is too small to fill the machine with 4-warp CTAs.  Warps never synchronise with
// each other; there is no __syncthreads in the attention kernels.  A sequence uses as many of the num_splits
// parts as it takes to give each about the tile count of the longest sequence's parts; partial results go to
// a workspace and merge_partials_kernel, launched with programmatic dependent launch, combines them.  For
// mid-size calls the parts are not numbered from num_splits at all: every warp derives one common part length from
// the actual seq_lens so that all parts fill whole resident waves of warps (plan_in_warp, the PLANNED
// instantiations).
//
// Data movement.  Each warp runs its own NST-deep ring of shared-memory stages filled by TMA: one
// cp.async.bulk.tensor tile load per 16x128-byte K tile and V tile, issued by lane 0, completion counted on an
// mbarrier per stage.  The tensor map views the cache as (bytes-in-row, token-in-block, head, block) and applies
// the 128-byte swizzle, which makes both access patterns below bank-conflict free.  Block ids come from
// block_tables through a register window (32 ids per load, next window prefetched; the first windows are read
// speculatively while seq_lens[b] is still in flight).  Waits are bounded: if a stage never arrives the warp
// sets a status bit, drains what it issued and returns.
//
// Math (INT8 cache).  S^T = K . Q^T with tokens on M (16 per tile), heads on N (8), dims on K, on the INT8 tensor
// cores (mma m16n8k32 s8 x s8 -> s32) with the K bytes exactly as they lie in the cache: the query is held as two
// INT8 limbs (16-bit fixed point per head) in B fragments whose k-order is permuted so that each lane's A operand
// is 32 consecutive bytes of a K row.  Two tiles are processed per loop iteration.  Online softmax runs in the
// log2 domain on the C fragments (max via three shuffles, the row sum is reduced once at the end).  P^T is
// obtained from the C fragments with movmatrix (8x8 transpose) and O^T = V^T . P^T runs as fp16 MMA m16n8k16 with
// dims on M: int8 -> fp16 is exact (bytes are spliced into 0x64xx = 1024+u and 1152 is subtracted), and the V^T
// A fragment needs pairs of tokens at one dim, produced by byte interleaving (prmt) of 16-byte row pieces on the
// way to fp16.  v_scale and 1/l are applied once in the epilogue.  The kDynScales mode reads one K and one V scale
// per (token, head) instead: they travel with the tile through the ring (cp.async, same mbarrier), K scales
// multiply the score rows, V scales ride on P behind a running power-of-two normalisation.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <utility>

#include "common.cuh"

namespace int8kv {

constexpr int kTile = 16;  // tokens per tile

// ---------------------------------------------------------------------------------------------
// Per-warp TMA ring over the tiles [t0, t1) of one (sequence, kv head).
// ---------------------------------------------------------------------------------------------
// With DYN each stage also carries the tile's 16 K scales and 16 V scales (fp32, one per token) in a 128-byte
// slot: every lane copies one of them with cp.async, whose completion arrives on the stage's mbarrier next to
// the TMA bytes.
template <int NST, int STAGE_BYTES, int LOADS_PER_TENSOR, bool DYN = false>
struct TileRing {
  uint32_t stage0;  // shared address of stage 0 (1024-byte aligned)
  uint32_t bar0;    // shared address of the first mbarrier
  const CUtensorMap* tmK;
  const CUtensorMap* tmV;
  const void* bt_row;  // block table row of this sequence
  int bt_is_i64;
  int64_t bt_stride;
  int64_t bt_limit;  // number of valid entries in the row
  int tpb;           // tiles per cache block
  int head;
  int t0;   // first tile
  int lb0;  // logical block of tile t0
  int cur_win;
  int bt_cur, bt_next;
  int lane;
  uint64_t kv_policy;  // L2 policy of the tile loads: every page is read once
  // DYN only
  uint32_t scale0;        // shared address of the first 128-byte scale slot
  const float* sc_src;    // this lane's scale cache (lanes 0-15: K, 16-31: V), offset to the lane's head
  int64_t sc_blk_stride;  // strides in elements of that cache: per block, per token
  int64_t sc_tok_stride;
  int64_t sc_blocks;      // number of blocks in the scale caches: ids outside are not read
  int seq_len;

  __device__ __forceinline__ int load_window(int win) const {
    const int64_t lb = static_cast<int64_t>(lb0) + static_cast<int64_t>(win) * 32 + lane;
    if (lb >= bt_limit) return -1;  // out-of-range ids make TMA zero-fill; such tiles are never consumed
    return static_cast<int>(load_index(bt_row, bt_is_i64, lb * bt_stride));
  }

  // Barrier set-up: touches shared memory only, so it may run before the grid dependency is resolved.
  __device__ __forceinline__ void init_barriers(int lane_) {
    lane = lane_;
    kv_policy = l2_evict_first_policy();
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < NST; ++s) mbar_init(bar0 + 8 * s, DYN ? 1 + kWarp : 1);
      mbar_fence_init();
    }
    __syncwarp();
  }

  // Speculative load of the first two block-id windows at `guess_lb0`, so that the block-table read overlaps
  // the seq_lens read that the true range depends on.
  __device__ __forceinline__ void prefetch_tables(int guess_lb0) {
    lb0 = guess_lb0;
    cur_win = 0;
    bt_cur = load_window(0);
    bt_next = load_window(1);
  }

  // Fix the range once it is known; the windows are reloaded only when the guess was wrong.
  __device__ __forceinline__ void set_range(int t0_, int tpb_) {
    t0 = t0_;
    const int real_lb0 = t0_ / tpb_;
    if (real_lb0 != lb0) {
      lb0 = real_lb0;
      bt_cur = load_window(0);
      bt_next = load_window(1);
    }
  }

  // Issue the loads of tile ordinal i (tile t0 + i) into stage i % NST.  Called by all lanes, in order of i.
  __device__ __forceinline__ void issue(int i) {
    const int tau = t0 + i;
    const int lb = tau / tpb;
    const int sub = tau - lb * tpb;
    const int idx = lb - lb0;
    const int win = idx >> 5;
    if (win != cur_win) {
      bt_cur = bt_next;
      cur_win = win;
      bt_next = load_window(win + 1);
    }
    const int blk = __shfl_sync(kFull, bt_cur, idx & 31);
    if constexpr (DYN) {
      const int st = i % NST;
      const int tok = lane & 15;
      const bool live = blk >= 0 && blk < sc_blocks && tau * kTile + tok < seq_len;  // others get scale 0
      const float* src = live ? sc_src + blk * sc_blk_stride + (sub * kTile + tok) * sc_tok_stride : sc_src;
      cp_async_4(scale0 + st * 128 + lane * 4, src, live ? 4u : 0u);
      cp_async_mbar_arrive_noinc(bar0 + 8 * st);
    }
    if (lane == 0) {
      const int st = i % NST;
      const uint32_t bar = bar0 + 8 * st;
      const uint32_t dst = stage0 + st * STAGE_BYTES;
      mbar_expect_tx(bar, STAGE_BYTES);
#pragma unroll
      for (int x = 0; x < LOADS_PER_TENSOR; ++x)
        tma_load_4d(dst + x * 2048, tmK, bar, x * 128, sub * kTile, head, blk, kv_policy);
#pragma unroll
      for (int x = 0; x < LOADS_PER_TENSOR; ++x)
        tma_load_4d(dst + (LOADS_PER_TENSOR + x) * 2048, tmV, bar, x * 128, sub * kTile, head, blk, kv_policy);
    }
  }

  // Wait for tile ordinal i; false if the bounded wait ran out on any lane.
  __device__ __forceinline__ bool wait(int i, uint32_t limit = kWaitSpinLimit) const {
    const bool ok = mbar_wait_bounded(bar0 + 8 * (i % NST), (i / NST) & 1, limit);
    return __all_sync(kFull, ok);
  }

  __device__ __forceinline__ uint32_t stage(int i) const { return stage0 + (i % NST) * STAGE_BYTES; }
  __device__ __forceinline__ uint32_t scales(int i) const { return scale0 + (i % NST) * 128; }
};

struct ItemCoord {
  int b, h, c;       // sequence, kv head, split
  int seq_len;       // tokens of the sequence (clamped to what the table can address)
  int t0, t1;        // tile range of this split
};

// Which (sequence, kv head, split) a work item is: arithmetic only.
__device__ __forceinline__ bool item_coords(const AttnParams& p, int64_t item, ItemCoord& it) {
  const int64_t total = static_cast<int64_t>(p.B) * p.num_splits * p.Hkv;
  if (item >= total) return false;
  // a grid has fewer than 2^31 CTAs, so the item number fits 32 bits: unsigned 32-bit divisions cost a fraction of
  // the 64-bit ones, and this runs in every warp's prologue
  const uint32_t i = static_cast<uint32_t>(item);
  const uint32_t r = i / static_cast<uint32_t>(p.Hkv);
  it.h = static_cast<int>(i - r * static_cast<uint32_t>(p.Hkv));
  const uint32_t b = r / static_cast<uint32_t>(p.num_splits);
  it.c = static_cast<int>(r - b * static_cast<uint32_t>(p.num_splits));
  it.b = static_cast<int>(b);
  return true;
}

// First logical block of split c if the sequence had the hinted maximum length (the guess used to start the
// block-table read early; exact for batches of full-length sequences).
__device__ __forceinline__ int guessed_first_block(const AttnParams& p, int c) {
  return static_cast<int>(static_cast<uint32_t>(c * p.per_longest) / static_cast<uint32_t>(p.tiles_per_block));
}

// The tile range of the item: reads seq_lens[b]; every sequence splits its own tiles evenly over the parts it uses.
__device__ __forceinline__ void item_range(const AttnParams& p, ItemCoord& it) {
  int64_t sl = load_index(p.sl, p.sl_is_i64, it.b);
  const int64_t cap = p.bt_width * p.block_size;
  if (sl > cap) sl = cap;
  if (sl < 0) sl = 0;
  it.seq_len = static_cast<int>(sl);
  const int ntiles = (it.seq_len + kTile - 1) / kTile;
  // A sequence uses as many of the num_splits parts as it takes to give each about the tile count that the
  // longest sequence's parts have, and leaves the rest empty: in a ragged batch every working warp then has
  // a similar amount to read, and short sequences write few partial rows.
  const uint32_t per_longest = static_cast<uint32_t>(p.per_longest);  // ceil(hint_tiles / num_splits), at least 1
  const int used = min(p.num_splits, max(1, static_cast<int>((static_cast<uint32_t>(ntiles) + per_longest - 1) / per_longest)));
  const int per = static_cast<int>(static_cast<uint32_t>(ntiles + used - 1) / static_cast<uint32_t>(used));
  it.t0 = it.c * per;
  it.t1 = it.c < used ? min(it.t0 + per, ntiles) : it.t0;
}

// Device-planned splits.  Every sequence is cut into parts of one common length P (in 16-token tiles), the smallest
// for which the parts of all sequences, W(P) = Hkv * sum_b max(1, ceil(tiles_b / P)), fit k resident waves of
// warps, for the largest k <= plan_k_max whose parts are still plan_min_part tiles long.  P comes from the actual
// lengths, so a ragged batch fills its waves as exactly as a batch of equal lengths.  There is no planning kernel
// and no item list: every warp reads seq_lens (B values, L1-resident after the first pass), computes the same P
// with the same integer arithmetic, and locates its own item in the order (sequence, part, kv head).  Returns
// false for an item number past the end.  row0 = first partial row of the item's query-head group, or -1 when
// the sequence has a single part and the result goes straight to `out`.
// Length of sequence b clamped to what its table row can address (the host admits a plan only when that bound
// is below 2^25 tokens).
__device__ __forceinline__ int plan_len(const AttnParams& p, int b, int cap) {
  if (p.sl_is_i64) {
    const long long v = __ldg(reinterpret_cast<const long long*>(p.sl) + b);
    return v > cap ? cap : (v < 0 ? 0 : static_cast<int>(v));
  }
  return min(max(__ldg(reinterpret_cast<const int*>(p.sl) + b), 0), cap);
}

// Parts of a sequence of `len` tokens cut into parts of P tiles: max(1, ceil(tiles / P)), 0 for len < 0 (no
// sequence).  No integer division: tiles + P < 2^22 is exact in fp32, rP and the product are rounded down, so the
// product can only fall short of the quotient, and by less than one.
__device__ __forceinline__ int plan_parts(int len, int P, float rP) {
  if (len < 0) return 0;
  const int n = ((len + kTile - 1) >> 4) + P - 1;
  int q = __float2int_rz(__fmul_rd(__int2float_rz(n), rP));
  if ((q + 1) * P <= n) ++q;
  return q < 1 ? 1 : q;
}

constexpr int kPlanRun = 16;  // sequences per lane: a plan covers up to 32 * 16 sequences
constexpr int kPlanShortestPart = 8;
constexpr int kPlanHeaderTag = 0x504c414e;  // marks the 16 bytes before the status word as a plan header

// What a planning warp has to leave in the workspace: the plan header (item 0) and its sequence's {first part, parts}
// entry (the warp of part 0, head 0).  The stores are made by plan_commit, which the kernels call once the grid
// dependency is resolved: with a deferred wait the preceding call's merge may still be reading the same bytes.
struct PlanNote {
  int count, part_tiles, waves;  // header, written when count >= 0
  int table_b;                   // sequence whose table entry this warp writes, or -1
  int2 table_entry;
};

__device__ __forceinline__ void plan_commit(const AttnParams& p, const PlanNote& note, int lane) {
  if (lane != 0) return;
  if (note.count >= 0 && p.plan_header != nullptr) {
    p.plan_header[0] = note.count;
    p.plan_header[1] = note.part_tiles;
    p.plan_header[2] = note.waves;
    p.plan_header[3] = kPlanHeaderTag;
  }
  if (note.table_b >= 0) p.plan_table[note.table_b] = note.table_entry;
}

__device__ __forceinline__ bool plan_in_warp(const AttnParams& p, int64_t item, int lane, ItemCoord& it, int64_t& row0,
                                             PlanNote& note) {
  // lane l holds the lengths of sequences [l * run, (l + 1) * run) in registers; every pass below works on them
  const int cap = static_cast<int>(p.bt_width * p.block_size);
  const int run = (p.B + kWarp - 1) / kWarp;
  const int b_lo = lane * run;
  int len[kPlanRun];
#pragma unroll
  for (int j = 0; j < kPlanRun; ++j) {
    len[j] = -1;
    if (j < run && b_lo + j < p.B) len[j] = plan_len(p, b_lo + j, cap);
  }
  long long total = 0;
  int longest = 0;
#pragma unroll
  for (int j = 0; j < kPlanRun; ++j) {
    if (j >= run) break;
    const int t = len[j] < 0 ? 0 : (len[j] + kTile - 1) >> 4;
    total += t;
    longest = max(longest, t);
  }
  for (int o = 16; o > 0; o >>= 1) {
    total += __shfl_xor_sync(kFull, total, o);
    longest = max(longest, __shfl_xor_sync(kFull, longest, o));
  }
  // estimate from W(P) ~ Hkv * (total / P + B / 2), then correct with the exact count
  const long long work = total * p.Hkv;
  const int floor_p = max(1, (longest + kMaxSplits - 1) / kMaxSplits);  // at most kMaxSplits parts per sequence
  int k = p.plan_k_max < 1 ? 1 : p.plan_k_max;
  int P = 1;
  for (; k >= 1; --k) {
    const long long room = static_cast<long long>(k) * p.plan_slots - static_cast<long long>(p.Hkv) * p.B / 2;
    if (room <= 0) continue;
    P = static_cast<int>((work + room - 1) / room);
    if (P >= p.plan_min_part || k == 1) break;
  }
  if (k < 1) k = 1;
  P = max(max(P, floor_p), kPlanShortestPart);  // below 8 tiles a part is mostly prologue and partial rows
  const long long target = min(static_cast<long long>(k) * p.plan_slots, static_cast<long long>(p.plan_grid_items));
  float rP = 1.f;
  int mine = 0, upto = 0;
  for (int round = 0; round < 64; ++round) {
    rP = __frcp_rd(__int2float_rz(P));
    mine = 0;
#pragma unroll
    for (int j = 0; j < kPlanRun; ++j) {
      if (j >= run) break;
      mine += plan_parts(len[j], P, rP);
    }
    upto = mine;  // inclusive scan over the lanes: lane 31 ends up with the number of parts
    for (int o = 1; o < kWarp; o <<= 1) {
      const int v = __shfl_up_sync(kFull, upto, o);
      if (lane >= o) upto += v;
    }
    const int parts = __shfl_sync(kFull, upto, kWarp - 1);
    // one part per sequence always fits: the launch covers at least B * Hkv items
    if (static_cast<long long>(parts) * p.Hkv <= target || P >= longest) break;
    P += round < 16 ? max(1, P >> 4) : P;
  }
  const int all_parts = __shfl_sync(kFull, upto, kWarp - 1);
  const long long count = static_cast<long long>(all_parts) * p.Hkv;
  note.count = item == 0 ? static_cast<int>(count) : -1;
  note.part_tiles = P;
  note.waves = k;
  note.table_b = -1;
  if (item >= count) return false;

  // the item in the order (sequence, part, kv head): its part index falls into exactly one lane's run
  const int part = static_cast<int>(item / p.Hkv);
  it.h = static_cast<int>(item - static_cast<int64_t>(part) * p.Hkv);
  const bool owner = part >= upto - mine && part < upto;
  int fb = 0, fc = 0, fused = 1, flen = 0;
  if (owner) {
    int first = upto - mine;
#pragma unroll
    for (int j = 0; j < kPlanRun; ++j) {
      if (j >= run) break;
      const int u = plan_parts(len[j], P, rP);
      if (part >= first && part < first + u) {
        fb = b_lo + j; fc = part - first; fused = u; flen = len[j];
      }
      first += u;
    }
  }
  const int src = __ffs(__ballot_sync(kFull, owner)) - 1;
  it.b = __shfl_sync(kFull, fb, src);
  it.c = __shfl_sync(kFull, fc, src);
  const int used = __shfl_sync(kFull, fused, src);
  it.seq_len = __shfl_sync(kFull, flen, src);
  const int tiles = (it.seq_len + kTile - 1) >> 4;
  const int per = (tiles + used - 1) / used;
  it.t0 = min(it.c * per, tiles);
  it.t1 = min(it.t0 + per, tiles);
  row0 = used == 1 ? -1 : static_cast<int64_t>(part) * p.Hq + it.h * p.G;
  if (it.c == 0 && it.h == 0) {
    note.table_b = it.b;
    note.table_entry = make_int2(part, used);
  }
  return true;
}

// First partial row of the item's query-head group when items are numbered arithmetically.
__device__ __forceinline__ int64_t arithmetic_row0(const AttnParams& p, const ItemCoord& it) {
  if (p.part == nullptr) return -1;
  return (static_cast<int64_t>(it.c) * p.B + it.b) * p.Hq + it.h * p.G;
}

// Where the item's result goes: the partial row of the group's first query head (the others follow), or null
// for `out`.  A planned sequence with a single part has no workspace row (row0 < 0): its result is final and
// goes to `out`, or to the caller's partial rows when those were asked for.
__device__ __forceinline__ float* result_row(const AttnParams& p, const ItemCoord& it, int64_t row0) {
  if (row0 >= 0) return p.part + row0 * p.row_floats;
  if (p.direct_part != nullptr) return p.direct_part + (static_cast<int64_t>(it.b) * p.Hq + it.h * p.G) * p.row_floats;
  return nullptr;
}

// Result of an empty tile range: zeros to `out` (direct mode) or lse = -inf (partial mode).
__device__ __forceinline__ void write_empty(const AttnParams& p, const ItemCoord& it, int lane, const float* prow) {
  if (prow == nullptr) {
    for (int hg = 0; hg < p.G; ++hg) {
      const int hq = it.h * p.G + hg;
      for (int d = lane; d < p.D; d += kWarp)
        store_from_float(p.out, p.out_dtype, it.b * p.o_st[0] + hq * p.o_st[1] + d * p.o_st[2], 0.f);
    }
  } else if (lane < p.G) {
    const_cast<float*>(prow)[lane * p.row_floats + p.D] = -INFINITY;
  }
}

// ---------------------------------------------------------------------------------------------
// Merge of one output row's partial rows by ONE warp (head_dim 128: a 16-byte piece of the row per lane).  Used by
// the chained launches, where the CTAs behind the attention items merge the PREVIOUS layer's rows while this
// layer's pages stream: off the critical path, so one warp per row, eight parts in flight, is enough.  Same
// arithmetic as merge_partials_kernel: weights exp(lse_r - max lse), parts with lse = -inf never read, all-empty
// rows give zeros.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void merge_row_by_warp(const MergeParams& p, int64_t row, int lane) {
  const int b = static_cast<int>(row / p.Hq), hq = static_cast<int>(row - static_cast<int64_t>(b) * p.Hq);
  int64_t stride_r = p.rows * p.row_floats;
  const float* base = p.parts + row * p.row_floats;
  int R = p.R;
  if (p.seq_table != nullptr) {
    const int2 e = __ldcg(p.seq_table + b);
    if (e.y <= 1) return;  // a single part went straight to the output
    R = e.y < kMaxSplits ? e.y : kMaxSplits;
    stride_r = static_cast<int64_t>(p.Hq) * p.row_floats;
    base = p.parts + (static_cast<int64_t>(e.x) * p.Hq + hq) * p.row_floats;
  }
  constexpr int kTrip = 16;  // parts whose rows are in flight together
  float w[kMaxSplits / kWarp], top = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxSplits / kWarp; ++j) {
    const int r = lane + kWarp * j;
    w[j] = r < R ? __ldcg(base + r * stride_r + p.D) : -INFINITY;
  }
  // The rows of the first trip are requested before the weights exist, so that both reads share one latency.  Rows
  // of empty parts were never written: whatever they hold is discarded by the weight test below.
  float4 o[kTrip];
#pragma unroll
  for (int u = 0; u < kTrip; ++u) {
    o[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (u < R) o[u] = __ldcg(reinterpret_cast<const float4*>(base + u * stride_r + 4 * lane));
  }
#pragma unroll
  for (int j = 0; j < kMaxSplits / kWarp; ++j) top = fmaxf(top, w[j]);
  for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, off));
  float den = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxSplits / kWarp; ++j) {
    w[j] = w[j] == -INFINITY ? 0.f : __expf(w[j] - top);
    den += w[j];
  }
  for (int off = 16; off > 0; off >>= 1) den += __shfl_xor_sync(kFull, den, off);
  const float inv = den > 0.f ? 1.f / den : 0.f;
  // Four running sums, part r into sum r % 4, added up in the order ((s0 + s1) + s2) + s3: the order in which the
  // four warps of merge_partials_kernel accumulate and combine, so that both merges return the same bits.
  float4 acc[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r0 = 0; r0 < R; r0 += kTrip) {
    const int slot = r0 >> 5;  // the same for all parts of this trip
    const float mine = slot == 0 ? w[0] : (slot == 1 ? w[1] : (slot == 2 ? w[2] : w[3]));
    float wr[kTrip];
#pragma unroll
    for (int u = 0; u < kTrip; ++u) {
      wr[u] = r0 + u < R ? __shfl_sync(kFull, mine, (r0 + u) & 31) : 0.f;
      if (r0 > 0 && wr[u] > 0.f) o[u] = __ldcg(reinterpret_cast<const float4*>(base + (r0 + u) * stride_r + 4 * lane));
    }
#pragma unroll
    for (int u = 0; u < kTrip; ++u) {
      if (wr[u] > 0.f) {
        float4& a = acc[u & 3];
        a.x += wr[u] * o[u].x; a.y += wr[u] * o[u].y; a.z += wr[u] * o[u].z; a.w += wr[u] * o[u].w;
      }
    }
  }
  float4 a;
  a.x = (acc[0].x + acc[1].x + acc[2].x + acc[3].x) * inv;
  a.y = (acc[0].y + acc[1].y + acc[2].y + acc[3].y) * inv;
  a.z = (acc[0].z + acc[1].z + acc[2].z + acc[3].z) * inv;
  a.w = (acc[0].w + acc[1].w + acc[2].w + acc[3].w) * inv;
  const int d = 4 * lane;
  const int64_t ob = b * p.o_st[0] + hq * p.o_st[1];
  if (p.out_dtype == INT8KV_BF16 && p.o_st[2] == 1 && ((reinterpret_cast<uintptr_t>(p.out) + 2 * (ob + d)) & 7u) == 0) {
    uint2 v;
    v.x = pack_bf162(a.x, a.y);
    v.y = pack_bf162(a.z, a.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + ob + d) = v;
  } else {
    store_from_float(p.out, p.out_dtype, ob + (d + 0) * p.o_st[2], a.x);
    store_from_float(p.out, p.out_dtype, ob + (d + 1) * p.o_st[2], a.y);
    store_from_float(p.out, p.out_dtype, ob + (d + 2) * p.o_st[2], a.z);
    store_from_float(p.out, p.out_dtype, ob + (d + 3) * p.o_st[2], a.w);
  }
}

// The merge share of a chained launch: warp `mw` of `cm.merge_warps` takes the rows mw, mw + merge_warps, ...
// The rows come from the launch that precedes this one on the stream, so the dependency is resolved first.
__device__ __forceinline__ void chained_merge(const ChainedMerge& cm, int mw, int lane) {
  grid_dependency_wait();
  grid_launch_dependents();
  for (int64_t row = mw; row < cm.m.rows; row += cm.merge_warps) merge_row_by_warp(cm.m, row, lane);
}
// The same share taken by an ATTENTION warp as its last act, after it has resolved the dependency for its own
// writes: attention item `item` of `cm.merge_warps` items merges the rows item, item + merge_warps, ...
__device__ __forceinline__ void chained_duty(const ChainedMerge& cm, int64_t item, int lane) {
  for (int64_t row = item; row < cm.m.rows; row += cm.merge_warps) merge_row_by_warp(cm.m, row, lane);
}

// ---------------------------------------------------------------------------------------------
// INT8 cache, D = 128, group <= 8
// ---------------------------------------------------------------------------------------------
// One V tile (16 tokens x 128 dims of one head, swizzled in shared memory) times P^T (two B registers):
// acc[j] += V^T[dims 16g+2j, 16g+2j+1 | tokens] . P^T.  `vx` are the lane's four 16-byte row pieces
// (tokens 2t, 2t+1, 2t+8, 2t+9; dims 16g..16g+15).
__device__ __forceinline__ void pv_tile(float (&acc)[8][4], const uint4 (&vx)[4], uint32_t pb0, uint32_t pb1) {
  const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&vx[0]);
  const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&vx[1]);
  const uint32_t* w2 = reinterpret_cast<const uint32_t*>(&vx[2]);
  const uint32_t* w3 = reinterpret_cast<const uint32_t*>(&vx[3]);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t x0 = w0[c] ^ 0x80808080u, x1 = w1[c] ^ 0x80808080u;
    const uint32_t x2 = w2[c] ^ 0x80808080u, x3 = w3[c] ^ 0x80808080u;
    const uint32_t lo01 = prmt(x0, x1, 0x5140u), hi01 = prmt(x0, x1, 0x7362u);
    const uint32_t lo23 = prmt(x2, x3, 0x5140u), hi23 = prmt(x2, x3, 0x7362u);
    mma_f16(acc[2 * c], u8pair_to_half2(lo01, 0x4140u), u8pair_to_half2(lo01, 0x4342u),
            u8pair_to_half2(lo23, 0x4140u), u8pair_to_half2(lo23, 0x4342u), pb0, pb1);
    mma_f16(acc[2 * c + 1], u8pair_to_half2(hi01, 0x4140u), u8pair_to_half2(hi01, 0x4342u),
            u8pair_to_half2(hi23, 0x4140u), u8pair_to_half2(hi23, 0x4342u), pb0, pb1);
  }
}

// Raw integer scores of one K tile: s[0..3] = 256 * (K . Qhi^T) + (K . Qlo^T) on the C fragment
// (rows = tokens g / g+8, cols = heads 2t / 2t+1).  The K bytes go to the tensor core as they are.
__device__ __forceinline__ void qk_tile(int (&s)[4], uint32_t kbase, const uint32_t (&koff)[4], const uint32_t (&qh)[8],
                                        const uint32_t (&ql)[8], bool two_limbs) {
  const uint4 a0 = lds128(kbase + koff[0]), a1 = lds128(kbase + koff[1]);
  const uint4 c0 = lds128(kbase + koff[2]), c1 = lds128(kbase + koff[3]);
  const uint32_t ka[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
  const uint32_t kc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
#pragma unroll
  for (int st = 0; st < 4; ++st) mma_s8(lo, ka[2 * st], kc[2 * st], ka[2 * st + 1], kc[2 * st + 1], ql[2 * st], ql[2 * st + 1]);
  if (two_limbs) {
#pragma unroll
    for (int st = 0; st < 4; ++st) mma_s8(hi, ka[2 * st], kc[2 * st], ka[2 * st + 1], kc[2 * st + 1], qh[2 * st], qh[2 * st + 1]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] = (hi[i] << 8) + lo[i];
}

// MODE: kPlain = static per-head scales; kFusedWrite = the same plus the decode step's cache write;
// kDynScales = one scale per (token, head) read from scale caches beside the INT8 pages.
constexpr int kPlain = 0, kFusedWrite = 1, kDynScales = 2;

__device__ __forceinline__ float lds32f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// The fused step's write of the new token's row, once per (sequence, kv head): quantise the row exactly as the
// cache-write kernel does, store it to the cache, and overwrite the row in the staged tile (TMA fetched the tile
// before this store, so the stage still holds the old bytes).  Out of line on purpose: one warp in Hkv-th of the
// grid runs it, once, and its 64-bit divisions and the quantiser's exact-division fallback would otherwise sit in
// the middle of every warp's streaming loop.
__device__ __noinline__ void fused_row_write(const void* kc, const void* vc, int64_t k_st0, int64_t k_st1, int64_t k_head,
                                             int64_t v_st0, int64_t v_st1, int64_t v_head, int64_t num_blocks,
                                             int block_size, int pos, int64_t new_slot, int64_t last_blk, float k0,
                                             float k1, float k2, float k3, float v0, float v1, float v2, float v3,
                                             float ks, float vsn, uint32_t stage, unsigned int* status, int lane) {
  const float rk = __frcp_rn(ks), rv = __frcp_rn(vsn);
  const uint32_t kw = pack4_sat(quant1(k0, ks, rk), quant1(k1, ks, rk), quant1(k2, ks, rk), quant1(k3, ks, rk));
  const uint32_t vw = pack4_sat(quant1(v0, vsn, rv), quant1(v1, vsn, rv), quant1(v2, vsn, rv), quant1(v3, vsn, rv));
  const int64_t expect = last_blk * block_size + pos % block_size;
  if (new_slot >= 0 && new_slot < num_blocks * block_size) {
    const int64_t blk = new_slot / block_size, off = new_slot - blk * block_size;
    int8_t* kcw = const_cast<int8_t*>(reinterpret_cast<const int8_t*>(kc));
    int8_t* vcw = const_cast<int8_t*>(reinterpret_cast<const int8_t*>(vc));
    *reinterpret_cast<uint32_t*>(kcw + blk * k_st0 + off * k_st1 + k_head + 4 * lane) = kw;
    *reinterpret_cast<uint32_t*>(vcw + blk * v_st0 + off * v_st1 + v_head + 4 * lane) = vw;
    if (new_slot == expect) {
      const uint32_t st = stage + swz128(pos & 15, lane >> 2) + (lane & 3) * 4;
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(st), "r"(kw) : "memory");
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(st + 2048), "r"(vw) : "memory");
    } else if (lane == 0 && status != nullptr) {
      atomicOr(status, INT8KV_DEV_SLOT_MISMATCH);
    }
  }
}

// PLANNED: the items come from plan_in_warp instead of being numbered arithmetically.  A template parameter rather
// than a run-time test, so that the kernel that serves small calls does not carry the planning code.
// QQ: the reference's optional INT8 query (quantize_q), one limb; its own instantiation as well.
// CHAINED: the CTAs behind the attention items merge the previous layer's partial rows (chained_merge).
template <int NST, int MODE, bool PLANNED, bool QQ, bool CHAINED>
__global__ void __launch_bounds__(kTiledWarpsPerCta * kWarp, 3)
paged_attn_int8_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const AttnParams p, const ChainedMerge cm) {
  static_assert(NST % 2 == 0, "tiles are consumed in pairs");
  constexpr bool FUSED_WRITE = MODE == kFusedWrite;
  constexpr bool DYN = MODE == kDynScales;
  constexpr int kStage = 4096;  // 16x128 K bytes + 16x128 V bytes
  extern __shared__ uint8_t smem_raw[];
  const int wpc = blockDim.x >> 5;  // warps per CTA: 1 for small grids (spread over all SMs), 4 otherwise
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if constexpr (CHAINED) {
    if (static_cast<int>(blockIdx.x) >= cm.attn_ctas) {  // a CTA seated behind the attention items only to merge
      chained_merge(cm, (static_cast<int>(blockIdx.x) - cm.attn_ctas) * wpc + warp, lane);
      return;
    }
  }

  ItemCoord it;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * wpc + warp;
  constexpr bool planned = PLANNED;
  if constexpr (planned) {
    if (item >= p.plan_grid_items) return;
  } else {
    if (!item_coords(p, item, it)) return;
  }

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  TileRing<NST, kStage, 1, DYN> ring;
  ring.stage0 = smem_base + warp * (NST * kStage);
  ring.bar0 = smem_base + wpc * NST * kStage + warp * (NST * 8);
  ring.tmK = &tmK;
  ring.tmV = &tmV;
  ring.bt_is_i64 = p.bt_is_i64;
  ring.bt_stride = p.bt_st[1];
  ring.bt_limit = p.bt_width;
  ring.tpb = p.tiles_per_block;
  if constexpr (DYN) {
    ring.scale0 = smem_base + wpc * NST * (kStage + 8) + warp * (NST * 128);
    ring.sc_blk_stride = lane >= 16 ? p.vs_st[0] : p.ks_st[0];
    ring.sc_tok_stride = lane >= 16 ? p.vs_st[1] : p.ks_st[1];
    ring.sc_blocks = p.num_blocks;
    ring.seq_len = 0;
  }
  if (lane == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  ring.init_barriers(lane);
  // Everything above used kernel parameters and shared memory only.  From here on global memory is read, which
  // the kernel launched just before this one may have written, unless the caller promised otherwise (defer_wait):
  // then the dependency is resolved only before this warp's first global write, see resolve_dependency below.
  const bool defer_wait = p.defer_wait != 0;
  if (!defer_wait) grid_dependency_wait();
  // Only now may the next kernel in the stream be scheduled (it waits for this grid before it reads): triggering
  // before the wait would let a whole chain of future kernels pile up on the SMs.  (With a deferred wait the
  // chain still ends at the merge kernel that follows, which triggers only after its own wait.)
  grid_launch_dependents();
  int64_t row0;  // first partial row of this item's query-head group, -1 = write `out`
  PlanNote note;
  note.count = -1;
  note.table_b = -1;
  // Every path that writes global memory (results, partial rows, the plan's notes) goes through here first.
  auto resolve_dependency = [&]() {
    if (defer_wait) grid_dependency_wait();
    if constexpr (planned) plan_commit(p, note, lane);
  };
  // The warp's last act in a chained launch: its share of the previous layer's merge (after resolve_dependency).
  auto merge_duty = [&]() {
    if constexpr (CHAINED) {
      if (cm.duty) chained_duty(cm, item, lane);
    }
  };
  if constexpr (planned) {
    if (!plan_in_warp(p, item, lane, it, row0, note)) {
      resolve_dependency();
      merge_duty();
      return;
    }
  }
  ring.bt_row = reinterpret_cast<const char*>(p.bt) + it.b * p.bt_st[0] * (p.bt_is_i64 ? 8 : 4);
  ring.head = it.h;
  // the head's scales are requested with the first loads of the warp; their first use is after the query's
  // conversion (k) and in the epilogue (v)
  float k_scale_head = 1.f, v_scale_head = 1.f;
  if constexpr (!DYN) {
    k_scale_head = __ldg(p.k_scale + it.h);
    v_scale_head = __ldg(p.v_scale + it.h);
  }
  if constexpr (DYN) ring.sc_src = lane >= 16 ? p.vs_cache + it.h * p.vs_st[2] : p.ks_cache + it.h * p.ks_st[2];
  if constexpr (planned) {
    ring.prefetch_tables(it.t0 / p.tiles_per_block);
  } else {
    ring.prefetch_tables(guessed_first_block(p, it.c));
    item_range(p, it);
    row0 = arithmetic_row0(p, it);
  }
  float* const prow = result_row(p, it, row0);
  if (it.t0 >= it.t1) {  // nothing was issued yet, so the warp may leave
    resolve_dependency();
    write_empty(p, it, lane, prow);
    merge_duty();
    return;
  }
  ring.set_range(it.t0, p.tiles_per_block);
  if constexpr (DYN) ring.seq_len = it.seq_len;

  // Fused decode step: the warp whose range ends with the sequence's last tile owns the step's new K/V row of
  // this head.  Everything it needs is requested right after the first tile loads below, long before the tile
  // arrives: the row (4 elements per lane), its slot, and the physical block of the last token.
  const int last_rel = ((it.seq_len - 1) >> 4) - it.t0;  // ordinal of the last tile inside this range, if any
  bool owns_new = false;
  float nk[4], nv[4];
  int64_t new_slot = -1, last_blk = -1;

  // The query is requested first (a strided or unaligned one is staged through the ring's first stage, which must
  // therefore still be idle), then the first tiles; the query's arithmetic runs while the tiles are in flight.
  float qv[32];
  if (g < p.G) {
    const int hq = it.h * p.G + g;
    load32_as_float(p.q, p.q_dtype, it.b * p.q_st[0] + hq * p.q_st[1] + 32 * t * p.q_st[2], p.q_st[2], qv, ring.stage0, lane);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) qv[i] = 0.f;
  }
  fence_proxy_async_smem();  // a staged query was written by the lanes; the first tile is written by the TMA unit
  __syncwarp();  // every lane is done with the staging area before the first tile may land in it

  const int n = it.t1 - it.t0;
  const int pre = n < NST ? n : NST;
  for (int i = 0; i < pre; ++i) ring.issue(i);
  if constexpr (FUSED_WRITE) {  // after the tile loads, so that none of these reads delays them
    owns_new = last_rel >= 0 && last_rel < it.t1 - it.t0;
    if (owns_new) {
      new_slot = load_index(p.new_slots, p.new_slot_is_i64, it.b);
      last_blk = load_index(p.bt, p.bt_is_i64, it.b * p.bt_st[0] + ((it.seq_len - 1) / p.block_size) * p.bt_st[1]);
      load4_as_float(p.new_k, p.new_dtype, it.b * p.nk_st[0] + it.h * p.nk_st[1] + 4 * lane * p.nk_st[2], p.nk_st[2], nk);
      load4_as_float(p.new_v, p.new_dtype, it.b * p.nv_st[0] + it.h * p.nv_st[1] + 4 * lane * p.nv_st[2], p.nv_st[2], nv);
    }
  }

  // ---- Q as two INT8 limbs: lane (g, t) holds head g of the group, dims [32t, 32t+32), 4 dims per word ----
  // q ~= q_mul * (256 * hi + lo) with |256 hi + lo| <= 32000: 16-bit fixed point per head, finer than the bf16
  // the query arrives in for every element that matters to the dot product.  With quantize_q the reference's
  // INT8 query (absmax/127, half away from zero) sits in the low limb alone.
  uint32_t qh[8], ql[8];
  float q_mul;
  constexpr bool two_limbs = !QQ;
  {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(qv[i]));
    amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
    int qi[32];
    if constexpr (QQ) {
      // The reference's INT8 query: q8 = clamp(round(q / qs), +-127) with qs = max(absmax / 127, 1e-6) (:137-146).
      // The quotient is formed with the reciprocal and rounded to nearest by the 1.5 * 2^23 addition: an IEEE division
      // and the reference's half-away-from-zero rule would give a different integer only for a quotient within two
      // ulp of a tie, where one query element moves by one INT8 step (far inside the attention tolerance); a chain of
      // 32 divisions, or a branch per element, costs a warp that runs alone on its SM more than a microsecond.
      const float qs = fmaxf(amax / 127.f, 1e-6f);
      const float rq = __frcp_rn(qs);
#pragma unroll
      for (int i = 0; i < 32; ++i)
        qi[i] = max(-127, min(127, __float_as_int(fmaf(qv[i], rq, kRoundMagic)) - kRoundMagicBits));
      q_mul = qs;
    } else {
      // the exact value of the factor is immaterial as long as q_mul undoes it: approximate reciprocal, no division
      // (a head whose largest element is below 1e-20 is treated as zero: its scores could not move the softmax)
      const bool live_q = amax > 1e-20f;
      const float inv = live_q ? __fdividef(32000.f, amax) : 0.f;
#pragma unroll
      // |q * inv| <= 32000 (+ rounding): adding 1.5 * 2^23 rounds to nearest and leaves the integer in the low
      // mantissa bits (an FMA on the full-rate pipe instead of a conversion)
      for (int i = 0; i < 32; ++i) qi[i] = __float_as_int(fmaf(qv[i], inv, kRoundMagic)) - kRoundMagicBits;
      q_mul = live_q ? __fdividef(1.f, inv) : 0.f;
    }
    // v = 256 * hi + lo with lo in [-128, 127]: lo is the low byte of v, hi the second byte of v + 128 (two's
    // complement), so four values pack into the two limb words with byte permutes
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t v0 = static_cast<uint32_t>(qi[4 * w]), v1 = static_cast<uint32_t>(qi[4 * w + 1]);
      const uint32_t v2 = static_cast<uint32_t>(qi[4 * w + 2]), v3 = static_cast<uint32_t>(qi[4 * w + 3]);
      ql[w] = prmt(prmt(v0, v1, 0x0040u), prmt(v2, v3, 0x0040u), 0x5410u);
      qh[w] = two_limbs ? prmt(prmt(v0 + 128u, v1 + 128u, 0x0051u), prmt(v2 + 128u, v3 + 128u, 0x0051u), 0x5410u) : 0u;
    }
  }
  // score multipliers for the two head columns (2t, 2t+1) this lane sees in the C fragment
  if constexpr (!DYN) {
    k_scale_head = fmaxf(k_scale_head, 1e-6f);
    v_scale_head = fmaxf(v_scale_head, 1e-6f);
  }
  const float kmul = k_scale_head * p.sm_scale_log2;
  const float sc0 = kmul * __shfl_sync(kFull, q_mul, (2 * t) * 4);
  const float sc1 = kmul * __shfl_sync(kFull, q_mul, (2 * t + 1) * 4);

  // swizzled offsets of this lane's row pieces inside a K tile and a V tile (constant over the loop)
  const uint32_t koff[4] = {swz128(g, 2 * t), swz128(g, 2 * t + 1), swz128(g + 8, 2 * t), swz128(g + 8, 2 * t + 1)};
  const uint32_t voff[4] = {swz128(2 * t, g), swz128(2 * t + 1, g), swz128(2 * t + 8, g), swz128(2 * t + 9, g)};

  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  // Dynamic V scales ride on P (p * v_scale[token]) into the fp16 MMA.  They are first multiplied by a power of
  // two that brings the largest scale of the first 32 tokens into [1/4, 1/2), so that the products keep fp16
  // precision whatever the magnitude of V; a later token whose scale is more than 2^11 times larger lowers the
  // factor (and the accumulators with it), like a new row maximum in the softmax.  The epilogue divides it out.
  float v_norm = 1.f, v_unnorm = 1.f;

  // Two tiles (32 tokens) per iteration: two independent score chains, one max reduction, one rescale test.
  // When the range holds an odd number of tiles the last pair's second tile is all-masked; its stage holds
  // stale bytes, which are finite integers and meet p = 0.
  bool timed_out = false;
  int i = 0;
  for (; i < n; i += 2) {
    const bool second = i + 1 < n;
    bool ok = ring.wait(i);
    if (ok && second) ok = ring.wait(i + 1);
    if (!ok) {
      timed_out = true;
      break;
    }
    const uint32_t sA = ring.stage(i), sB = ring.stage(i + 1);

    if constexpr (FUSED_WRITE) {
      // (The row's store to the cache does not need the grid dependency resolved: under the inputs-ready promise
      // nothing that precedes this call on the stream still touches this layer's cache.)
      if (owns_new && (last_rel == i || last_rel == i + 1)) {
        fused_row_write(p.kc, p.vc, p.kc_st[0], p.kc_st[1], it.h * p.kc_st[2], p.vc_st[0], p.vc_st[1], it.h * p.vc_st[2],
                        p.num_blocks, p.block_size, it.seq_len - 1, new_slot, last_blk, nk[0], nk[1], nk[2], nk[3],
                        nv[0], nv[1], nv[2], nv[3], k_scale_head, v_scale_head, ring.stage(last_rel), p.status, lane);
        fence_proxy_async_smem();  // the patched stage is refilled by the TMA unit at the end of this trip
        __syncwarp();
      }
    }

    int ia[4], ib[4];
    qk_tile(ia, sA, koff, qh, ql, two_limbs);
    qk_tile(ib, sB, koff, qh, ql, two_limbs);
    uint4 va[4], vb[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      va[r] = lds128(sA + 2048 + voff[r]);
      vb[r] = lds128(sB + 2048 + voff[r]);
    }

    // ---- online softmax on the C fragments: rows = tokens g, g+8 (tile A) and 16+g, 24+g (tile B) ----------
    const int tok0 = (it.t0 + i) * kTile + g;
    float v[8];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      v[r] = static_cast<float>(ia[r]) * ((r & 1) ? sc1 : sc0);
      v[4 + r] = static_cast<float>(ib[r]) * ((r & 1) ? sc1 : sc0);
    }
    float vsr[4] = {1.f, 1.f, 1.f, 1.f};  // V scales of rows g, g+8 (tile A), g, g+8 (tile B)
    if constexpr (DYN) {
      const uint32_t qa = ring.scales(i), qb = ring.scales(i + 1);
      const float ka0 = lds32f(qa + g * 4), ka1 = lds32f(qa + (g + 8) * 4);
      const float kb0 = second ? lds32f(qb + g * 4) : 0.f, kb1 = second ? lds32f(qb + (g + 8) * 4) : 0.f;
      v[0] *= ka0; v[1] *= ka0; v[2] *= ka1; v[3] *= ka1;
      v[4] *= kb0; v[5] *= kb0; v[6] *= kb1; v[7] *= kb1;
      vsr[0] = lds32f(qa + 64 + g * 4);
      vsr[1] = lds32f(qa + 64 + (g + 8) * 4);
      vsr[2] = second ? lds32f(qb + 64 + g * 4) : 0.f;
      vsr[3] = second ? lds32f(qb + 64 + (g + 8) * 4) : 0.f;
      // (Re)normalise: at the first pair of tiles, and whenever a token's scale would push p * scale towards the
      // top of the fp16 range; the accumulators follow by the same power of two.
      float top = fmaxf(fmaxf(vsr[0], vsr[1]), fmaxf(vsr[2], vsr[3]));
      if (i == 0 || __any_sync(kFull, top * v_norm > 1024.f)) {
        top = fmaxf(top, __shfl_xor_sync(kFull, top, 4));
        top = fmaxf(top, __shfl_xor_sync(kFull, top, 8));
        top = fmaxf(top, __shfl_xor_sync(kFull, top, 16));
        if (top > 0.f && top < INFINITY) {
          int e = (__float_as_int(top) >> 23) & 0xff;  // biased exponent: top in [2^(e-127), 2^(e-126))
          e = e < 24 ? 24 : (e > 230 ? 230 : e);
          const float nn = __int_as_float((252 - e) << 23);  // 2^(125 - e): top * nn in [1/4, 1/2)
          const float f = nn * v_unnorm;                     // new over old factor, an exact power of two
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[j][0] *= f; acc[j][1] *= f; acc[j][2] *= f; acc[j][3] *= f;
          }
          v_norm = nn;
          v_unnorm = __int_as_float((e + 2) << 23);
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) vsr[r] = fminf(vsr[r] * v_norm, 60000.f);
    }
    if (tok0 >= it.seq_len) v[0] = v[1] = -INFINITY;
    if (tok0 + 8 >= it.seq_len) v[2] = v[3] = -INFINITY;
    if (!second || tok0 + 16 >= it.seq_len) v[4] = v[5] = -INFINITY;
    if (!second || tok0 + 24 >= it.seq_len) v[6] = v[7] = -INFINITY;
    float mx0 = fmaxf(fmaxf(v[0], v[2]), fmaxf(v[4], v[6]));
    float mx1 = fmaxf(fmaxf(v[1], v[3]), fmaxf(v[5], v[7]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 4));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 4));
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 8));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 8));
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 16));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 16));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    if (__any_sync(kFull, (mn0 != m0) || (mn1 != m1))) {
      const float al0 = exp2_fast(m0 - mn0), al1 = exp2_fast(m1 - mn1);
      l0 *= al0;
      l1 *= al1;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j][0] *= al0; acc[j][1] *= al1; acc[j][2] *= al0; acc[j][3] *= al1;
      }
      m0 = mn0;
      m1 = mn1;
    }
    float pr[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) pr[r] = exp2_fast(v[r] - ((r & 1) ? m1 : m0));
    l0 += (pr[0] + pr[2]) + (pr[4] + pr[6]);
    l1 += (pr[1] + pr[3]) + (pr[5] + pr[7]);
    if constexpr (DYN) {
#pragma unroll
      for (int r = 0; r < 8; ++r) pr[r] *= vsr[r >> 1];
    }
    // P^T as B operands: (tokens 2t,2t+1 | head g), (tokens 2t+8,2t+9 | head g) for each tile
    const uint32_t pa0 = movmatrix_trans(pack_half2(pr[0], pr[1]));
    const uint32_t pa1 = movmatrix_trans(pack_half2(pr[2], pr[3]));
    const uint32_t pb0 = movmatrix_trans(pack_half2(pr[4], pr[5]));
    const uint32_t pb1 = movmatrix_trans(pack_half2(pr[6], pr[7]));

    // ---- O^T += V^T . P^T ------------------------------------------------------------------------------
    pv_tile(acc, va, pa0, pa1);
    pv_tile(acc, vb, pb0, pb1);

    __syncwarp();  // every lane has consumed both stages before lane 0 refills them
    if (i + NST < n) ring.issue(i + NST);
    if (i + 1 + NST < n) ring.issue(i + 1 + NST);
  }

  if (timed_out) {
    if (lane == 0 && p.status != nullptr) atomicOr(p.status, INT8KV_DEV_WAIT_TIMEOUT);
    // drain the loads that were already issued, again with a limit, so that none lands after this warp left
    const int issued = (i + NST < n) ? i + NST : n;
    for (int j = i; j < issued; ++j) ring.wait(j, 1u << 12);
    return;
  }

  // ---- epilogue: reduce the row sums over the token lanes, normalise, apply v_scale ----------------------
  resolve_dependency();
  l0 += __shfl_xor_sync(kFull, l0, 4);
  l1 += __shfl_xor_sync(kFull, l1, 4);
  l0 += __shfl_xor_sync(kFull, l0, 8);
  l1 += __shfl_xor_sync(kFull, l1, 8);
  l0 += __shfl_xor_sync(kFull, l0, 16);
  l1 += __shfl_xor_sync(kFull, l1, 16);
  const float vs = DYN ? v_unnorm : v_scale_head;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int hg = 2 * t + e;
    if (hg >= p.G) continue;
    const int hq = it.h * p.G + hg;
    const float l = e ? l1 : l0;
    const float m = e ? m1 : m0;
    const float inv = l > 0.f ? vs / l : 0.f;
    float o[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[2 * j] = acc[j][e] * inv;
      o[2 * j + 1] = acc[j][e + 2] * inv;
    }
    if (prow == nullptr) {
      store16_from_float(p.out, p.out_dtype, it.b * p.o_st[0] + hq * p.o_st[1] + 16 * g * p.o_st[2], p.o_st[2], o, ring.stage0, lane);
    } else {
      float* row = prow + hg * p.row_floats;
      float4* dst = reinterpret_cast<float4*>(row + 16 * g);
#pragma unroll
      for (int d = 0; d < 4; ++d) dst[d] = make_float4(o[4 * d], o[4 * d + 1], o[4 * d + 2], o[4 * d + 3]);
      if (g == 0) row[p.D] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }
  merge_duty();
}

// ---------------------------------------------------------------------------------------------
// bf16 / fp16 cache, D = 128, group <= 8: same ring, fragments straight from shared memory with ldmatrix
// ---------------------------------------------------------------------------------------------
template <bool IS_BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  return IS_BF16 ? pack_bf162(lo, hi) : pack_half2(lo, hi);
}
template <bool IS_BF16>
__device__ __forceinline__ void mma16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (IS_BF16) mma_bf16(d, a[0], a[1], a[2], a[3], b0, b1);
  else mma_f16(d, a[0], a[1], a[2], a[3], b0, b1);
}

template <int NST, bool IS_BF16, bool PLANNED, bool CHAINED>
__global__ void __launch_bounds__(kTiledWarpsPerCta * kWarp)
paged_attn_f16_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                      const AttnParams p, const ChainedMerge cm) {
  constexpr int kStage = 8192;  // K: two 16x128-byte halves (dims 0-63, 64-127), then V likewise
  extern __shared__ uint8_t smem_raw[];
  const int wpc = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if constexpr (CHAINED) {
    if (static_cast<int>(blockIdx.x) >= cm.attn_ctas) {  // a CTA seated behind the attention items only to merge
      chained_merge(cm, (static_cast<int>(blockIdx.x) - cm.attn_ctas) * wpc + warp, lane);
      return;
    }
  }

  ItemCoord it;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * wpc + warp;
  constexpr bool planned = PLANNED;
  if constexpr (planned) {
    if (item >= p.plan_grid_items) return;
  } else {
    if (!item_coords(p, item, it)) return;
  }

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  TileRing<NST, kStage, 2> ring;
  ring.stage0 = smem_base + warp * (NST * kStage);
  ring.bar0 = smem_base + wpc * NST * kStage + warp * (NST * 8);
  ring.tmK = &tmK;
  ring.tmV = &tmV;
  ring.bt_is_i64 = p.bt_is_i64;
  ring.bt_stride = p.bt_st[1];
  ring.bt_limit = p.bt_width;
  ring.tpb = p.tiles_per_block;
  if (lane == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  ring.init_barriers(lane);
  // Everything above used kernel parameters and shared memory only.  From here on global memory is read, which
  // the kernel launched just before this one may have written, unless the caller promised otherwise (defer_wait):
  // then the dependency is resolved only before this warp's first global write, see resolve_dependency below.
  const bool defer_wait = p.defer_wait != 0;
  if (!defer_wait) grid_dependency_wait();
  // Only now may the next kernel in the stream be scheduled (it waits for this grid before it reads): triggering
  // before the wait would let a whole chain of future kernels pile up on the SMs.  (With a deferred wait the
  // chain still ends at the merge kernel that follows, which triggers only after its own wait.)
  grid_launch_dependents();
  int64_t row0;  // first partial row of this item's query-head group, -1 = write `out`
  PlanNote note;
  note.count = -1;
  note.table_b = -1;
  // Every path that writes global memory (results, partial rows, the plan's notes) goes through here first.
  auto resolve_dependency = [&]() {
    if (defer_wait) grid_dependency_wait();
    if constexpr (planned) plan_commit(p, note, lane);
  };
  // The warp's last act in a chained launch: its share of the previous layer's merge (after resolve_dependency).
  auto merge_duty = [&]() {
    if constexpr (CHAINED) {
      if (cm.duty) chained_duty(cm, item, lane);
    }
  };
  if constexpr (planned) {
    if (!plan_in_warp(p, item, lane, it, row0, note)) {
      resolve_dependency();
      merge_duty();
      return;
    }
  }
  ring.bt_row = reinterpret_cast<const char*>(p.bt) + it.b * p.bt_st[0] * (p.bt_is_i64 ? 8 : 4);
  ring.head = it.h;
  if constexpr (planned) {
    ring.prefetch_tables(it.t0 / p.tiles_per_block);
  } else {
    ring.prefetch_tables(guessed_first_block(p, it.c));
    item_range(p, it);
    row0 = arithmetic_row0(p, it);
  }
  float* const prow = result_row(p, it, row0);
  if (it.t0 >= it.t1) {  // nothing was issued yet, so the warp may leave
    resolve_dependency();
    write_empty(p, it, lane, prow);
    merge_duty();
    return;
  }
  ring.set_range(it.t0, p.tiles_per_block);

  const int n = it.t1 - it.t0;
  const int pre = n < NST ? n : NST;
  for (int i = 0; i < pre; ++i) ring.issue(i);

  // Q as B fragments: step s covers dims 16s..16s+15; lane (g,t) holds head g, dims 16s+2t,+1 and 16s+8+2t,+1
  uint32_t qf[16];
  {
    const int hq = it.h * p.G + g;
    const int64_t base = it.b * p.q_st[0] + hq * p.q_st[1];
    // a query already in the cache's 16-bit type, contiguous and 4-byte aligned, is the fragment as it lies in memory
    const bool same_type = p.q_dtype == (IS_BF16 ? INT8KV_BF16 : INT8KV_FP16) && p.q_st[2] == 1 &&
                           ((reinterpret_cast<uintptr_t>(p.q) + 2 * base) & 3u) == 0;
    if (g >= p.G) {
#pragma unroll
      for (int s = 0; s < 16; ++s) qf[s] = 0u;
    } else if (same_type) {
      const uint32_t* words = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.q) + base);
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        qf[2 * s] = __ldg(words + 8 * s + t);
        qf[2 * s + 1] = __ldg(words + 8 * s + 4 + t);
      }
    } else {
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const float a = load_as_float(p.q, p.q_dtype, base + (16 * s + 2 * t) * p.q_st[2]);
        const float b = load_as_float(p.q, p.q_dtype, base + (16 * s + 2 * t + 1) * p.q_st[2]);
        const float c = load_as_float(p.q, p.q_dtype, base + (16 * s + 8 + 2 * t) * p.q_st[2]);
        const float d = load_as_float(p.q, p.q_dtype, base + (16 * s + 9 + 2 * t) * p.q_st[2]);
        qf[2 * s] = pack16<IS_BF16>(a, b);
        qf[2 * s + 1] = pack16<IS_BF16>(c, d);
      }
    }
  }
  const float sc = p.sm_scale_log2;

  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // ldmatrix lane roles: matrix mi = lane / 8, row r = lane % 8
  const int mi = lane >> 3, r = lane & 7;
  const int k_tok = r + 8 * (mi & 1), k_chunk = mi >> 1;   // K (non-transposed): matrices (tok lo/hi, chunk +0/+1)
  const int v_tok = r + 8 * (mi >> 1), v_chunk = mi & 1;   // V (transposed)

  bool timed_out = false;
  int i = 0;
  for (; i < n; ++i) {
    if (!ring.wait(i)) {
      timed_out = true;
      break;
    }
    const uint32_t kb = ring.stage(i);
    const uint32_t vb = kb + 4096;

    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const int ch = 2 * s + k_chunk;  // 16-byte chunk of the 256-byte row
      uint32_t a[4];
      ldmatrix_x4(a, kb + (ch >> 3) * 2048 + swz128(k_tok, ch & 7));
      if (s & 1) mma16<IS_BF16>(sb, a, qf[2 * s], qf[2 * s + 1]);
      else mma16<IS_BF16>(sa, a, qf[2 * s], qf[2 * s + 1]);
    }

    const int tile_tok = (it.t0 + i) * kTile;
    const int tok0 = tile_tok + g;
    float v0 = (sa[0] + sb[0]) * sc, v1 = (sa[1] + sb[1]) * sc;
    float v2 = (sa[2] + sb[2]) * sc, v3 = (sa[3] + sb[3]) * sc;
    if (tok0 >= it.seq_len) v0 = v1 = -INFINITY;
    if (tok0 + 8 >= it.seq_len) v2 = v3 = -INFINITY;
    float mx0 = fmaxf(v0, v2), mx1 = fmaxf(v1, v3);
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 4));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 4));
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 8));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 8));
    mx0 = fmaxf(mx0, __shfl_xor_sync(kFull, mx0, 16));
    mx1 = fmaxf(mx1, __shfl_xor_sync(kFull, mx1, 16));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    if (__any_sync(kFull, (mn0 != m0) || (mn1 != m1))) {
      const float al0 = exp2_fast(m0 - mn0), al1 = exp2_fast(m1 - mn1);
      l0 *= al0;
      l1 *= al1;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j][0] *= al0; acc[j][1] *= al1; acc[j][2] *= al0; acc[j][3] *= al1;
      }
      m0 = mn0;
      m1 = mn1;
    }
    const float p0 = exp2_fast(v0 - m0), p1 = exp2_fast(v1 - m1);
    const float p2 = exp2_fast(v2 - m0), p3 = exp2_fast(v3 - m1);
    l0 += p0 + p2;
    l1 += p1 + p3;
    const uint32_t pb0 = movmatrix_trans(pack16<IS_BF16>(p0, p1));
    const uint32_t pb1 = movmatrix_trans(pack16<IS_BF16>(p2, p3));

    // In the last tile of a sequence the rows past seq_len hold whatever the block had before; a float cache
    // may hold NaN/Inf there, and 0 * NaN would poison the sum, so those V values are zeroed.
    const int nvalid = it.seq_len - tile_tok;  // >= 1
    uint32_t keep_lo = 0xffffffffu, keep_hi = 0xffffffffu;  // masks for (tokens 2t,2t+1) and (2t+8,2t+9)
    if (nvalid < kTile) {
      keep_lo = (2 * t < nvalid ? 0x0000ffffu : 0u) | (2 * t + 1 < nvalid ? 0xffff0000u : 0u);
      keep_hi = (2 * t + 8 < nvalid ? 0x0000ffffu : 0u) | (2 * t + 9 < nvalid ? 0xffff0000u : 0u);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int ch = 2 * j + v_chunk;
      uint32_t a[4];
      ldmatrix_x4_trans(a, vb + (ch >> 3) * 2048 + swz128(v_tok, ch & 7));
      a[0] &= keep_lo; a[1] &= keep_lo; a[2] &= keep_hi; a[3] &= keep_hi;
      mma16<IS_BF16>(acc[j], a, pb0, pb1);
    }

    __syncwarp();
    if (i + NST < n) ring.issue(i + NST);
  }

  if (timed_out) {
    if (lane == 0 && p.status != nullptr) atomicOr(p.status, INT8KV_DEV_WAIT_TIMEOUT);
    const int issued = (i + NST < n) ? i + NST : n;
    for (int j = i + 1; j < issued; ++j) ring.wait(j, 1u << 12);
    return;
  }

  resolve_dependency();
  l0 += __shfl_xor_sync(kFull, l0, 4);
  l1 += __shfl_xor_sync(kFull, l1, 4);
  l0 += __shfl_xor_sync(kFull, l0, 8);
  l1 += __shfl_xor_sync(kFull, l1, 8);
  l0 += __shfl_xor_sync(kFull, l0, 16);
  l1 += __shfl_xor_sync(kFull, l1, 16);
  // C fragment of tile j: rows = dims 16j+g (regs 0,1) and 16j+g+8 (regs 2,3), cols = heads 2t, 2t+1
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int hg = 2 * t + e;
    if (hg >= p.G) continue;
    const int hq = it.h * p.G + hg;
    const float l = e ? l1 : l0;
    const float m = e ? m1 : m0;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (prow == nullptr) {
      const int64_t base = it.b * p.o_st[0] + hq * p.o_st[1];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        store_from_float(p.out, p.out_dtype, base + (16 * j + g) * p.o_st[2], acc[j][e] * inv);
        store_from_float(p.out, p.out_dtype, base + (16 * j + g + 8) * p.o_st[2], acc[j][e + 2] * inv);
      }
    } else {
      float* dst = prow + hg * p.row_floats;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dst[16 * j + g] = acc[j][e] * inv;
        dst[16 * j + g + 8] = acc[j][e + 2] * inv;
      }
      if (g == 0) dst[p.D] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }
  merge_duty();
}

// ---------------------------------------------------------------------------------------------
// Generic kernel: any head_dim <= 512, any block size, any group, any strides.  One warp per
// (sequence, query head, split); correctness path for shapes the tiled kernels do not cover.
// ---------------------------------------------------------------------------------------------
constexpr int kGenericMaxD = 512;

__device__ __forceinline__ float cache_elem(const void* base, int kind, int64_t idx) {
  if (kind == kCacheInt8) return static_cast<float>(reinterpret_cast<const int8_t*>(base)[idx]);
  if (kind == kCacheBf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

// KIND: cache element type (no per-element dtype branch); SLOTS: elements per lane, head_dim <= 32 * SLOTS.
// Four tokens per iteration: their loads, dot products and reductions are independent, one softmax update serves
// all four.
template <int KIND>
__device__ __forceinline__ float generic_elem(const void* base, int64_t idx) {
  if constexpr (KIND == kCacheInt8) return static_cast<float>(__ldg(reinterpret_cast<const int8_t*>(base) + idx));
  else if constexpr (KIND == kCacheBf16) return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(base) + idx));
  else return __half2float(__ldg(reinterpret_cast<const __half*>(base) + idx));
}

template <int KIND, int SLOTS>
__global__ void __launch_bounds__(128) paged_attn_generic_kernel(const AttnParams p) {
  grid_dependency_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  const int64_t total = static_cast<int64_t>(p.B) * p.num_splits * p.Hq;
  if (item >= total) return;
  const int hq = static_cast<int>(item % p.Hq);
  const int64_t rr = item / p.Hq;
  const int c = static_cast<int>(rr % p.num_splits);
  const int b = static_cast<int>(rr / p.num_splits);
  const int hkv = hq / p.G;
  int64_t sl = load_index(p.sl, p.sl_is_i64, b);
  const int64_t cap = p.bt_width * p.block_size;
  sl = sl > cap ? cap : (sl < 0 ? 0 : sl);
  const int64_t nblk = (sl + p.block_size - 1) / p.block_size;
  const int64_t per = (nblk + p.num_splits - 1) / p.num_splits;
  const int64_t tok_lo = c * per * p.block_size;
  int64_t tok_hi = (c + 1) * per * p.block_size;
  if (tok_hi > sl) tok_hi = sl;
  const int64_t row = (static_cast<int64_t>(c) * p.B + b) * p.Hq + hq;

  float q[SLOTS], acc[SLOTS];
  float q_mul = 1.f;
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int d = lane + kWarp * s;
    q[s] = d < p.D ? load_as_float(p.q, p.q_dtype, b * p.q_st[0] + hq * p.q_st[1] + d * p.q_st[2]) : 0.f;
    acc[s] = 0.f;
  }
  if (p.quantize_q) {
    float amax = 0.f;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) amax = fmaxf(amax, fabsf(q[s]));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, o));
    const float qs = fmaxf(amax / 127.f, 1e-6f);
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const float x = q[s] / qs;
      const float r = x >= 0.f ? floorf(x + 0.5f) : -floorf(-x + 0.5f);
      q[s] = fminf(fmaxf(r, -127.f), 127.f);
    }
    q_mul = qs;
  }
  const float ks = p.k_scale ? fmaxf(__ldg(p.k_scale + hkv), 1e-6f) : 1.f;
  const float vs = p.v_scale ? fmaxf(__ldg(p.v_scale + hkv), 1e-6f) : 1.f;
  const float sc = ks * q_mul * p.sm_scale_log2;
  const bool dyn = p.ks_cache != nullptr;
  float m = -INFINITY, l = 0.f;
  constexpr int kTok = 4;
  for (int64_t tok = tok_lo; tok < tok_hi; tok += kTok) {
    bool ok[kTok];
    int64_t kof[kTok], vof[kTok];
    float kt[kTok], vt[kTok], dot[kTok];
    int64_t lb = tok / p.block_size;  // one division per four tokens; the others step from it
    int off = static_cast<int>(tok - lb * p.block_size);
#pragma unroll
    for (int u = 0; u < kTok; ++u) {
      const int64_t t = tok + u;
      ok[u] = t < tok_hi;
      kof[u] = vof[u] = 0;
      kt[u] = vt[u] = 1.f;
      dot[u] = 0.f;
      if (u > 0) {
        ++off;
        while (off >= p.block_size) {
          off -= p.block_size;
          ++lb;
        }
      }
      if (ok[u]) {
        const int64_t blk = load_index(p.bt, p.bt_is_i64, b * p.bt_st[0] + lb * p.bt_st[1]);
        ok[u] = blk >= 0 && blk < p.num_blocks;  // never read outside the cache
        if (ok[u]) {
          kof[u] = blk * p.kc_st[0] + off * p.kc_st[1] + hkv * p.kc_st[2];
          vof[u] = blk * p.vc_st[0] + off * p.vc_st[1] + hkv * p.vc_st[2];
          if (dyn) {  // per-token scales of the dynamic scheme
            kt[u] = __ldg(p.ks_cache + blk * p.ks_st[0] + off * p.ks_st[1] + hkv * p.ks_st[2]);
            vt[u] = __ldg(p.vs_cache + blk * p.vs_st[0] + off * p.vs_st[1] + hkv * p.vs_st[2]);
          }
        }
      }
    }
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int d = lane + kWarp * s;
      if (d < p.D) {
#pragma unroll
        for (int u = 0; u < kTok; ++u)
          if (ok[u]) dot[u] += q[s] * generic_elem<KIND>(p.kc, kof[u] + d * p.kc_st[3]);
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < kTok; ++u) dot[u] += __shfl_xor_sync(kFull, dot[u], o);
    }
    float sv[kTok], mn = m;
#pragma unroll
    for (int u = 0; u < kTok; ++u) {
      sv[u] = ok[u] ? dot[u] * sc * kt[u] : -INFINITY;
      mn = fmaxf(mn, sv[u]);
    }
    if (mn == -INFINITY) continue;  // nothing valid so far
    const float al = exp2f(m - mn);
    float pe[kTok], sum = 0.f;
#pragma unroll
    for (int u = 0; u < kTok; ++u) {
      pe[u] = ok[u] ? exp2f(sv[u] - mn) : 0.f;
      sum += pe[u];
      pe[u] *= vt[u];
    }
    l = l * al + sum;
#pragma unroll
    for (int s = 0; s < SLOTS; ++s) {
      const int d = lane + kWarp * s;
      if (d < p.D) {
        float a = acc[s] * al;
#pragma unroll
        for (int u = 0; u < kTok; ++u)
          if (ok[u]) a += pe[u] * generic_elem<KIND>(p.vc, vof[u] + d * p.vc_st[3]);
        acc[s] = a;
      }
    }
    m = mn;
  }
  const float inv = l > 0.f ? vs / l : 0.f;
#pragma unroll
  for (int s = 0; s < SLOTS; ++s) {
    const int d = lane + kWarp * s;
    if (d >= p.D) continue;
    if (p.part == nullptr) store_from_float(p.out, p.out_dtype, b * p.o_st[0] + hq * p.o_st[1] + d * p.o_st[2], acc[s] * inv);
    else p.part[row * p.row_floats + d] = acc[s] * inv;
  }
  if (p.part != nullptr && lane == 0)
    p.part[row * p.row_floats + p.D] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
}

// ---------------------------------------------------------------------------------------------
// Grouped kernel for INT8 caches outside the tiled kernels' shapes (head_dim != 128, odd block sizes): one warp per
// (sequence, KV head, split) serves the whole GQA group from one read of the pages, with plain loads, 32 tokens
// per step.
//   rows:    lane = token.  A part's first rows are requested into L2 before the queries are staged, and the rows
//            of the NEXT step at the top of every step, so that the loads that need them find them there
//            instead of in DRAM.
//   scores:  lane = token.  Each lane walks its token's K row (16-byte loads when the layout allows) against the
//            group's queries, which sit in shared memory as two INT8 limbs per element and are read as
//            broadcasts: one dp4a per K word, head and limb, no shuffle and no conversion per dot product.
//   softmax: per head over the 32 tokens of the step (warp max and sum); the probabilities go to shared memory.
//   P.V:     32 / TPI lanes share a token, each with E consecutive dims (TPI = 2 for head_dim <= 64: two tokens
//            per load instruction, their partial sums added at the end).  The V rows of the step are requested
//            BEFORE the scores are computed (they do not depend on them), one load of E bytes per token and
//            lane; afterwards, token by token, the group's probabilities are one broadcast read and the row is
//            already in registers.
// GM bounds the group (registers per head); head_dim % 4 == 0, head_dim <= 32 * E / TPI.
// ---------------------------------------------------------------------------------------------
// Byte i of a word of four INT8 values (already XORed with 0x80808080) as a float, without the conversion unit:
// the byte becomes the low mantissa of 2^23 * 1.5 and the offset is subtracted on the FP32 adder.
template <int I>
__device__ __forceinline__ float s8_of_word(uint32_t biased) {
  return __uint_as_float(prmt(biased, 0x4B400000u, 0x7650u | I)) - 12583040.f;  // 12582912 + 128
}

__device__ __forceinline__ void prefetch_to_l2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

template <int GM, int E, int TPI>
__global__ void __launch_bounds__(128, GM == 4 ? 4 : (GM == 8 ? 3 : 2)) paged_attn_grouped_kernel(const AttnParams p) {
  static_assert((E == 4 && (TPI == 1 || TPI == 2)) || (E == 8 && TPI == 1), "lane layouts of the P.V phase");
  constexpr int LPT = kWarp / TPI;  // lanes that share one token in the P.V phase
  extern __shared__ __align__(16) float q_smem[];
  grid_dependency_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  const int64_t total = static_cast<int64_t>(p.B) * p.num_splits * p.Hkv;
  if (item >= total) return;
  const int hkv = static_cast<int>(item % p.Hkv);
  const int64_t rr = item / p.Hkv;
  const int c = static_cast<int>(rr % p.num_splits);
  const int b = static_cast<int>(rr / p.num_splits);
  const int G = p.G, D = p.D;
  int64_t sl = load_index(p.sl, p.sl_is_i64, b);
  const int64_t cap = p.bt_width * p.block_size;
  sl = sl > cap ? cap : (sl < 0 ? 0 : sl);
  const int64_t nblk = (sl + p.block_size - 1) / p.block_size;
  const int64_t per = (nblk + p.num_splits - 1) / p.num_splits;
  const int64_t tok_lo = c * per * p.block_size;
  int64_t tok_hi = (c + 1) * per * p.block_size;
  if (tok_hi > sl) tok_hi = sl;

  const int8_t* kc = reinterpret_cast<const int8_t*>(p.kc) + hkv * p.kc_st[2];  // this head's column of the caches
  const int8_t* vc = reinterpret_cast<const int8_t*>(p.vc) + hkv * p.vc_st[2];
  // whole-launch layout facts: K rows readable 16 bytes at a time, a lane's V elements readable as one word
  const bool k_vec = D % 16 == 0 && ((reinterpret_cast<uintptr_t>(p.kc) | static_cast<uintptr_t>(p.kc_st[0]) |
                                      static_cast<uintptr_t>(p.kc_st[1]) | static_cast<uintptr_t>(p.kc_st[2])) & 15u) == 0;
  const bool v_vec = D % E == 0 && ((reinterpret_cast<uintptr_t>(p.vc) | static_cast<uintptr_t>(p.vc_st[0]) |
                                     static_cast<uintptr_t>(p.vc_st[1]) | static_cast<uintptr_t>(p.vc_st[2])) & (E - 1)) == 0;

  // lane = token: logical block and offset of the lane's token, advanced by 32 tokens per step without a division
  const int step_blocks = kWarp / p.block_size, step_rest = kWarp % p.block_size;
  int64_t lb = (tok_lo + lane) / p.block_size;
  int off = static_cast<int>(tok_lo + lane - lb * p.block_size);
  // Physical block of token t (lane = token); -1 when the token is outside the part or its table entry is outside
  // the cache (such a token is never read and gets weight 0).
  auto locate = [&](int64_t t) -> int64_t {
    if (t >= tok_hi) return -1;
    const int64_t blk = load_index(p.bt, p.bt_is_i64, b * p.bt_st[0] + lb * p.bt_st[1]);
    return blk >= 0 && blk < p.num_blocks ? blk : -1;
  };
  auto advance = [&]() {
    lb += step_blocks;
    off += step_rest;
    if (off >= p.block_size) {
      off -= p.block_size;
      ++lb;
    }
  };

  // The first step's rows are located and requested into L2 before anything else, so that the query staging below
  // runs under their latency.
  int64_t blk = locate(tok_lo + lane);
  int off_cur = off;
  if (blk >= 0) {
    const int8_t* kr = kc + blk * p.kc_st[0] + off_cur * p.kc_st[1];
    const int8_t* vr_first = vc + blk * p.vc_st[0] + off_cur * p.vc_st[1];
    for (int d0 = 0; d0 < D; d0 += 32) {
      prefetch_to_l2(kr + d0);
      prefetch_to_l2(vr_first + d0);
    }
  }

  // Queries of the group as two INT8 limbs per element, four elements per word, in this warp's shared memory:
  // q ~= q_mul * (256 * hi + lo), |256 hi + lo| <= 32000 (16-bit fixed point per head, as in the tiled kernel), so
  // that a K word meets a query word in one dp4a per limb.  With quantize_q the reference's INT8 query (absmax/127,
  // half away from zero) sits in the low limb alone.  Behind the limbs: the step's probabilities [token][GM].
  int2* qw = reinterpret_cast<int2*>(q_smem + warp * (GM * 16 * E + GM * 32));
  float* ps = reinterpret_cast<float*>(qw + GM * 8 * E);
  const int row_words = D >> 2;
  const float ksc = p.k_scale ? fmaxf(__ldg(p.k_scale + hkv), 1e-6f) : 1.f;
  const float vsc = p.v_scale ? fmaxf(__ldg(p.v_scale + hkv), 1e-6f) : 1.f;
  float hmul[GM];  // score multiplier per head: k_scale * softmax scale * log2(e) * q_mul
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    hmul[g] = 0.f;
    if (g >= G) {  // unused heads of the template's group: zero limbs, so that the score loop needs no test per head
#pragma unroll
      for (int r = 0; r < E / 4; ++r)
        if (lane + kWarp * r < row_words) qw[g * row_words + lane + kWarp * r] = make_int2(0, 0);
      continue;
    }
    const int hq = hkv * G + g;
    float x[E];
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int d = 4 * lane + 128 * (e >> 2) + (e & 3);  // word lane + 32 (e / 4), element e % 4
      x[e] = d < D ? load_as_float(p.q, p.q_dtype, b * p.q_st[0] + hq * p.q_st[1] + d * p.q_st[2]) : 0.f;
      amax = fmaxf(amax, fabsf(x[e]));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, o));
    int qi[E];
    float q_mul;
    if (p.quantize_q) {
      const float qscale = fmaxf(amax / 127.f, 1e-6f);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const float y = x[e] / qscale;
        const float r = y >= 0.f ? floorf(y + 0.5f) : -floorf(-y + 0.5f);
        qi[e] = static_cast<int>(fminf(fmaxf(r, -127.f), 127.f));
      }
      q_mul = qscale;
    } else {
      const float inv = amax > 0.f ? 32000.f / amax : 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) qi[e] = __float_as_int(fmaf(x[e], inv, kRoundMagic)) - kRoundMagicBits;
      q_mul = amax > 0.f ? amax / 32000.f : 0.f;
    }
    hmul[g] = ksc * p.sm_scale_log2 * q_mul;
    // v = 256 * hi + lo with lo in [-128, 127]: lo is the low byte of v, hi the second byte of v + 128
#pragma unroll
    for (int r = 0; r < E / 4; ++r) {
      const uint32_t v0 = static_cast<uint32_t>(qi[4 * r]), v1 = static_cast<uint32_t>(qi[4 * r + 1]);
      const uint32_t v2 = static_cast<uint32_t>(qi[4 * r + 2]), v3 = static_cast<uint32_t>(qi[4 * r + 3]);
      const uint32_t lo = prmt(prmt(v0, v1, 0x0040u), prmt(v2, v3, 0x0040u), 0x5410u);
      const uint32_t hi = p.quantize_q ? 0u
                                       : prmt(prmt(v0 + 128u, v1 + 128u, 0x0051u), prmt(v2 + 128u, v3 + 128u, 0x0051u), 0x5410u);
      const int word = lane + kWarp * r;
      if (word < row_words) qw[g * row_words + word] = make_int2(static_cast<int>(hi), static_cast<int>(lo));
    }
  }
  __syncwarp();

  const bool dyn = p.ks_cache != nullptr;
  float m[GM], l[GM], acc[GM][E];
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
  }
  constexpr int VW = E / 4;                                // registers per load of a lane's V elements
  constexpr int VI = kWarp / TPI;                          // V loads per step and lane (TPI tokens per load)
  constexpr int VU = (E == 8 || GM >= 16) ? 8 : (GM >= 8 && VI > 16 ? 16 : VI);  // loads in flight together
  const int ts = lane / LPT, wcol = lane % LPT;            // P.V phase: token slot and word column of this lane
  const bool v_lane = E * wcol < D;


  for (int64_t tok0 = tok_lo; tok0 < tok_hi; tok0 += kWarp) {
    // the next step's rows: found now and requested into L2
    advance();
    const int64_t blk_next = locate(tok0 + kWarp + lane);
    const int off_next = off;
    if (blk_next >= 0) {
      const int8_t* kr = kc + blk_next * p.kc_st[0] + off_next * p.kc_st[1];
      const int8_t* vr_next = vc + blk_next * p.vc_st[0] + off_next * p.vc_st[1];
      for (int d0 = 0; d0 < D; d0 += 32) {
        prefetch_to_l2(kr + d0);
        prefetch_to_l2(vr_next + d0);
      }
    }
    const int steps = static_cast<int>(min(static_cast<int64_t>(kWarp), tok_hi - tok0));
    const bool ok = blk >= 0;
    const int64_t voff = ok ? blk * p.vc_st[0] + off_cur * p.vc_st[1] : -1;

    // V elements [E wcol, E wcol + E) of tokens i TPI + ts, for loads i0 .. i0 + VU - 1, as raw bytes
    uint32_t vr[VU][VW];
    auto load_v = [&](int i0) {
#pragma unroll
      for (int u = 0; u < VU; ++u) {
        const int64_t vo = __shfl_sync(kFull, voff, ((i0 + u) * TPI + ts) & 31);
#pragma unroll
        for (int w = 0; w < VW; ++w) vr[u][w] = 0u;
        if (vo >= 0 && v_lane) {
          const int8_t* row = vc + vo + E * wcol;
          if (v_vec) {
            if constexpr (E == 4) vr[u][0] = __ldg(reinterpret_cast<const uint32_t*>(row));
            if constexpr (E == 8) {
              const uint2 x = __ldg(reinterpret_cast<const uint2*>(row));
              vr[u][0] = x.x;
              vr[u][VW - 1] = x.y;
            }
          } else {
#pragma unroll
            for (int e = 0; e < E; ++e)
              if (E * wcol + e < D)
                vr[u][e / 4] |= static_cast<uint32_t>(static_cast<uint8_t>(__ldg(row + e))) << (8 * (e & 3));
          }
        }
      }
    };
    // O += P . V for those tokens; absent tokens have probability 0 and V bytes 0
    auto use_v = [&](int i0) {
#pragma unroll
      for (int u = 0; u < VU; ++u) {
        const int j = (i0 + u) * TPI + ts;
        float pj[GM];
#pragma unroll
        for (int g4 = 0; g4 < GM; g4 += 4) {
          const float4 x = *reinterpret_cast<const float4*>(ps + j * GM + g4);  // one address per token slot
          pj[g4] = x.x; pj[g4 + 1] = x.y; pj[g4 + 2] = x.z; pj[g4 + 3] = x.w;
        }
        float v[E];
        {
          const uint32_t w0 = vr[u][0] ^ 0x80808080u;
          v[0] = s8_of_word<0>(w0);
          v[1] = s8_of_word<1>(w0);
          v[2] = s8_of_word<2>(w0);
          v[3] = s8_of_word<3>(w0);
          if constexpr (E == 8) {
            const uint32_t w1 = vr[u][VW - 1] ^ 0x80808080u;
            v[4] = s8_of_word<0>(w1);
            v[5] = s8_of_word<1>(w1);
            v[6] = s8_of_word<2>(w1);
            v[7] = s8_of_word<3>(w1);
          }
        }
#pragma unroll
        for (int e = 0; e < E; ++e) {
#pragma unroll
          for (int g = 0; g < GM; ++g) acc[g][e] = fmaf(pj[g], v[e], acc[g][e]);
        }
      }
    };
    load_v(0);

    // ---- scores of token tok0 + lane against every head of the group ----
    int sc_hi[GM], sc_lo[GM];  // integer dot products of the K row with the two query limbs
#pragma unroll
    for (int g = 0; g < GM; ++g) sc_hi[g] = sc_lo[g] = 0;
    float vt = 1.f, kt = 1.f;
    if (ok) {
      const int8_t* krow = kc + blk * p.kc_st[0] + off_cur * p.kc_st[1];
      const bool aligned = (reinterpret_cast<uintptr_t>(krow) & 3u) == 0;
      if (dyn) {
        kt = __ldg(p.ks_cache + blk * p.ks_st[0] + off_cur * p.ks_st[1] + hkv * p.ks_st[2]);
        vt = __ldg(p.vs_cache + blk * p.vs_st[0] + off_cur * p.vs_st[1] + hkv * p.vs_st[2]);
      }
      // 64 elements at a time: all their loads are issued before the first is used
      for (int d0 = 0; d0 < D; d0 += 64) {
        int w[16];
        if (k_vec) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            int4 x = make_int4(0, 0, 0, 0);
            if (d0 + 16 * i < D) x = __ldg(reinterpret_cast<const int4*>(krow + d0 + 16 * i));
            w[4 * i] = x.x; w[4 * i + 1] = x.y; w[4 * i + 2] = x.z; w[4 * i + 3] = x.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int d = d0 + 4 * i;
            w[i] = 0;
            if (d < D) {
              if (aligned) {
                w[i] = __ldg(reinterpret_cast<const int*>(krow + d));
              } else {
                w[i] = (static_cast<int>(static_cast<uint8_t>(__ldg(krow + d)))) |
                       (static_cast<int>(static_cast<uint8_t>(__ldg(krow + d + 1))) << 8) |
                       (static_cast<int>(static_cast<uint8_t>(__ldg(krow + d + 2))) << 16) |
                       (static_cast<int>(static_cast<uint8_t>(__ldg(krow + d + 3))) << 24);
              }
            }
          }
        }
        // Words beyond the row were loaded as 0 and meet whatever limbs follow in shared memory (still inside this
        // warp's region): no test per word or per head.
        const int2* qrow = qw + (d0 >> 2);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
#pragma unroll
          for (int g = 0; g < GM; ++g) {
            const int2 qq = qrow[g * row_words + i];  // same address in every lane
            sc_hi[g] = __dp4a(w[i], qq.x, sc_hi[g]);
            sc_lo[g] = __dp4a(w[i], qq.y, sc_lo[g]);
          }
        }
      }
    }
    // ---- online softmax per head over the step's 32 tokens ----
    float pr[GM];
#pragma unroll
    for (int g = 0; g < GM; ++g) {
      pr[g] = 0.f;
      if (g < G) {
        const float score = static_cast<float>(sc_hi[g] * 256 + sc_lo[g]) * (hmul[g] * kt);
        float top = ok ? score : -INFINITY;
        for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, o));
        const float mn = fmaxf(m[g], top);
        if (mn != -INFINITY) {
          const float al = exp2f(m[g] - mn);
          const float pe = ok ? exp2f(score - mn) : 0.f;
          float sum = pe;
          for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(kFull, sum, o);
          l[g] = l[g] * al + sum;
          m[g] = mn;
          pr[g] = pe * vt;
#pragma unroll
          for (int e = 0; e < E; ++e) acc[g][e] *= al;
        }
      }
    }
    __syncwarp();  // the previous step's probabilities have been read by every lane
#pragma unroll
    for (int g4 = 0; g4 < GM; g4 += 4)
      *reinterpret_cast<float4*>(ps + lane * GM + g4) = make_float4(pr[g4], pr[g4 + 1], pr[g4 + 2], pr[g4 + 3]);
    __syncwarp();

    // ---- O += P . V ----
    use_v(0);
    for (int i0 = VU; i0 * TPI < steps; i0 += VU) {
      load_v(i0);
      use_v(i0);
    }
    blk = blk_next;
    off_cur = off_next;
  }

  if constexpr (TPI == 2) {  // the two token slots hold partial sums of the same dims
#pragma unroll
    for (int g = 0; g < GM; ++g)
#pragma unroll
      for (int e = 0; e < E; ++e) acc[g][e] += __shfl_xor_sync(kFull, acc[g][e], LPT);
  }
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    if (g >= G) continue;
    const int hq = hkv * G + g;
    const float inv = l[g] > 0.f ? vsc / l[g] : 0.f;
    const int64_t row = (static_cast<int64_t>(c) * p.B + b) * p.Hq + hq;
    if (ts == 0) {
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int d = E * wcol + e;
        if (d >= D) continue;
        if (p.part == nullptr) store_from_float(p.out, p.out_dtype, b * p.o_st[0] + hq * p.o_st[1] + d * p.o_st[2], acc[g][e] * inv);
        else p.part[row * p.row_floats + d] = acc[g][e] * inv;
      }
    }
    if (p.part != nullptr && lane == 0)
      p.part[row * p.row_floats + D] = l[g] > 0.f ? (m[g] + log2f(l[g])) * 0.6931471805599453f : -INFINITY;
  }
}

// ---------------------------------------------------------------------------------------------
// Merge of partial rows [R, rows, row_floats] (out | lse | pad): one CTA of four warps per row.
// The weights exp(lse_r - max) are computed once, in parallel over r, into shared memory; then warp w
// accumulates the parts r = w, w+4, ... with four independent 16-byte loads in flight per lane, and the four
// warp sums are combined through shared memory.  Parts with lse = -inf have weight 0 and are not read (their
// rows were never written).
// ---------------------------------------------------------------------------------------------
constexpr int kMergeWarps = 4;

// 16- and 8-byte accesses that are neither cached in L1 nor reordered with one another: the (value, epoch) pairs of
// the sequence-parallel exchange (see exchange_push_kernel)
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint2 ld_volatile_v2(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void st_volatile_v2(void* p, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

template <bool PUSH>
struct PushTarget {};
template <>
struct PushTarget<true> {
  ExchangeParams e;
};

// PUSH (sequence-parallel exchange, head dims that are multiples of 4): the merged row (out | lse) is not kept locally
// but stored as (value, epoch) pairs into slab[epoch & 1][rank] of every rank's exchange buffer, which is what
// exchange_push_kernel would have done with it in a launch of its own; p.part_out is the local staging area, where
// the attention kernel has left the rows of sequences with a single part, and those are forwarded as they are.
template <bool PUSH>
__global__ void __launch_bounds__(kMergeWarps * kWarp) merge_partials_kernel(const MergeParams p,
                                                                             const PushTarget<PUSH> push) {
  __shared__ float w_s[kMaxSplits];
  __shared__ float red_s[kMergeWarps][4 * kWarp];
  __shared__ float top_s[kMergeWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x;
  const int b = static_cast<int>(row / p.Hq), hq = static_cast<int>(row % p.Hq);
  int64_t stride_r = p.rows * p.row_floats;
  const float* base = p.parts + row * p.row_floats;
  int R = p.R;

  grid_dependency_wait();    // the partial rows come from the attention kernel launched just before
  if (p.early_trigger) grid_launch_dependents();  // the next kernel may be scheduled; it waits for this grid before reading
  uint32_t push_epoch = 0;
  int64_t push_off = 0;  // byte offset of this row in slab[epoch & 1][rank] of any rank's buffer
  int push_lo = 0, push_hi = 0;  // destination ranks
  if constexpr (PUSH) {
    const ExchangeParams& e = push.e;
    push_epoch = static_cast<uint32_t>(ld_acquire_sys(reinterpret_cast<const int*>(e.peer[e.rank]) + 1)) + 1u;
    const int64_t rank_floats = e.rows * e.row_floats;
    push_off = kExchCtrlBytes + rank_floats * 4 + (((push_epoch & 1u) * e.world + e.rank) * rank_floats + row * p.row_floats) * 8;
    if (e.scatter) {  // the row goes to its owner only
      push_lo = static_cast<int>(row / (e.rows / e.world));
      push_hi = push_lo + 1;
    } else {
      push_hi = e.world;
    }
  }
  if (p.seq_table != nullptr) {
    // device-planned splits: this sequence's parts are consecutive part indices; a single part was written to
    // `out` by the attention kernel itself
    const int2 e = __ldg(p.seq_table + b);
    if (e.y <= 1) {
      if constexpr (PUSH) {  // ... or, here, to the staging area: forward the row
        // two floats -> one 16-byte store per thread: a warp's store covers 512 consecutive bytes
        for (int t = threadIdx.x; 2 * t < p.row_floats; t += blockDim.x) {
          const float2 v = __ldcg(reinterpret_cast<const float2*>(p.part_out + row * p.row_floats) + t);
          const uint4 q = make_uint4(__float_as_uint(v.x), push_epoch, __float_as_uint(v.y), push_epoch);
          for (int r = push_lo; r < push_hi; ++r) st_volatile_v4(push.e.peer[r] + push_off + 16 * t, q);
        }
      }
      return;
    }
    R = e.y < kMaxSplits ? e.y : kMaxSplits;
    stride_r = static_cast<int64_t>(p.Hq) * p.row_floats;
    base = p.parts + (static_cast<int64_t>(e.x) * p.Hq + hq) * p.row_floats;
  }
  float lse = -INFINITY;
  if (static_cast<int>(threadIdx.x) < R) lse = __ldcg(base + threadIdx.x * stride_r + p.D);  // R <= kMaxSplits = blockDim
  // The first batch of rows is requested before the weights exist, so that both reads share one latency.
  // Rows of empty parts were never written: whatever they hold is discarded by the weight test below.
  float4 pre[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int r = warp + u * kMergeWarps;
    pre[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < R && 4 * lane < p.D) pre[u] = __ldcg(reinterpret_cast<const float4*>(base + r * stride_r + 4 * lane));
  }
  float top = lse;
  for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, o));
  if (lane == 0) top_s[warp] = top;
  __syncthreads();
  top = fmaxf(fmaxf(top_s[0], top_s[1]), fmaxf(top_s[2], top_s[3]));
  if (static_cast<int>(threadIdx.x) < R) w_s[threadIdx.x] = lse == -INFINITY ? 0.f : __expf(lse - top);
  __syncthreads();
  float den = 0.f;
  for (int r = lane; r < R; r += kWarp) den += w_s[r];
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(kFull, den, o);
  const float inv = den > 0.f ? 1.f / den : 0.f;

  for (int d0 = 0; d0 < p.D; d0 += 4 * kWarp) {
    const int d = d0 + 4 * lane;
    const bool live = d < p.D;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = warp; r0 < R; r0 += 4 * kMergeWarps) {
      float w[4];
      float4 o[4];
      const bool have = d0 == 0 && r0 == warp;  // this batch was prefetched
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * kMergeWarps;
        w[u] = r < R ? w_s[r] : 0.f;
        o[u] = pre[u];
        if (!have && live && r < R && w[u] > 0.f) o[u] = __ldcg(reinterpret_cast<const float4*>(base + r * stride_r + d));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (w[u] > 0.f) {
          a.x += w[u] * o[u].x; a.y += w[u] * o[u].y; a.z += w[u] * o[u].z; a.w += w[u] * o[u].w;
        }
      }
    }
    *reinterpret_cast<float4*>(&red_s[warp][4 * lane]) = a;
    __syncthreads();
    if (warp == 0 && live) {
      const float4 x1 = *reinterpret_cast<const float4*>(&red_s[1][4 * lane]);
      const float4 x2 = *reinterpret_cast<const float4*>(&red_s[2][4 * lane]);
      const float4 x3 = *reinterpret_cast<const float4*>(&red_s[3][4 * lane]);
      a.x = (a.x + x1.x + x2.x + x3.x) * inv;
      a.y = (a.y + x1.y + x2.y + x3.y) * inv;
      a.z = (a.z + x1.z + x2.z + x3.z) * inv;
      a.w = (a.w + x1.w + x2.w + x3.w) * inv;
      if constexpr (PUSH) {
        *reinterpret_cast<float4*>(&red_s[0][4 * lane]) = a;  // this lane's own slot: stored below by two warps
      } else if (p.part_out != nullptr) {
        *reinterpret_cast<float4*>(p.part_out + row * p.row_floats + d) = a;
      } else if (p.out_dtype == INT8KV_BF16 && p.o_st[2] == 1 && d + 3 < p.D &&
                 ((reinterpret_cast<uintptr_t>(p.out) + 2 * (b * p.o_st[0] + hq * p.o_st[1] + d)) & 7u) == 0) {
        uint2 v;
        v.x = pack_bf162(a.x, a.y);
        v.y = pack_bf162(a.z, a.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + b * p.o_st[0] + hq * p.o_st[1] + d) = v;
      } else {
        const int64_t ob = b * p.o_st[0] + hq * p.o_st[1];
        store_from_float(p.out, p.out_dtype, ob + (d + 0) * p.o_st[2], a.x);
        if (d + 1 < p.D) store_from_float(p.out, p.out_dtype, ob + (d + 1) * p.o_st[2], a.y);
        if (d + 2 < p.D) store_from_float(p.out, p.out_dtype, ob + (d + 2) * p.o_st[2], a.z);
        if (d + 3 < p.D) store_from_float(p.out, p.out_dtype, ob + (d + 3) * p.o_st[2], a.w);
      }
    }
    __syncthreads();
    if constexpr (PUSH) {
      // the chunk's merged floats leave as pairs, two floats -> one 16-byte store per thread, so that every store
      // instruction of a warp covers 512 consecutive bytes of the peer's slab (whole 128-byte lines on the links)
      const int t = threadIdx.x;
      if (t < 2 * kWarp && d0 + 2 * t < p.D) {
        const float2 v = *reinterpret_cast<const float2*>(&red_s[0][2 * t]);
        const uint4 q = make_uint4(__float_as_uint(v.x), push_epoch, __float_as_uint(v.y), push_epoch);
        for (int r = push_lo; r < push_hi; ++r) st_volatile_v4(push.e.peer[r] + push_off + 8 * d0 + 16 * t, q);
      }
      __syncthreads();  // before the next chunk reuses the slot
    }
  }
  if constexpr (PUSH) {
    if (threadIdx.x == 0) {
      const float l = den > 0.f ? top + __logf(den) : -INFINITY;
      for (int r = push_lo; r < push_hi; ++r)
        st_volatile_v2(push.e.peer[r] + push_off + 8 * p.D, make_uint2(__float_as_uint(l), push_epoch));
    }
  } else if (p.part_out != nullptr && threadIdx.x == 0) {
    p.part_out[row * p.row_floats + p.D] = den > 0.f ? top + __logf(den) : -INFINITY;
  }
}

// ---------------------------------------------------------------------------------------------
// Sequence-parallel exchange over NVLink: partial rows travel as (value, epoch) pairs.
//
// A rank's buffer is [256 B control: ticket, epoch | staging rows, fp32 | 2 slabs x world x rows x row_floats pairs |
// output slab, rows x out_floats pairs].
// Every float of a row crosses as an 8-byte pair {value, epoch of the step}; a pair is written by one store (or
// by one half of a 16-byte store) and therefore arrives whole, so the receiver needs no flag behind the data and
// the sender no system-scope fence before such a flag: it reads a pair, and the pair is this step's as soon as
// its second word says so.  (A first version sent bare rows, a fence per CTA, a ticket, and one flag per rank: the
// push alone then cost 19 us per step on two GPUs, most of it fences.)  The slab alternates with the parity of
// the epoch, so a fast rank's next step cannot overwrite what a slow rank is still merging: a rank pushes step
// e + 1 only after its own merge of step e, which needed every rank's push of step e, which followed that rank's
// merge of step e - 1.  The epoch lives in the local buffer and is advanced by the last CTA of the step's last
// kernel, so a captured graph replays.  From four ranks on a row is not sent to every rank but to one owner, which
// sends the merged row to every rank's output slab (ExchangeParams::scatter); that slab needs no second copy: an
// owner can only write step e + 1 into it after it has every rank's push of step e + 1, which follows that rank's
// last kernel of step e.
// ---------------------------------------------------------------------------------------------
// End of a step's last kernel: the ticket; the last CTA advances the epoch for the next step's kernels.  That grid
// does not wait for the push before it on the stream: whoever waits for it may find that push still waiting for the
// other GPUs to acknowledge its stores (measured: 8 us per step on two GPUs), but never reading or storing locally,
// because every row of the local push has arrived, and the next push writes the other slab.
__device__ __forceinline__ void step_ticket(int* ctrl, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int ticket = atomicAdd(ctrl, 1);
    if (ticket == static_cast<int>(gridDim.x) - 1) {
      ctrl[0] = 0;
      __threadfence();
      st_release_sys(ctrl + 1, static_cast<int>(epoch));
    }
  }
}

// Push of this rank's staged rows into slab[epoch & 1][rank] of EVERY rank's buffer: plain 16-byte stores of two
// pairs each to peer-mapped memory (no TMA, no multicast, no fence).  Nothing here waits for another GPU.
__global__ void __launch_bounds__(256) exchange_push_kernel(const ExchangeParams e) {
  grid_dependency_wait();  // the staged rows come from the kernel launched just before
  grid_launch_dependents();
  const uint32_t epoch = static_cast<uint32_t>(ld_acquire_sys(reinterpret_cast<const int*>(e.peer[e.rank]) + 1)) + 1u;
  const int64_t rank_floats = e.rows * e.row_floats;
  const int64_t n2 = rank_floats / 2;  // row_floats is a multiple of 4
  const float2* src = reinterpret_cast<const float2*>(e.peer[e.rank] + kExchCtrlBytes);
  const int64_t dst_off = kExchCtrlBytes + rank_floats * 4 + ((epoch & 1u) * e.world + e.rank) * rank_floats * 8;
  // two floats -> one 16-byte store per thread: a warp's store instruction covers 512 consecutive bytes
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n2;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float2 v = __ldcg(src + i);
    const uint4 q = make_uint4(__float_as_uint(v.x), epoch, __float_as_uint(v.y), epoch);
    if (e.scatter) {  // the row goes to its owner only
      const int owner = static_cast<int>((2 * i / e.row_floats) / (e.rows / e.world));
      st_volatile_v4(e.peer[owner] + dst_off + 16 * i, q);
    } else {
      for (int r = 0; r < e.world; ++r) st_volatile_v4(e.peer[r] + dst_off + 16 * i, q);
    }
  }
}

// Merge of the rows that all ranks pushed for the current step, from LOCAL memory: one warp per output row.  Lane r
// asks for rank r's log-sum-exp and, in the same breath, every lane for its piece of the first eight ranks' rows; the
// warp then polls until all of that carries the step's epoch (re-reading only what does not yet), so one round trip
// covers weights and data.  The arithmetic is that of merge_partials_kernel over `world` parts, operation for
// operation (weights, the shuffle tree of their sum, part r into running sum r % 4, sums combined as
// ((s0 + s1) + s2) + s3), so both exchanges return the same bits.  Waits are bounded (attempts 50 ns to 1 us apart,
// about a second in all); a rank that never arrives is reported in the status word and the row is left unwritten.
constexpr int kExchMergeWarps = 4;
constexpr int kExchChunk = 8;  // ranks whose rows a lane holds at once (two 16-byte vectors each)
// The kernel's piece of an output row to `out`, in its type and strides.
__device__ __forceinline__ void store_out4(const MergeParams& p, int b, int hq, int d, const float4& a) {
  const int64_t ob = b * p.o_st[0] + hq * p.o_st[1];
  if (p.out_dtype == INT8KV_BF16 && p.o_st[2] == 1 && d + 3 < p.D &&
      ((reinterpret_cast<uintptr_t>(p.out) + 2 * (ob + d)) & 7u) == 0) {
    uint2 v;
    v.x = pack_bf162(a.x, a.y);
    v.y = pack_bf162(a.z, a.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + ob + d) = v;
  } else {
    store_from_float(p.out, p.out_dtype, ob + (d + 0) * p.o_st[2], a.x);
    if (d + 1 < p.D) store_from_float(p.out, p.out_dtype, ob + (d + 1) * p.o_st[2], a.y);
    if (d + 2 < p.D) store_from_float(p.out, p.out_dtype, ob + (d + 2) * p.o_st[2], a.z);
    if (d + 3 < p.D) store_from_float(p.out, p.out_dtype, ob + (d + 3) * p.o_st[2], a.w);
  }
}

// SCATTER: the grid covers the rows this rank owns; the merged fp32 row is not written to `out` but, as pairs, into
// the output slab of EVERY rank, and gather_outputs_kernel (next on the stream) finishes the step.
template <bool SCATTER>
__global__ void __launch_bounds__(kExchMergeWarps * kWarp) merge_exchanged_kernel(const MergeParams p, const ExchangeParams e) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t local = static_cast<int64_t>(blockIdx.x) * kExchMergeWarps + warp;
  const int64_t owned = SCATTER ? p.rows / e.world : p.rows;
  const int64_t row = SCATTER ? e.rank * owned + local : local;
  int* ctrl = const_cast<int*>(p.exchange_ctrl);
  // The epoch is only advanced by the last CTA of the step's last kernel, after every CTA has read it.
  const uint32_t epoch = static_cast<uint32_t>(ld_acquire_sys(ctrl + 1)) + 1u;
  grid_launch_dependents();  // the next kernel may be scheduled; it waits for this grid before it reads
  if (local < owned) {
    const int R = p.exchange_world;
    const int b = static_cast<int>(row / p.Hq), hq = static_cast<int>(row - static_cast<int64_t>(b) * p.Hq);
    const int64_t rank_stride = p.rows * p.row_floats * 8;
    const char* base = reinterpret_cast<const char*>(p.parts) + (epoch & 1u) * p.slab_floats * 8 + row * p.row_floats * 8;
    uint32_t budget = kFlagSpinLimit;
    bool ok = true;
    uint2 lse_pair = make_uint2(0u, epoch);  // lanes beyond the ranks count as arrived, with weight 0
    bool lse_known = false;
    float w_mine = 0.f, inv = 0.f;
    for (int d0 = 0; ok && d0 < p.D; d0 += 4 * kWarp) {
      const int d = d0 + 4 * lane;
      const bool live = d < p.D;
      float4 acc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; ok && r0 < R; r0 += kExchChunk) {
        uint4 lo[kExchChunk], hi[kExchChunk];
        const char* src = base + r0 * rank_stride + 8 * d;
#pragma unroll
        for (int u = 0; u < kExchChunk; ++u) {
          lo[u] = hi[u] = make_uint4(0u, epoch, 0u, epoch);  // what is not asked for counts as arrived
          if (live && r0 + u < R) {
            lo[u] = ld_volatile_v4(src + u * rank_stride);
            hi[u] = ld_volatile_v4(src + u * rank_stride + 16);
          }
        }
        if (!lse_known && lane < R) lse_pair = ld_volatile_v2(base + lane * rank_stride + 8 * p.D);
        for (;;) {
          bool here = lse_pair.y == epoch;
#pragma unroll
          for (int u = 0; u < kExchChunk; ++u)
            here = here && lo[u].y == epoch && lo[u].w == epoch && hi[u].y == epoch && hi[u].w == epoch;
          if (__all_sync(kFull, here)) break;
          if (budget == 0) {
            ok = false;
            break;
          }
          --budget;
          __nanosleep(budget + 64 > kFlagSpinLimit ? 50 : 1000);
          if (lse_pair.y != epoch) lse_pair = ld_volatile_v2(base + lane * rank_stride + 8 * p.D);
#pragma unroll
          for (int u = 0; u < kExchChunk; ++u) {
            if (lo[u].y != epoch || lo[u].w != epoch) lo[u] = ld_volatile_v4(src + u * rank_stride);
            if (hi[u].y != epoch || hi[u].w != epoch) hi[u] = ld_volatile_v4(src + u * rank_stride + 16);
          }
        }
        if (!ok) break;
        if (!lse_known) {
          lse_known = true;
          const float lse = lane < R ? __uint_as_float(lse_pair.x) : -INFINITY;
          float top = lse;
          for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, o));
          w_mine = lse == -INFINITY ? 0.f : __expf(lse - top);
          float den = w_mine;
          for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(kFull, den, o);
          inv = den > 0.f ? 1.f / den : 0.f;
        }
#pragma unroll
        for (int u = 0; u < kExchChunk; ++u) {
          const float w = __shfl_sync(kFull, w_mine, (r0 + u) & 31);
          if (r0 + u < R && w > 0.f) {
            float4& a = acc[u & 3];  // kExchChunk is a multiple of 4: (r0 + u) % 4 == u % 4
            a.x += w * __uint_as_float(lo[u].x); a.y += w * __uint_as_float(lo[u].z);
            a.z += w * __uint_as_float(hi[u].x); a.w += w * __uint_as_float(hi[u].z);
          }
        }
      }
      if (!ok || !live) continue;
      float4 a;
      a.x = (acc[0].x + acc[1].x + acc[2].x + acc[3].x) * inv;
      a.y = (acc[0].y + acc[1].y + acc[2].y + acc[3].y) * inv;
      a.z = (acc[0].z + acc[1].z + acc[2].z + acc[3].z) * inv;
      a.w = (acc[0].w + acc[1].w + acc[2].w + acc[3].w) * inv;
      if constexpr (SCATTER) {
        const int64_t off = exch_out_off(e.world, e.rows, e.row_floats) + (row * e.out_floats + d) * 8;
        const uint4 lo = make_uint4(__float_as_uint(a.x), epoch, __float_as_uint(a.y), epoch);
        const uint4 hi = make_uint4(__float_as_uint(a.z), epoch, __float_as_uint(a.w), epoch);
        for (int r = 0; r < e.world; ++r) {
          st_volatile_v4(e.peer[r] + off, lo);
          st_volatile_v4(e.peer[r] + off + 16, hi);
        }
      } else {
        store_out4(p, b, hq, d, a);
      }
    }
    if (!ok && lane == 0 && p.status != nullptr) atomicOr(p.status, INT8KV_DEV_WAIT_TIMEOUT);
  }
  if constexpr (!SCATTER) step_ticket(ctrl, epoch);
}

// Last kernel of a step in the scatter form: every rank takes every merged row from its output slab (one warp per
// row, polling as above, bounded) and writes it to `out`.
__global__ void __launch_bounds__(kExchMergeWarps * kWarp) gather_outputs_kernel(const MergeParams p, const ExchangeParams e) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * kExchMergeWarps + warp;
  int* ctrl = const_cast<int*>(p.exchange_ctrl);
  const uint32_t epoch = static_cast<uint32_t>(ld_acquire_sys(ctrl + 1)) + 1u;
  grid_launch_dependents();
  if (row < p.rows) {
    const int b = static_cast<int>(row / p.Hq), hq = static_cast<int>(row - static_cast<int64_t>(b) * p.Hq);
    const char* base = e.peer[e.rank] + exch_out_off(e.world, e.rows, e.row_floats) + row * e.out_floats * 8;
    uint32_t budget = kFlagSpinLimit;
    bool ok = true;
    for (int d0 = 0; ok && d0 < p.D; d0 += 4 * kWarp) {
      const int d = d0 + 4 * lane;
      const bool live = d < p.D;
      uint4 lo = make_uint4(0u, epoch, 0u, epoch), hi = lo;  // lanes beyond the row count as arrived
      if (live) {
        lo = ld_volatile_v4(base + 8 * d);
        hi = ld_volatile_v4(base + 8 * d + 16);
      }
      for (;;) {
        const bool here = lo.y == epoch && lo.w == epoch && hi.y == epoch && hi.w == epoch;
        if (__all_sync(kFull, here)) break;
        if (budget == 0) {
          ok = false;
          break;
        }
        --budget;
        __nanosleep(budget + 64 > kFlagSpinLimit ? 50 : 1000);
        if (lo.y != epoch || lo.w != epoch) lo = ld_volatile_v4(base + 8 * d);
        if (hi.y != epoch || hi.w != epoch) hi = ld_volatile_v4(base + 8 * d + 16);
      }
      if (ok && live)
        store_out4(p, b, hq, d, make_float4(__uint_as_float(lo.x), __uint_as_float(lo.z), __uint_as_float(hi.x), __uint_as_float(hi.z)));
    }
    if (!ok && lane == 0 && p.status != nullptr) atomicOr(p.status, INT8KV_DEV_WAIT_TIMEOUT);
  }
  step_ticket(ctrl, epoch);
}

int launch_exchange_push(const ExchangeParams& e, cudaStream_t stream) {
  const int64_t n2 = e.rows * e.row_floats / 2;
  if (n2 <= 0) return INT8KV_OK;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n2 + 255) / 256, 148 * 8));
  return launch_pdl(exchange_push_kernel, grid, 256, 0, stream, e);
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one warp arms an mbarrier for bytes that no copy will ever deliver, waits with a
// small attempt limit, and reports the timeout in the status word exactly as the attention kernels do.  It
// returns normally; the context stays usable.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(unsigned int* status, unsigned int attempts) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(addr, 1);
    mbar_fence_init();
    mbar_expect_tx(addr, 16);  // the phase now waits for 16 bytes that nothing sends
  }
  __syncwarp();
  const bool ok = mbar_wait_bounded(addr, 0, attempts);
  if (!__all_sync(kFull, ok) && threadIdx.x == 0) atomicOr(status, INT8KV_DEV_WAIT_TIMEOUT);
}

int launch_bounded_wait_selftest(unsigned int* status, unsigned int attempts, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, attempts);
  return cudaGetLastError() == cudaSuccess ? INT8KV_OK : INT8KV_E_LAUNCH;
}

// ---------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------
constexpr int kInt8Stages = 4;
constexpr int kF16Stages = 3;

// The dynamic shared-memory limit is raised once per (kernel, device); later calls, which may sit inside a
// stream capture, launch without touching function attributes.
template <int KERNEL_TAG, typename K>  // the tag keeps one flag array per kernel: the kernels share a signature
static int set_smem(K kernel, int bytes) {
  static std::atomic<bool> done[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  const bool track = dev >= 0 && dev < 64;
  if (track && done[dev].load(std::memory_order_acquire)) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -1;
  if (track) done[dev].store(true, std::memory_order_release);
  return 0;
}

// Item numbers a tiled launch covers: the capacity of the planned list, or B * num_splits * Hkv.
static int64_t grid_items(const AttnParams& p) {
  if (p.plan_table != nullptr) return p.plan_grid_items;
  return static_cast<int64_t>(p.B) * p.num_splits * p.Hkv;
}

// Warps per CTA: a grid that cannot fill the machine with 4-warp CTAs is launched as 1-warp CTAs so that its
// warps spread over all SMs instead of stacking four to an SM.
static int pick_wpc(int64_t items, int sm_count) {
  return items <= static_cast<int64_t>(sm_count) * 12 ? 1 : kTiledWarpsPerCta;
}

// Grid of a tiled launch, and who merges the previous layer's rows when the launch carries such a merge (chained
// layers).  Measured per layer on B200, trailing CTAs against duty:
//   * one-warp CTAs with parts of 8 tiles or more (the mid-size calls, device-planned parts included): the attention
//     warps take the merge as their last act — B=8 x 4096 tokens 8.6 -> 6.2 us, B=1 x 4096 7.0 -> 4.0 us, one KV head x
//     128 ragged sequences (one full wave of warps, so trailing CTAs would find no free slot until it drains)
//     33.0 -> 29.2 us;
//   * four-warp CTAs (several waves): CTAs appended behind the attention items, which run in the shadow of the last
//     wave — the ragged 256-sequence batch 191.7 us against 194.8 us with the duty, which adds a merge to every warp's life;
//   * parts shorter than 8 tiles (a few megabytes per call): appended CTAs as well, which merge beside the attention
//     warps' own writes instead of behind them — B=1 x 512 tokens 2.8 us against 3.7 us.
// Appended CTAs number as many as the previous layer has rows per CTA's warps, but no more than the slots the
// attention CTAs leave free on the device (so that the whole grid is scheduled at once and the next launch is not
// held back), and at least one per SM; each merge warp then walks several rows.
struct TiledGrid {
  unsigned ctas;
  ChainedMerge cm;
};
static TiledGrid tiled_grid(const AttnParams& p, int64_t items, int wpc, int ctas_per_sm, int sm_count,
                            const MergeParams* prev) {
  TiledGrid g;
  std::memset(&g, 0, sizeof(g));
  const int64_t attn = (items + wpc - 1) / wpc;
  g.cm.attn_ctas = static_cast<int>(attn);
  g.ctas = static_cast<unsigned>(attn);
  if (prev == nullptr || prev->rows <= 0) return g;
  g.cm.m = *prev;
  const int part_tiles = p.plan_table != nullptr ? 8 : p.per_longest;  // a plan never cuts parts below 8 tiles
  if (wpc == 1 && part_tiles >= 8) {
    g.cm.duty = 1;
    g.cm.merge_warps = static_cast<int>(items);
    return g;
  }
  const int64_t want = (prev->rows + wpc - 1) / wpc;
  const int64_t spare = static_cast<int64_t>(sm_count) * ctas_per_sm - attn;
  const int64_t merge_ctas = std::max<int64_t>(1, std::min<int64_t>(want, std::max<int64_t>(sm_count, spare)));
  g.cm.merge_warps = static_cast<int>(merge_ctas * wpc);
  g.ctas += static_cast<unsigned>(merge_ctas);
  return g;
}

// One instantiation of the INT8 kernel: raises its dynamic shared-memory limit once, sizes the grid, launches.
template <int NST, int MODE, bool PLANNED, bool QQ = false, bool CHAINED = false>
static int launch_int8_variant(const AttnParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, int sm_count,
                               cudaStream_t stream, const MergeParams* prev = nullptr) {
  constexpr int per_warp = NST * (4096 + 8 + (MODE == kDynScales ? 128 : 0));  // stages, barriers, scale slots
  auto kernel = paged_attn_int8_kernel<NST, MODE, PLANNED, QQ, CHAINED>;
  if (set_smem<100 + NST * 32 + MODE * 8 + (PLANNED ? 4 : 0) + (QQ ? 2 : 0) + (CHAINED ? 1 : 0)>(
          kernel, kTiledWarpsPerCta * per_warp + 1024) != 0)
    return INT8KV_E_LAUNCH;
  const int64_t items = grid_items(p);
  if (items <= 0) return INT8KV_OK;
  if (items >= (int64_t(1) << 31)) return INT8KV_E_UNSUPPORTED;  // the kernels number their items in 32 bits
  const int wpc = pick_wpc(items, sm_count);
  const size_t smem = static_cast<size_t>(wpc) * per_warp + 1024;
  const int ctas_per_sm = std::min<int>(wpc == 1 ? 32 : 3, static_cast<int>((227 * 1024) / smem));
  const TiledGrid g = tiled_grid(p, items, wpc, ctas_per_sm, sm_count, CHAINED ? prev : nullptr);
  return launch_pdl(kernel, g.ctas, wpc * kWarp, smem, stream, tmK, tmV, p, g.cm);
}

int launch_attn_tiled_int8(const AttnParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, int sm_count,
                           cudaStream_t stream, const MergeParams* prev) {
  constexpr int N = kInt8Stages;
  const bool planned = p.plan_table != nullptr;
  if (prev != nullptr && prev->rows > 0) {  // static scales, no INT8 query: the caller has checked
    if (planned)
      return p.new_k != nullptr ? launch_int8_variant<N, kFusedWrite, true, false, true>(p, tmK, tmV, sm_count, stream, prev)
                                : launch_int8_variant<N, kPlain, true, false, true>(p, tmK, tmV, sm_count, stream, prev);
    return p.new_k != nullptr ? launch_int8_variant<N, kFusedWrite, false, false, true>(p, tmK, tmV, sm_count, stream, prev)
                              : launch_int8_variant<N, kPlain, false, false, true>(p, tmK, tmV, sm_count, stream, prev);
  }
  if (p.ks_cache != nullptr)
    return planned ? launch_int8_variant<N, kDynScales, true>(p, tmK, tmV, sm_count, stream)
                   : launch_int8_variant<N, kDynScales, false>(p, tmK, tmV, sm_count, stream);
  if (p.quantize_q && p.new_k == nullptr)  // the INT8 query exists without the fused write only
    return planned ? launch_int8_variant<N, kPlain, true, true>(p, tmK, tmV, sm_count, stream)
                   : launch_int8_variant<N, kPlain, false, true>(p, tmK, tmV, sm_count, stream);
  if (planned)
    return p.new_k != nullptr ? launch_int8_variant<N, kFusedWrite, true>(p, tmK, tmV, sm_count, stream)
                              : launch_int8_variant<N, kPlain, true>(p, tmK, tmV, sm_count, stream);
  return p.new_k != nullptr ? launch_int8_variant<N, kFusedWrite, false>(p, tmK, tmV, sm_count, stream)
                            : launch_int8_variant<N, kPlain, false>(p, tmK, tmV, sm_count, stream);
}

template <bool IS_BF16, bool PLANNED, bool CHAINED = false>
static int launch_f16(const AttnParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, int sm_count,
                      cudaStream_t stream, const MergeParams* prev = nullptr) {
  constexpr int smem_max = kTiledWarpsPerCta * kF16Stages * 8192 + kTiledWarpsPerCta * kF16Stages * 8 + 1024;
  auto kernel = paged_attn_f16_kernel<kF16Stages, IS_BF16, PLANNED, CHAINED>;
  if (set_smem<(IS_BF16 ? 1 : 2) + (PLANNED ? 2 : 0) + (CHAINED ? 4 : 0)>(kernel, smem_max) != 0) return INT8KV_E_LAUNCH;
  const int64_t items = grid_items(p);
  if (items <= 0) return INT8KV_OK;
  if (items >= (int64_t(1) << 31)) return INT8KV_E_UNSUPPORTED;  // the kernels number their items in 32 bits
  const int wpc = pick_wpc(items, sm_count);
  const size_t smem = static_cast<size_t>(wpc) * kF16Stages * 8192 + wpc * kF16Stages * 8 + 1024;
  const int ctas_per_sm = std::min<int>(wpc == 1 ? 32 : 4, static_cast<int>((227 * 1024) / smem));
  const TiledGrid g = tiled_grid(p, items, wpc, ctas_per_sm, sm_count, CHAINED ? prev : nullptr);
  return launch_pdl(kernel, g.ctas, wpc * kWarp, smem, stream, tmK, tmV, p, g.cm);
}

int launch_attn_tiled_f16(const AttnParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, int sm_count,
                          cudaStream_t stream, const MergeParams* prev) {
  const bool planned = p.plan_table != nullptr;
  if (prev != nullptr && prev->rows > 0) {
    if (p.cache_kind == kCacheBf16)
      return planned ? launch_f16<true, true, true>(p, tmK, tmV, sm_count, stream, prev)
                     : launch_f16<true, false, true>(p, tmK, tmV, sm_count, stream, prev);
    return planned ? launch_f16<false, true, true>(p, tmK, tmV, sm_count, stream, prev)
                   : launch_f16<false, false, true>(p, tmK, tmV, sm_count, stream, prev);
  }
  if (p.cache_kind == kCacheBf16)
    return planned ? launch_f16<true, true>(p, tmK, tmV, sm_count, stream)
                   : launch_f16<true, false>(p, tmK, tmV, sm_count, stream);
  return planned ? launch_f16<false, true>(p, tmK, tmV, sm_count, stream)
                 : launch_f16<false, false>(p, tmK, tmV, sm_count, stream);
}

int launch_attn_generic(const AttnParams& p, cudaStream_t stream) {
  if (p.D > kGenericMaxD) return INT8KV_E_UNSUPPORTED;
  const int64_t items = static_cast<int64_t>(p.B) * p.num_splits * p.Hq;
  if (items <= 0) return INT8KV_OK;
  // INT8 caches with a head_dim that is a multiple of 4 (up to 256) and a group of up to 16: one read of the pages
  // serves the whole group
  if (p.cache_kind == kCacheInt8 && p.D % 4 == 0 && p.D <= 256 && p.G <= 16 && p.kc_st[3] == 1 && p.vc_st[3] == 1) {
    const int gm = p.G <= 4 ? 4 : (p.G <= 8 ? 8 : 16);
    const int e = p.D <= 128 ? 4 : 8;       // elements per lane in the P.V phase
    const int tpi = p.D <= 64 ? 2 : 1;      // tokens per V load: half a warp covers a row of up to 64 bytes
    if (gm * e <= 64) {
      const int64_t gitems = static_cast<int64_t>(p.B) * p.num_splits * p.Hkv;
      const unsigned ggrid = static_cast<unsigned>((gitems + 3) / 4);
      const size_t smem = static_cast<size_t>(4) * (gm * 16 * e + gm * 32) * sizeof(float);  // query limbs + probabilities
      auto grouped = [&](auto kernel) { return launch_pdl(kernel, ggrid, 128, smem, stream, p); };
      if (gm == 4 && tpi == 2) return grouped(paged_attn_grouped_kernel<4, 4, 2>);
      if (gm == 4 && e == 4) return grouped(paged_attn_grouped_kernel<4, 4, 1>);
      if (gm == 4 && e == 8) return grouped(paged_attn_grouped_kernel<4, 8, 1>);
      if (gm == 8 && tpi == 2) return grouped(paged_attn_grouped_kernel<8, 4, 2>);
      if (gm == 8 && e == 4) return grouped(paged_attn_grouped_kernel<8, 4, 1>);
      if (gm == 8 && e == 8) return grouped(paged_attn_grouped_kernel<8, 8, 1>);
      if (tpi == 2) return grouped(paged_attn_grouped_kernel<16, 4, 2>);
      return grouped(paged_attn_grouped_kernel<16, 4, 1>);
    }
  }
  const unsigned grid = static_cast<unsigned>((items + 3) / 4);
  auto go = [&](auto kernel) { return launch_pdl(kernel, grid, 128, 0, stream, p); };
  auto by_slots = [&](auto kind) {
    constexpr int K = decltype(kind)::value;
    if (p.D <= 64) return go(paged_attn_generic_kernel<K, 2>);
    if (p.D <= 128) return go(paged_attn_generic_kernel<K, 4>);
    if (p.D <= 256) return go(paged_attn_generic_kernel<K, 8>);
    return go(paged_attn_generic_kernel<K, 16>);
  };
  if (p.cache_kind == kCacheInt8) return by_slots(std::integral_constant<int, kCacheInt8>{});
  if (p.cache_kind == kCacheBf16) return by_slots(std::integral_constant<int, kCacheBf16>{});
  return by_slots(std::integral_constant<int, kCacheFp16>{});
}

int launch_merge(const MergeParams& p_in, cudaStream_t stream) {
  MergeParams p = p_in;
  // A short merge lets the next kernel in the stream be scheduled while it runs (measured: 0.4-0.8 us per call on
  // small decode calls); a long one would only have that kernel's CTAs crowd the SMs it still needs.
  p.early_trigger = p.inputs_ready || p.rows * p.R <= 4096;
  if (p.rows <= 0) return INT8KV_OK;
  return launch_pdl(merge_partials_kernel<false>, static_cast<unsigned>(p.rows), kMergeWarps * kWarp, 0, stream, p,
                    PushTarget<false>{});
}

int launch_merge_push(const MergeParams& p_in, const ExchangeParams& e, cudaStream_t stream) {
  MergeParams p = p_in;
  p.early_trigger = 1;  // what follows is the merge of the exchanged rows, which polls for them
  if (p.rows <= 0) return INT8KV_OK;
  PushTarget<true> t;
  t.e = e;
  return launch_pdl(merge_partials_kernel<true>, static_cast<unsigned>(p.rows), kMergeWarps * kWarp, 0, stream, p, t);
}

// phase: INT8KV_EXCHANGE_BOTH_PHASES, or one of the two halves of the scatter form (without the scatter form the merge
// phase is the whole step and the gather phase nothing)
int launch_merge_exchanged(const MergeParams& p, const ExchangeParams& e, int phase, cudaStream_t stream) {
  if (p.rows <= 0) return INT8KV_OK;
  const unsigned grid = static_cast<unsigned>((p.rows + kExchMergeWarps - 1) / kExchMergeWarps);
  if (!e.scatter) {
    if (phase == INT8KV_EXCHANGE_GATHER_PHASE) return INT8KV_OK;
    return launch_pdl(merge_exchanged_kernel<false>, grid, kExchMergeWarps * kWarp, 0, stream, p, e);
  }
  if (phase != INT8KV_EXCHANGE_GATHER_PHASE) {
    const int64_t owned = p.rows / e.world;
    const unsigned own_grid = static_cast<unsigned>((owned + kExchMergeWarps - 1) / kExchMergeWarps);
    const int rc = launch_pdl(merge_exchanged_kernel<true>, own_grid, kExchMergeWarps * kWarp, 0, stream, p, e);
    if (rc != INT8KV_OK || phase == INT8KV_EXCHANGE_MERGE_PHASE) return rc;
  }
  return launch_pdl(gather_outputs_kernel, grid, kExchMergeWarps * kWarp, 0, stream, p, e);
}

}  // namespace int8kv
