// Parameter blocks and host launchers shared by the kernel files and the C-ABI layer.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace int8kv {

struct WriteParams {
  const void* key;
  const void* value;
  int in_dtype;
  int64_t T;
  int Hkv, D;
  int64_t k_st[3], v_st[3];
  int8_t* kc;
  int8_t* vc;
  int64_t kc_st[4], vc_st[4];
  int64_t num_slots;
  int block_size;
  const void* slots;
  int slot_is_i64;
  const float* k_scale;
  const float* v_scale;
};

struct DynWriteParams {
  const void* key;
  const void* value;
  int in_dtype;
  int64_t T;
  int Hkv, D;
  int64_t k_st[3], v_st[3];
  int8_t* kc;
  int8_t* vc;
  int64_t kc_st[4], vc_st[4];
  float* ks;  // per-(slot, head) scale caches [num_blocks, BS, Hkv]
  float* vs;
  int64_t ks_st[3], vs_st[3];
  int64_t num_slots;
  int block_size;
  const void* slots;
  int slot_is_i64;
};

// cache element kinds
enum CacheKind { kCacheInt8 = 0, kCacheBf16 = 1, kCacheFp16 = 2 };

struct AttnParams {
  const void* q;
  int q_dtype;
  int64_t q_st[3];
  int B, Hq, Hkv, G, D;
  const void* kc;  // cache base pointers (used directly by the generic kernel; the tiled kernels use tensor maps)
  const void* vc;
  int cache_kind;
  int64_t kc_st[4];
  int64_t vc_st[4];
  int64_t num_blocks;
  int block_size;
  int tiles_per_block;  // block_size / 16 (tiled kernels)
  int hint_tiles;       // ceil(max_seq_len hint / 16): sizes the grid and seeds the block-table prefetch
  int per_longest;      // ceil(hint_tiles / num_splits), at least 1: tiles per part of the longest sequence
  const void* bt;
  int bt_is_i64;
  int64_t bt_st[2];
  int64_t bt_width;
  const void* sl;
  int sl_is_i64;
  const float* k_scale;  // null for float caches
  const float* v_scale;
  void* out;  // final output, used when `part` is null
  int out_dtype;
  int64_t o_st[3];
  int num_splits;
  float* part;  // [num_splits, B*Hq, row_floats] partial rows; null = write `out` directly (num_splits must be 1)
  int row_floats;
  int quantize_q;
  float sm_scale_log2;   // log2(e) / sqrt(D)
  unsigned int* status;  // device status word, may be null
  // Caller's promise that nothing this call reads is written by the kernel that precedes it on the stream: the
  // tiled kernels then start reading at once and resolve the grid dependency only before their first global write
  // (the split-KV workspace may still be in use by the preceding call's merge until then).
  int defer_wait;
  // fused decode step: the step's new K/V row of every sequence ([B, Hkv, D]) is quantised and written at
  // new_slots[b] by the warp that owns the sequence's last tile, which also patches its staged copy of the tile
  const void* new_k;  // null = plain attention
  const void* new_v;
  int new_dtype;
  int64_t nk_st[3], nv_st[3];
  const void* new_slots;
  int new_slot_is_i64;
  // dynamic scales: one fp32 scale per (block, token-in-block, kv head) for K and for V (null = the static
  // per-head k_scale / v_scale above)
  const float* ks_cache;
  const float* vs_cache;
  int64_t ks_st[3], vs_st[3];
  // device-planned splits (plan_table != null): every warp derives the common part length from seq_lens and finds
  // its own item, instead of numbering the items arithmetically from B, num_splits, Hkv; see plan_in_warp
  float* direct_part;   // planned + caller wants partial rows: where a single-part sequence's row goes ([B*Hq, row_floats])
  int2* plan_table;     // [B] {row0, used}: written by the warp of (part 0, head 0), read by the merge kernel
  int* plan_header;     // {items, part length in tiles, waves, 0}, written by item 0
  int plan_grid_items;  // item numbers the launch covers (>= the items of any plan it can choose)
  int plan_slots;       // resident warps of the kernel on the device
  int plan_k_max;       // most waves to aim for
  int plan_min_part;    // shortest part (tiles) the plan may choose when it aims for more than one wave
};

// Cross-GPU exchange of partial rows through peer-mapped buffers (sequence-parallel attention).  Every rank owns one
// buffer of the same layout, mapped into every other rank's address space:
//   [0, 256)    control words of the owner: {ticket of the last kernel of a step, epoch = steps completed}
//   [256, ...)  staging [rows, row_floats] fp32: rows that a kernel leaves for a separate push
//   then        2 slabs x [world, rows, row_floats] pairs {fp32 value, epoch}, used alternately (epoch parity):
//               slab[s][q] = rows of rank q
//   then        output slab [rows, out_floats] pairs (scatter form only): merged rows from their owners
constexpr int kMaxPeers = 16;
constexpr int kExchCtrlBytes = 256;
struct ExchangeParams {
  int world, rank;
  char* peer[kMaxPeers];  // base of every rank's buffer as mapped here; peer[rank] is the local buffer
  int64_t rows;           // B * Hq
  int row_floats;
  // Scatter form (many ranks, rows divisible by them): rank q owns rows [q, q + 1) * rows / world.  A push sends a row
  // to its owner only, the owner merges it and stores the merged fp32 row, again as pairs, into every rank's output
  // slab, from which every rank writes its `out`: 1/world of the bytes of sending every row to every rank.
  int scatter;
  int out_floats;         // floats of an output-slab row (head_dim rounded up to 4)
};
// Offset of the output slab: behind the control block, the staging rows and the two slabs of row pairs.
__host__ __device__ inline int64_t exch_out_off(int world, int64_t rows, int row_floats) {
  return kExchCtrlBytes + rows * row_floats * 4 + 2 * static_cast<int64_t>(world) * rows * row_floats * 8;
}

struct MergeParams {
  const float* parts;  // [R, rows, row_floats]
  int R;
  int64_t rows;  // B*Hq
  int Hq, D;
  int row_floats;
  void* out;  // final output (dtype/strides) when part_out is null
  int out_dtype;
  int64_t o_st[3];
  float* part_out;  // [rows, row_floats] merged partial rows (out | lse), or null
  const int2* seq_table;  // device-planned splits: parts of row (b, hq) are rows (row0 + c) * Hq + hq, c < used
  int early_trigger;  // call griddepcontrol.launch_dependents right after the dependency wait
  int inputs_ready;   // the call that produced the parts carried the inputs-ready promise: always trigger early
  // Rows that all ranks pushed into the local exchange buffer as (value, epoch) pairs (merge_exchanged_kernel only):
  // exchange_ctrl is the buffer's control block, `parts` points at slab 0 and slab_floats counts the pairs of a slab.
  const int* exchange_ctrl;
  int exchange_world;
  int64_t slab_floats;
  unsigned int* status;
};

// A merge carried by the NEXT layer's attention launch (chained layers), one warp per output row, `merge_warps`
// warps in all.  Two ways to seat those warps:
//  duty = 0  extra CTAs behind the attention items (from CTA `attn_ctas` on) that do nothing else;
//  duty = 1  the attention warps themselves, each as its last act (after it resolved the dependency for its own
//            writes), with no extra CTAs.
struct ChainedMerge {
  MergeParams m;    // m.rows == 0: nothing to merge
  int attn_ctas;
  int merge_warps;
  int duty;
};

int launch_cache_write(const WriteParams& p, int sm_count, cudaStream_t stream);
int launch_cache_write_dynamic(const DynWriteParams& p, cudaStream_t stream);
// `prev`: null, or the merge of the previous layer's partial rows to be carried by this launch (tiled kernels with
// static scales only; the caller has made sure of that).
int launch_attn_tiled_int8(const AttnParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, int sm_count,
                           cudaStream_t stream, const MergeParams* prev = nullptr);
int launch_attn_tiled_f16(const AttnParams& p, const CUtensorMap& tmK, const CUtensorMap& tmV, int sm_count,
                          cudaStream_t stream, const MergeParams* prev = nullptr);
int launch_attn_generic(const AttnParams& p, cudaStream_t stream);
int launch_merge(const MergeParams& p, cudaStream_t stream);
int launch_exchange_push(const ExchangeParams& e, cudaStream_t stream);
int launch_merge_exchanged(const MergeParams& p, const ExchangeParams& e, int phase, cudaStream_t stream);
// The merge of a rank's split-KV parts and the push of the merged rows in one kernel (head_dim % 4 == 0): p.part_out
// names the staging area of the local exchange buffer, where rows of sequences with a single part already lie; the
// merged rows go straight into every rank's slab.
int launch_merge_push(const MergeParams& p, const ExchangeParams& e, cudaStream_t stream);
int launch_bounded_wait_selftest(unsigned int* status, unsigned int attempts, cudaStream_t stream);

// resident warps per SM the tiled int8 kernel is sized for (used by the split heuristic)
constexpr int kTiledWarpsPerCta = 4;
constexpr int kMaxSplits = 128;

}  // namespace int8kv
