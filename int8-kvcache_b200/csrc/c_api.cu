// extern "C" entry points declared in include/int8kv_b200.h: argument validation, path selection
// (TMA-tiled kernels vs the generic kernel), tensor-map construction, split-KV planning and launches.
// Nothing here synchronises, allocates device memory or throws.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

using namespace int8kv;

namespace {

// ---- per-device facts, queried once -----------------------------------------------------------------
constexpr int kMaxDevices = 64;
std::atomic<int> g_sm_count[kMaxDevices];

int device_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = g_sm_count[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  g_sm_count[dev].store(n, std::memory_order_relaxed);
  return n;
}

// ---- cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda) -----------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// Tensor map over a cache [num_blocks, BS, Hkv, row_bytes] viewed in bytes as
// (byte-in-row, token-in-block, head, block) with a 128 B x 16 token box and the 128-byte swizzle.
bool make_cache_map(CUtensorMap* map, const void* base, int elem_bytes, int D, int Hkv, int64_t num_blocks,
                    int block_size, const int64_t st[4]) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (enc == nullptr) return false;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D) * elem_bytes, static_cast<cuuint64_t>(block_size),
                              static_cast<cuuint64_t>(Hkv), static_cast<cuuint64_t>(num_blocks)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(st[1]) * elem_bytes, static_cast<cuuint64_t>(st[2]) * elem_bytes,
                                 static_cast<cuuint64_t>(st[0]) * elem_bytes};
  const cuuint32_t box[4] = {128, 16, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool tma_friendly(const void* base, int elem_bytes, const int64_t st[4], int64_t num_blocks) {
  if (reinterpret_cast<uintptr_t>(base) & 15u) return false;
  if (st[3] != 1) return false;
  for (int i = 0; i < 3; ++i) {
    const int64_t bytes = st[i] * elem_bytes;
    if (bytes <= 0 || (bytes & 15) != 0 || bytes >= (int64_t(1) << 40)) return false;
  }
  return num_blocks > 0 && num_blocks < (int64_t(1) << 31);
}

bool valid_float_dtype(int d) { return d == INT8KV_BF16 || d == INT8KV_FP16 || d == INT8KV_FP32; }

int partial_row_floats(int D) { return ((D + 1) + 3) / 4 * 4; }

int64_t ws_bytes(int B, int Hq, int D, int S) {
  int64_t rows = S > 1 ? static_cast<int64_t>(S) * B * Hq * partial_row_floats(D) * 4 : 0;
  return rows + 16;  // trailing 16 bytes hold the status word
}

static int64_t pow2_floor(int64_t x) {
  int64_t p = 1;
  while (p * 2 <= x) p *= 2;
  return p;
}

// `chained`: the call is one layer of a chained sequence (run_layers), where consecutive layers overlap and what
// counts is the period of a layer, not the latency of one call.  A layer's merge is the one piece of a chained layer
// that cannot overlap the merge of the layer before it, and it costs one round trip to the L2 per 16 parts, so the
// latency-driven count is capped at 16 parts (measured on the 8 x 4096-token cell, per layer: 32 parts 11.1 us, of
// which the second round trip of the merge is about 2 us) and the rule that cuts the smallest calls into more,
// shorter parts is left out.
int choose_splits(int B, int Hkv, int64_t max_seq, int block_size, int sm_count, bool chained = false) {
  (void)block_size;
  if (B <= 0 || Hkv <= 0 || max_seq <= 0) return 1;
  const int64_t tiles = (max_seq + 15) / 16;
  const int64_t items = static_cast<int64_t>(B) * Hkv;
  // One warp serves one (sequence, kv head, split); 12 warps are resident per SM.  Two regimes, both measured on
  // B200, powers of two throughout:
  //  * small calls are bound by the latency chain of one warp, so the splits fill at most one resident wave of
  //    warps, down to 2 tiles per part for short sequences (16 parts) and 8 tiles per part for long ones;
  //  * large calls are bound by HBM, where ragged batches balance best with about four waves of warps, but a part
  //    of fewer than 32 tiles would spend too much of its traffic on its partial rows.
  const int64_t slots = static_cast<int64_t>(sm_count) * 12;
  const int64_t by_latency = chained ? std::min<int64_t>(tiles / 2, 16)
                                     : std::min<int64_t>(tiles / 2, std::max<int64_t>(16, tiles / 8));
  int64_t s_fill = std::min(pow2_floor(std::max<int64_t>(1, slots / items)), pow2_floor(std::max<int64_t>(1, by_latency)));
  // the smallest calls (512 warps or fewer in total) still gain from parts of only 4 tiles
  const int64_t s_quarter = std::min<int64_t>(pow2_floor(std::max<int64_t>(1, tiles / 4)), kMaxSplits);
  if (!chained && s_quarter > s_fill && items * s_quarter <= 512) s_fill = s_quarter;
  int64_t s_bw = 1;
  while (s_bw * items < slots * 4) s_bw *= 2;
  s_bw = std::min(s_bw, pow2_floor(std::max<int64_t>(1, tiles / 32)));
  int64_t s = std::max(s_fill, s_bw);
  if (s > kMaxSplits) s = kMaxSplits;
  if (s < 1) s = 1;
  return static_cast<int>(s);
}

// Split count for the kernels outside the tiled shapes.  They hide their load latency with resident warps, not
// with a ring, and every part pays a prologue (query staging) and a partial row.
//  - grouped INT8 kernel: the best count fills ONE resident wave, as many one-warp items as the SMs hold at the
//    kernel's register cap (16 warps per SM for groups up to 4, 12 up to 8, 8 up to 16).  Measured on a head_dim-64
//    layer of 64 x 2048 tokens with 8 KV heads (512 items): 2 parts 174 us, 4 parts (2048 warps, one wave) 98 us,
//    8 parts 104 us, 16 parts 116 us, 32 parts 128 us.
//  - generic kernel: one item per query head, fewer registers and more waiting per instruction, so it keeps about
//    32 warps per SM (head_dim 66, 512 items: 2 parts 813 us, 4 parts 544 us, 8 parts 456 us).
// Parts stay at least 8 blocks of 16 tokens long.
int untiled_splits(int B, int Hq, int Hkv, int D, bool int8_cache, int64_t max_seq, int sm_count) {
  const int G = Hq / std::max(1, Hkv);
  const bool grouped = int8_cache && D % 4 == 0 && D <= 256 && G <= 16 && !(G > 8 && D > 128);
  const int64_t items = std::max<int64_t>(1, static_cast<int64_t>(B) * (grouped ? Hkv : Hq));
  const int per_sm = !grouped ? 32 : (G <= 4 ? 16 : (G <= 8 ? 12 : 8));
  const int64_t tiles = (max_seq + 15) / 16;
  int64_t s = static_cast<int64_t>(sm_count) * per_sm / items;
  s = std::min<int64_t>(s, std::max<int64_t>(1, tiles / 8));
  return static_cast<int>(std::min<int64_t>(std::max<int64_t>(s, 1), kMaxSplits));
}

// ---- device-planned splits ----------------------------------------------------------------------------
// Large calls (HBM-bound, up to a few resident waves of warps) choose the part length on the device from the
// actual sequence lengths, so that the parts fill whole waves; see plan_in_warp.  INT8KV_PLAN=0 turns it off.
struct PlanShape {
  int k_max;       // most waves the plan may aim for
  int max_items;   // capacity of the item list = item numbers the attention launch covers
  int min_part;
};

int env_int_or(const char* name, int fallback) {
  const char* e = std::getenv(name);
  return e ? std::atoi(e) : fallback;
}

// Whether the shape can be planned at all: every warp walks seq_lens a few times, which stays cheap up to a few
// hundred sequences, and one part per (sequence, head) must fit one wave.
constexpr int kPlanMaxBatch = 512;
bool plan_possible(int B, int Hkv, int sm_count) {
  return B <= kPlanMaxBatch && static_cast<int64_t>(B) * Hkv <= static_cast<int64_t>(sm_count) * 12;
}

// Whether planning pays: enough nominal work for one wave of parts of at least 12 tiles, and a split
// heuristic that could not reach four waves of warps for this shape (with four or more waves the tail is small and
// the plan's longer prologue, every warp reading seq_lens before its block table, costs more than it gains:
// measured 222 us against 216 us per call on the 256-sequence ragged batch).
bool plan_pays(int B, int Hkv, int64_t max_seq, int block_size, int sm_count) {
  static const int enabled = env_int_or("INT8KV_PLAN", 1);
  if (!enabled || !plan_possible(B, Hkv, sm_count)) return false;
  const int64_t slots = static_cast<int64_t>(sm_count) * 12;
  const int64_t items = static_cast<int64_t>(B) * Hkv;
  const int64_t tiles = (max_seq + 15) / 16;
  if (items * tiles < slots * 12) return false;
  return items * choose_splits(B, Hkv, max_seq, block_size, sm_count) < slots * 4;
}

// Warps per SM that a plan counts as one wave.  A single call fills the machine exactly (12 resident warps per SM).
// A layer of a chained sequence aims for two thirds of that: with every slot taken by one layer, the next layer's
// warps can only enter as these leave, and each layer pays its prologue and epilogue with idle memory pipes; at 8 per
// SM two layers interleave.  Measured per layer, chained, 12 -> 8 warps per SM: one KV head x 128 ragged sequences
// (the 8-GPU shard of the 256-sequence batch) 29.7 -> 25.4 us (0.83 -> 0.97 of the HBM peak), 64 ragged sequences x 4
// heads 50.1 -> 48.3 us, 16 sequences 17.5 -> 15.1 us; 6 per SM gains nothing more on the small ones and loses on
// the large ones (53 us), 10 sits between.
constexpr int kPlanWaveSingle = 12, kPlanWaveChained = 8;

PlanShape plan_shape(int B, int Hkv, int64_t tiles, int sm_count, int wave_warps = kPlanWaveSingle) {
  constexpr int min_part = 48;  // shortest part (16-token tiles) a plan aiming for more than one wave may choose
  const int64_t slots = static_cast<int64_t>(sm_count) * wave_warps;
  const int64_t items = static_cast<int64_t>(B) * Hkv;
  PlanShape s{1, 0, min_part};
  // the same rule the plan kernel applies, on the nominal lengths: the actual k can only be smaller
  for (int k = 4; k >= 1; --k) {
    const int64_t room = k * slots - items / 2;
    if (room <= 0) continue;
    const int64_t P = (items * tiles + room - 1) / room;
    if (P >= min_part || k == 1) {
      s.k_max = k;
      break;
    }
  }
  s.max_items = static_cast<int>(std::max<int64_t>(s.k_max * slots, items));
  return s;
}

// Workspace of a planned call: partial rows (one per item and query head of its group), the sequence table,
// then header and status word at the end.
struct PlanLayout {
  int64_t table_off, header_off, total;
};
PlanLayout plan_layout(int B, int Hq, int Hkv, int D, int max_items) {
  const int G = Hq / Hkv;
  PlanLayout l;
  const int64_t rows = static_cast<int64_t>(max_items) * G * partial_row_floats(D) * 4;
  l.table_off = (rows + 15) & ~int64_t(15);
  l.header_off = (l.table_off + static_cast<int64_t>(B) * 8 + 15) & ~int64_t(15);  // earliest place for the header
  l.total = l.header_off + 16 + 16;
  return l;
}

struct AttnCall {
  const void* query; int q_dtype; const int64_t* q_st;
  int B, Hq, Hkv, D;
  const void* kc; const void* vc; int cache_kind; const int64_t* kc_st; const int64_t* vc_st;
  int64_t num_blocks; int block_size;
  const void* bt; int bt_is_i64; const int64_t* bt_st; int64_t bt_width;
  const void* sl; int sl_is_i64; int64_t max_seq_hint;
  const float* k_scale; const float* v_scale;
  void* out; int out_dtype; const int64_t* o_st;
  float* partial_out;  // non-null: emit merged partial rows instead of `out`
  int num_splits; void* ws; int64_t ws_bytes;
  int flags; cudaStream_t stream;  // INT8KV_FLAG_* bits
  // fused decode step (null new_k = plain attention)
  const void* new_k = nullptr; const void* new_v = nullptr; int new_dtype = 0;
  const int64_t* nk_st = nullptr; const int64_t* nv_st = nullptr;
  const void* new_slots = nullptr; int new_slot_is_i64 = 0;
  // dynamic per-(token, head) scales (null ks_cache = static scales)
  const float* ks_cache = nullptr; const float* vs_cache = nullptr;
  const int64_t* ks_st = nullptr; const int64_t* vs_st = nullptr;
  // device status word to use instead of the one at the end of `ws` (a call that works in a part of a larger workspace)
  unsigned int* status = nullptr;
  bool chained = false;  // one layer of a chained sequence: the automatic split count favours throughput
  // partial rows that go to the other ranks: when the call needs a merge, that merge stores its rows into every
  // rank's exchange buffer itself and sets *pushed; otherwise the rows lie in partial_out and the caller pushes them
  const ExchangeParams* push = nullptr;
  bool* pushed = nullptr;
};

// What a call will do, decided from its arguments alone (no launch, no device access beyond the SM count).
struct AttnPlan {
  int G, sm, S, rf, esz;
  int64_t max_seq, tiles, need;
  bool tiled, planned, dyn;
  int quantize_q;
  PlanShape ps;
  PlanLayout pl;
};

int plan_attention(const AttnCall& a, AttnPlan& t) {
  if (a.B < 0 || a.Hq <= 0 || a.Hkv <= 0 || a.D <= 0 || a.block_size <= 0 || a.num_blocks < 0 || a.bt_width < 0)
    return INT8KV_E_BAD_SHAPE;
  if (a.Hq % a.Hkv != 0) return INT8KV_E_BAD_SHAPE;
  if (a.num_splits < INT8KV_SPLITS_PLANNED || a.num_splits > kMaxSplits) return INT8KV_E_BAD_SHAPE;
  if (a.flags & ~(INT8KV_FLAG_QUANTIZE_Q | INT8KV_FLAG_INPUTS_READY)) return INT8KV_E_BAD_SHAPE;
  t.quantize_q = (a.flags & INT8KV_FLAG_QUANTIZE_Q) ? 1 : 0;
  if (t.quantize_q && (a.cache_kind != kCacheInt8 || a.ks_cache != nullptr || a.new_k != nullptr)) return INT8KV_E_UNSUPPORTED;
  if (!valid_float_dtype(a.q_dtype)) return INT8KV_E_BAD_DTYPE;
  if (a.partial_out == nullptr && !valid_float_dtype(a.out_dtype)) return INT8KV_E_BAD_DTYPE;
  if (a.B == 0) return INT8KV_OK;
  if (!a.query || !a.kc || !a.vc || !a.bt || !a.sl || !a.q_st || !a.kc_st || !a.vc_st || !a.bt_st)
    return INT8KV_E_NULLPTR;
  if (a.partial_out == nullptr && (!a.out || !a.o_st)) return INT8KV_E_NULLPTR;
  t.dyn = a.ks_cache != nullptr || a.vs_cache != nullptr;
  if (t.dyn && (!a.ks_cache || !a.vs_cache || !a.ks_st || !a.vs_st)) return INT8KV_E_NULLPTR;
  if (t.dyn && (a.cache_kind != kCacheInt8 || a.new_k != nullptr)) return INT8KV_E_UNSUPPORTED;
  if (a.cache_kind == kCacheInt8 && !t.dyn && (!a.k_scale || !a.v_scale)) return INT8KV_E_NULLPTR;
  if (a.kc_st[3] != 1 || a.vc_st[3] != 1) return INT8KV_E_UNSUPPORTED;  // the reference asserts unit last stride too

  t.G = a.Hq / a.Hkv;
  t.sm = device_sm_count();
  t.max_seq = a.max_seq_hint > 0 ? a.max_seq_hint : a.bt_width * a.block_size;
  if (t.max_seq > a.bt_width * a.block_size) t.max_seq = a.bt_width * a.block_size;
  t.S = a.num_splits > 0 ? a.num_splits : choose_splits(a.B, a.Hkv, t.max_seq, a.block_size, t.sm, a.chained);
  // more splits than 16-token tiles only produces empty parts
  t.tiles = (t.max_seq + 15) / 16;
  if (t.S > t.tiles) t.S = t.tiles > 0 ? static_cast<int>(t.tiles) : 1;

  t.rf = partial_row_floats(a.D);
  t.esz = a.cache_kind == kCacheInt8 ? 1 : 2;
  t.tiled = a.D == 128 && (a.block_size % 16) == 0 && t.G <= 8 && a.num_blocks > 0 &&
            tma_friendly(a.kc, t.esz, a.kc_st, a.num_blocks) && tma_friendly(a.vc, t.esz, a.vc_st, a.num_blocks) &&
            (t.rf % 4 == 0);
  if (!t.tiled && a.num_splits == 0) {
    // the automatic count above is fitted to the tiled kernels; use the untiled one if the workspace allows it
    int su = untiled_splits(a.B, a.Hq, a.Hkv, a.D, a.cache_kind == kCacheInt8, t.max_seq, t.sm);
    if (su > t.tiles) su = t.tiles > 0 ? static_cast<int>(t.tiles) : 1;
    if (su <= 1 || (a.ws != nullptr && a.ws_bytes >= ws_bytes(a.B, a.Hq, a.D, su))) t.S = su;
  }
  // Device-planned splits: asked for explicitly, or chosen for a large automatic call when the workspace has
  // room for the plan (callers that sized it with int8kv_workspace_bytes_auto always have).
  t.planned = false;
  if (a.num_splits <= 0 && t.tiled && t.tiles > 0 &&
      a.bt_width * a.block_size < (int64_t(1) << 21) * 16 &&  // tile counts stay exact in fp32 on the device
      (a.num_splits == INT8KV_SPLITS_PLANNED ? plan_possible(a.B, a.Hkv, t.sm)
                                              : plan_pays(a.B, a.Hkv, t.max_seq, a.block_size, t.sm))) {
    t.ps = plan_shape(a.B, a.Hkv, t.tiles, t.sm, a.chained ? kPlanWaveChained : kPlanWaveSingle);
    t.pl = plan_layout(a.B, a.Hq, a.Hkv, a.D, t.ps.max_items);
    // the plan's header sits in the 16 bytes before the status word, wherever the workspace ends
    t.planned = a.ws != nullptr && a.ws_bytes >= t.pl.total && (reinterpret_cast<uintptr_t>(a.ws) & 15u) == 0 &&
                t.pl.header_off + 16 <= int8kv_workspace_status_offset(a.ws_bytes);
    if (t.planned) t.pl.header_off = int8kv_workspace_status_offset(a.ws_bytes) - 16;
    if (!t.planned && a.num_splits == INT8KV_SPLITS_PLANNED) return INT8KV_E_WORKSPACE;
  } else if (a.num_splits == INT8KV_SPLITS_PLANNED) {
    return INT8KV_E_UNSUPPORTED;
  }
  if (t.planned) t.S = kMaxSplits;  // upper bound of the parts of one sequence; the real count is in the plan
  t.need = t.planned ? t.pl.total : ws_bytes(a.B, a.Hq, a.D, t.S);
  if (t.S > 1) {
    if (a.ws == nullptr || a.ws_bytes < t.need) return INT8KV_E_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(a.ws) & 15u) return INT8KV_E_WORKSPACE;
  }
  if (a.new_k != nullptr && !(t.tiled && a.cache_kind == kCacheInt8)) return INT8KV_E_UNSUPPORTED;
  if (!t.tiled && a.cache_kind != kCacheInt8 && t.quantize_q) return INT8KV_E_UNSUPPORTED;
  return INT8KV_OK;
}

// A sequence of layer calls whose split-KV merges ride on the NEXT layer's attention launch (chained layers): the
// merge of layer l runs in extra CTAs of layer l+1's launch, beside that layer's page stream, instead of in a launch
// of its own between the two.  Possible when the caller promised that the layers are independent (the outputs of
// layer l are not inputs of layer l+1) and every layer has its own half of the workspace.
struct Chain {
  bool active = false;    // merges may be deferred to the next launch
  bool pending = false;   // `merge` has not been launched or carried yet
  MergeParams merge;
};

int flush_chain(Chain* chain, cudaStream_t stream) {
  if (chain == nullptr || !chain->pending) return INT8KV_OK;
  chain->pending = false;
  return launch_merge(chain->merge, stream);
}

int run_attention(const AttnCall& a, Chain* chain = nullptr) {
  AttnPlan t;
  std::memset(&t, 0, sizeof(t));
  const int checked = plan_attention(a, t);
  if (checked != INT8KV_OK || a.B == 0) return checked;
  const int G = t.G, sm = t.sm, S = t.S, rf = t.rf, esz = t.esz;
  const int64_t tiles = t.tiles;
  const bool tiled = t.tiled, planned = t.planned, dyn = t.dyn;
  const PlanShape& ps = t.ps;
  const PlanLayout& pl = t.pl;
  unsigned int* status = a.status;
  if (status == nullptr && a.ws != nullptr && a.ws_bytes >= 16)
    status = reinterpret_cast<unsigned int*>(static_cast<char*>(a.ws) + int8kv_workspace_status_offset(a.ws_bytes));

  AttnParams p;
  std::memset(&p, 0, sizeof(p));
  p.q = a.query; p.q_dtype = a.q_dtype;
  for (int i = 0; i < 3; ++i) p.q_st[i] = a.q_st[i];
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = G; p.D = a.D;
  p.kc = a.kc; p.vc = a.vc; p.cache_kind = a.cache_kind;
  for (int i = 0; i < 4; ++i) { p.kc_st[i] = a.kc_st[i]; p.vc_st[i] = a.vc_st[i]; }
  p.num_blocks = a.num_blocks; p.block_size = a.block_size;
  p.tiles_per_block = a.block_size / 16;
  p.hint_tiles = static_cast<int>(tiles);
  p.bt = a.bt; p.bt_is_i64 = a.bt_is_i64; p.bt_st[0] = a.bt_st[0]; p.bt_st[1] = a.bt_st[1]; p.bt_width = a.bt_width;
  p.sl = a.sl; p.sl_is_i64 = a.sl_is_i64;
  p.k_scale = a.k_scale; p.v_scale = a.v_scale;
  p.out = a.out; p.out_dtype = a.out_dtype;
  if (a.o_st) for (int i = 0; i < 3; ++i) p.o_st[i] = a.o_st[i];
  p.num_splits = S;
  p.per_longest = static_cast<int>(std::max<int64_t>(1, (tiles + S - 1) / S));
  p.row_floats = rf;
  p.quantize_q = t.quantize_q;
  p.defer_wait = (a.flags & INT8KV_FLAG_INPUTS_READY) ? 1 : 0;
  p.sm_scale_log2 = static_cast<float>(1.4426950408889634 / std::sqrt(static_cast<double>(a.D)));
  p.status = status;
  if (S > 1) p.part = reinterpret_cast<float*>(a.ws);
  else p.part = a.partial_out;  // null for the ordinary call: write `out` directly

  if (dyn) {
    p.ks_cache = a.ks_cache; p.vs_cache = a.vs_cache;
    for (int i = 0; i < 3; ++i) { p.ks_st[i] = a.ks_st[i]; p.vs_st[i] = a.vs_st[i]; }
  }
  if (a.new_k != nullptr) {
    p.new_k = a.new_k; p.new_v = a.new_v; p.new_dtype = a.new_dtype;
    for (int i = 0; i < 3; ++i) { p.nk_st[i] = a.nk_st[i]; p.nv_st[i] = a.nv_st[i]; }
    p.new_slots = a.new_slots; p.new_slot_is_i64 = a.new_slot_is_i64;
  }
  int rc;
  if (planned) {
    char* base = static_cast<char*>(a.ws);
    p.plan_table = reinterpret_cast<int2*>(base + pl.table_off);
    p.plan_header = reinterpret_cast<int*>(base + pl.header_off);
    p.plan_grid_items = ps.max_items;
    p.plan_slots = sm * (a.chained ? kPlanWaveChained : kPlanWaveSingle);
    p.plan_k_max = ps.k_max;
    p.plan_min_part = ps.min_part;
    p.direct_part = a.partial_out;
  }
  // A merge left over from the previous layer rides on this launch when this launch can carry it (tiled kernels,
  // static scales, plain query); otherwise it gets its own launch first.
  const bool carry = chain != nullptr && chain->pending && tiled && !dyn && !t.quantize_q;
  if (chain != nullptr && chain->pending && !carry) {
    rc = flush_chain(chain, a.stream);
    if (rc != INT8KV_OK) return rc;
  }
  if (tiled) {
    alignas(64) CUtensorMap tmK, tmV;
    if (!make_cache_map(&tmK, a.kc, esz, a.D, a.Hkv, a.num_blocks, a.block_size, a.kc_st) ||
        !make_cache_map(&tmV, a.vc, esz, a.D, a.Hkv, a.num_blocks, a.block_size, a.vc_st))
      return INT8KV_E_LAUNCH;
    const MergeParams* prev = carry ? &chain->merge : nullptr;
    rc = a.cache_kind == kCacheInt8 ? launch_attn_tiled_int8(p, tmK, tmV, sm, a.stream, prev)
                                    : launch_attn_tiled_f16(p, tmK, tmV, sm, a.stream, prev);
    if (carry && rc == INT8KV_OK) chain->pending = false;
  } else {
    rc = launch_attn_generic(p, a.stream);
  }
  if (rc != INT8KV_OK || S == 1) return rc;

  MergeParams m;
  std::memset(&m, 0, sizeof(m));
  m.parts = p.part; m.R = S; m.rows = static_cast<int64_t>(a.B) * a.Hq; m.Hq = a.Hq; m.D = a.D; m.row_floats = rf;
  m.out = a.out; m.out_dtype = a.out_dtype;
  if (a.o_st) for (int i = 0; i < 3; ++i) m.o_st[i] = a.o_st[i];
  m.part_out = a.partial_out;
  m.inputs_ready = p.defer_wait;
  if (planned) m.seq_table = reinterpret_cast<const int2*>(static_cast<char*>(a.ws) + pl.table_off);
  if (chain != nullptr && chain->active && tiled && a.partial_out == nullptr) {
    chain->merge = m;  // the next layer's launch carries it (or flush_chain launches it)
    chain->pending = true;
    return INT8KV_OK;
  }
  if (a.push != nullptr && a.partial_out != nullptr && a.D % 4 == 0) {
    rc = launch_merge_push(m, *a.push, a.stream);
    if (rc == INT8KV_OK && a.pushed != nullptr) *a.pushed = true;
    return rc;
  }
  return launch_merge(m, a.stream);
}

}  // namespace

extern "C" {

int int8kv_abi_version(void) { return INT8KV_ABI_VERSION; }

const char* int8kv_status_str(int status) {
  switch (status) {
    case INT8KV_OK: return "ok";
    case INT8KV_E_NULLPTR: return "null pointer argument";
    case INT8KV_E_BAD_SHAPE: return "inconsistent shape or stride";
    case INT8KV_E_BAD_DTYPE: return "unknown dtype code";
    case INT8KV_E_UNSUPPORTED: return "unsupported configuration";
    case INT8KV_E_LAUNCH: return "CUDA launch or set-up error";
    case INT8KV_E_WORKSPACE: return "split-KV workspace missing, misaligned or too small";
    default: return "unknown status";
  }
}

int int8kv_partial_row_floats(int head_dim) { return partial_row_floats(head_dim); }

int64_t int8kv_workspace_bytes(int batch, int num_q_heads, int head_dim, int num_splits) {
  if (batch < 0 || num_q_heads <= 0 || head_dim <= 0 || num_splits < 0) return -1;
  return ws_bytes(batch, num_q_heads, head_dim, num_splits);
}

int64_t int8kv_workspace_bytes_auto(int batch, int num_q_heads, int num_kv_heads, int head_dim, int64_t max_seq_len,
                                    int block_size, int sm_count) {
  if (batch < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || max_seq_len < 0 ||
      num_q_heads % num_kv_heads != 0)
    return -1;
  const int sm = sm_count > 0 ? sm_count : 148;
  const int64_t tiles = (max_seq_len + 15) / 16;
  int64_t n = ws_bytes(batch, num_q_heads, head_dim, choose_splits(batch, num_kv_heads, max_seq_len, block_size, sm));
  // a shape for the untiled kernels, which have their own split rule
  if (head_dim != 128 || block_size % 16 != 0 || num_q_heads / num_kv_heads > 8)
    for (const bool int8_cache : {true, false})
      n = std::max(n, ws_bytes(batch, num_q_heads, head_dim,
                               untiled_splits(batch, num_q_heads, num_kv_heads, head_dim, int8_cache, max_seq_len, sm)));
  if (batch > 0 && tiles > 0 && plan_possible(batch, num_kv_heads, sm)) {
    for (const int wave : {kPlanWaveSingle, kPlanWaveChained}) {  // a chained layer may plan more, shorter waves
      const PlanShape ps = plan_shape(batch, num_kv_heads, tiles, sm, wave);
      n = std::max(n, plan_layout(batch, num_q_heads, num_kv_heads, head_dim, ps.max_items).total);
    }
  }
  return n;
}

int64_t int8kv_workspace_status_offset(int64_t workspace_bytes) {
  return workspace_bytes >= 16 ? ((workspace_bytes - 16) & ~int64_t(15)) : 0;
}

int int8kv_choose_splits(int batch, int num_kv_heads, int64_t max_seq_len, int block_size, int sm_count) {
  return choose_splits(batch, num_kv_heads, max_seq_len, block_size, sm_count > 0 ? sm_count : 148);
}

int int8kv_max_splits(void) { return kMaxSplits; }

int int8kv_cache_write(const void* key, const void* value, int in_dtype, int64_t num_tokens, int num_kv_heads,
                       int head_dim, const int64_t key_strides[3], const int64_t value_strides[3],
                       int8_t* key_cache, int8_t* value_cache, const int64_t key_cache_strides[4],
                       const int64_t value_cache_strides[4], int64_t num_blocks, int block_size,
                       const void* slot_mapping, int slot_is_i64, const float* k_scale, const float* v_scale,
                       void* stream) {
  if (num_tokens < 0 || num_kv_heads <= 0 || head_dim <= 0 || num_blocks < 0 || block_size <= 0)
    return INT8KV_E_BAD_SHAPE;
  if (!valid_float_dtype(in_dtype)) return INT8KV_E_BAD_DTYPE;
  if (num_tokens == 0) return INT8KV_OK;
  if (!key || !value || !key_cache || !value_cache || !slot_mapping || !k_scale || !v_scale || !key_strides ||
      !value_strides || !key_cache_strides || !value_cache_strides)
    return INT8KV_E_NULLPTR;
  WriteParams p;
  std::memset(&p, 0, sizeof(p));
  p.key = key; p.value = value; p.in_dtype = in_dtype;
  p.T = num_tokens; p.Hkv = num_kv_heads; p.D = head_dim;
  for (int i = 0; i < 3; ++i) { p.k_st[i] = key_strides[i]; p.v_st[i] = value_strides[i]; }
  p.kc = key_cache; p.vc = value_cache;
  for (int i = 0; i < 4; ++i) { p.kc_st[i] = key_cache_strides[i]; p.vc_st[i] = value_cache_strides[i]; }
  p.num_slots = num_blocks * block_size;
  p.block_size = block_size;
  p.slots = slot_mapping; p.slot_is_i64 = slot_is_i64;
  p.k_scale = k_scale; p.v_scale = v_scale;
  return launch_cache_write(p, device_sm_count(), static_cast<cudaStream_t>(stream));
}

int int8kv_paged_attn_int8(const void* query, int q_dtype, const int64_t q_strides[3], int batch, int num_q_heads,
                           int num_kv_heads, int head_dim, const int8_t* key_cache, const int8_t* value_cache,
                           const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                           int64_t num_blocks, int block_size, const void* block_tables, int bt_is_i64,
                           const int64_t bt_strides[2], int64_t bt_width, const void* seq_lens, int sl_is_i64,
                           int64_t max_seq_len_hint, const float* k_scale, const float* v_scale, void* out,
                           int out_dtype, const int64_t out_strides[3], int num_splits, void* workspace,
                           int64_t workspace_bytes, int flags, void* stream) {
  AttnCall a{query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
             key_cache, value_cache, kCacheInt8, key_cache_strides, value_cache_strides, num_blocks, block_size,
             block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
             k_scale, v_scale, out, out_dtype, out_strides, nullptr,
             num_splits, workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream)};
  return run_attention(a);
}

int int8kv_paged_attn_bf16(const void* query, int q_dtype, const int64_t q_strides[3], int batch, int num_q_heads,
                           int num_kv_heads, int head_dim, const void* key_cache, const void* value_cache,
                           int cache_dtype, const int64_t key_cache_strides[4],
                           const int64_t value_cache_strides[4], int64_t num_blocks, int block_size,
                           const void* block_tables, int bt_is_i64, const int64_t bt_strides[2], int64_t bt_width,
                           const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint, void* out, int out_dtype,
                           const int64_t out_strides[3], int num_splits, void* workspace, int64_t workspace_bytes,
                           int flags, void* stream) {
  if (cache_dtype != INT8KV_BF16 && cache_dtype != INT8KV_FP16) return INT8KV_E_BAD_DTYPE;
  AttnCall a{query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
             key_cache, value_cache, cache_dtype == INT8KV_BF16 ? kCacheBf16 : kCacheFp16,
             key_cache_strides, value_cache_strides, num_blocks, block_size,
             block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
             nullptr, nullptr, out, out_dtype, out_strides, nullptr,
             num_splits, workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream)};
  return run_attention(a);
}

int int8kv_paged_attn_int8_partial(const void* query, int q_dtype, const int64_t q_strides[3], int batch,
                                   int num_q_heads, int num_kv_heads, int head_dim, const int8_t* key_cache,
                                   const int8_t* value_cache, const int64_t key_cache_strides[4],
                                   const int64_t value_cache_strides[4], int64_t num_blocks, int block_size,
                                   const void* block_tables, int bt_is_i64, const int64_t bt_strides[2],
                                   int64_t bt_width, const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                                   const float* k_scale, const float* v_scale, float* partial, int num_splits,
                                   void* workspace, int64_t workspace_bytes, int flags, void* stream) {
  if (partial == nullptr) return INT8KV_E_NULLPTR;
  if (reinterpret_cast<uintptr_t>(partial) & 15u) return INT8KV_E_BAD_SHAPE;
  AttnCall a{query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
             key_cache, value_cache, kCacheInt8, key_cache_strides, value_cache_strides, num_blocks, block_size,
             block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
             k_scale, v_scale, nullptr, INT8KV_FP32, nullptr, partial,
             num_splits, workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream)};
  return run_attention(a);
}

int int8kv_paged_attn_int8_dynamic(const void* query, int q_dtype, const int64_t q_strides[3], int batch,
                                   int num_q_heads, int num_kv_heads, int head_dim, const int8_t* key_cache,
                                   const int8_t* value_cache, const int64_t key_cache_strides[4],
                                   const int64_t value_cache_strides[4], const float* k_scale_cache,
                                   const float* v_scale_cache, const int64_t k_scale_strides[3],
                                   const int64_t v_scale_strides[3], int64_t num_blocks, int block_size,
                                   const void* block_tables, int bt_is_i64, const int64_t bt_strides[2],
                                   int64_t bt_width, const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                                   void* out, int out_dtype, const int64_t out_strides[3], int num_splits,
                                   void* workspace, int64_t workspace_bytes, int flags, void* stream) {
  if (batch > 0 && (!k_scale_cache || !v_scale_cache || !k_scale_strides || !v_scale_strides)) return INT8KV_E_NULLPTR;
  AttnCall a{query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
             key_cache, value_cache, kCacheInt8, key_cache_strides, value_cache_strides, num_blocks, block_size,
             block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
             nullptr, nullptr, out, out_dtype, out_strides, nullptr,
             num_splits, workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream)};
  a.ks_cache = k_scale_cache; a.vs_cache = v_scale_cache; a.ks_st = k_scale_strides; a.vs_st = v_scale_strides;
  return run_attention(a);
}

int int8kv_merge_partials(const float* parts, int num_parts, int batch, int num_q_heads, int head_dim, void* out,
                          int out_dtype, const int64_t out_strides[3], void* stream) {
  if (num_parts <= 0 || num_parts > kMaxSplits || batch < 0 || num_q_heads <= 0 || head_dim <= 0)
    return INT8KV_E_BAD_SHAPE;
  if (!valid_float_dtype(out_dtype)) return INT8KV_E_BAD_DTYPE;
  if (batch == 0) return INT8KV_OK;
  if (!parts || !out || !out_strides) return INT8KV_E_NULLPTR;
  if (reinterpret_cast<uintptr_t>(parts) & 15u) return INT8KV_E_BAD_SHAPE;
  MergeParams m;
  std::memset(&m, 0, sizeof(m));
  m.parts = parts; m.R = num_parts; m.rows = static_cast<int64_t>(batch) * num_q_heads; m.Hq = num_q_heads;
  m.D = head_dim; m.row_floats = partial_row_floats(head_dim);
  m.out = out; m.out_dtype = out_dtype;
  for (int i = 0; i < 3; ++i) m.o_st[i] = out_strides[i];
  m.part_out = nullptr;
  return launch_merge(m, static_cast<cudaStream_t>(stream));
}

int64_t int8kv_exchange_bytes(int world, int batch, int num_q_heads, int head_dim) {
  if (world <= 0 || world > kMaxPeers || batch < 0 || num_q_heads <= 0 || head_dim <= 0) return -1;
  // control block | staging rows (fp32) | 2 slabs x world ranks x rows of (value, epoch) pairs | output slab of pairs
  const int64_t rows = static_cast<int64_t>(batch) * num_q_heads;
  return exch_out_off(world, rows, partial_row_floats(head_dim)) + rows * ((head_dim + 3) / 4 * 4) * 8;
}

// Ranks from which the exchange scatters rows to owners instead of sending every row to every rank.  Measured per
// step on B200s (32 sequences x 65536 tokens, 64 query heads), all-to-all against scatter: 2 ranks 359.8 / 361.1 us
// (the second phase costs more than the halved bytes save), 4 ranks 206.7 / 203.4 us, 8 ranks 137.1 / 112.7 us.
constexpr int kScatterMinWorld = 4;

static int exchange_params(const int8kv_exchange* ex, int batch, int num_q_heads, int head_dim, ExchangeParams* e) {
  if (ex == nullptr) return INT8KV_E_NULLPTR;
  if (ex->world <= 0 || ex->world > kMaxPeers || ex->rank < 0 || ex->rank >= ex->world) return INT8KV_E_BAD_SHAPE;
  if (ex->buffer_bytes < int8kv_exchange_bytes(ex->world, batch, num_q_heads, head_dim)) return INT8KV_E_WORKSPACE;
  std::memset(e, 0, sizeof(*e));
  e->world = ex->world;
  e->rank = ex->rank;
  for (int r = 0; r < ex->world; ++r) {
    if (ex->peer_buffers[r] == nullptr) return INT8KV_E_NULLPTR;
    if (reinterpret_cast<uintptr_t>(ex->peer_buffers[r]) & 255u) return INT8KV_E_WORKSPACE;
    e->peer[r] = static_cast<char*>(ex->peer_buffers[r]);
  }
  e->rows = static_cast<int64_t>(batch) * num_q_heads;
  e->row_floats = partial_row_floats(head_dim);
  e->out_floats = (head_dim + 3) / 4 * 4;
  // many ranks: a row goes to one owner, the owner sends the merged row to everyone (on eight GPUs the 15 MB of pairs
  // that a rank sends per step become 3.7 MB)
  e->scatter = ex->world >= kScatterMinWorld && e->rows % ex->world == 0 && e->rows > 0;
  return INT8KV_OK;
}

int int8kv_paged_attn_int8_partial_push(const void* query, int q_dtype, const int64_t q_strides[3], int batch,
                                        int num_q_heads, int num_kv_heads, int head_dim, const int8_t* key_cache,
                                        const int8_t* value_cache, const int64_t key_cache_strides[4],
                                        const int64_t value_cache_strides[4], int64_t num_blocks, int block_size,
                                        const void* block_tables, int bt_is_i64, const int64_t bt_strides[2],
                                        int64_t bt_width, const void* seq_lens, int sl_is_i64,
                                        int64_t max_seq_len_hint, const float* k_scale, const float* v_scale,
                                        const int8kv_exchange* exchange, int num_splits, void* workspace,
                                        int64_t workspace_bytes, int flags, void* stream) {
  if (batch < 0 || num_q_heads <= 0 || head_dim <= 0) return INT8KV_E_BAD_SHAPE;
  ExchangeParams e;
  int rc = exchange_params(exchange, batch, num_q_heads, head_dim, &e);
  if (rc != INT8KV_OK) return rc;
  if (batch == 0) return INT8KV_OK;
  float* staging = reinterpret_cast<float*>(e.peer[e.rank] + kExchCtrlBytes);
  AttnCall a{query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
             key_cache, value_cache, kCacheInt8, key_cache_strides, value_cache_strides, num_blocks, block_size,
             block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
             k_scale, v_scale, nullptr, INT8KV_FP32, nullptr, staging,
             num_splits, workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream)};
  bool pushed = false;
  a.push = &e;  // measured on two GPUs, 32 sequences of 65536 tokens: 359 us per step against 366 us with a push launch of its own
  a.pushed = &pushed;
  rc = run_attention(a);
  if (rc != INT8KV_OK || pushed) return rc;
  return launch_exchange_push(e, static_cast<cudaStream_t>(stream));  // an unsplit call: its rows lie in the staging area
}

int int8kv_merge_exchanged(const int8kv_exchange* exchange, int batch, int num_q_heads, int head_dim, void* out,
                           int out_dtype, const int64_t out_strides[3], void* workspace, int64_t workspace_bytes,
                           void* stream) {
  return int8kv_merge_exchanged_phase(exchange, batch, num_q_heads, head_dim, out, out_dtype, out_strides, workspace,
                                      workspace_bytes, INT8KV_EXCHANGE_BOTH_PHASES, stream);
}

int int8kv_merge_exchanged_phase(const int8kv_exchange* exchange, int batch, int num_q_heads, int head_dim, void* out,
                                 int out_dtype, const int64_t out_strides[3], void* workspace, int64_t workspace_bytes,
                                 int phase, void* stream) {
  if (phase != INT8KV_EXCHANGE_BOTH_PHASES && phase != INT8KV_EXCHANGE_MERGE_PHASE && phase != INT8KV_EXCHANGE_GATHER_PHASE)
    return INT8KV_E_BAD_SHAPE;
  if (batch < 0 || num_q_heads <= 0 || head_dim <= 0) return INT8KV_E_BAD_SHAPE;
  if (!valid_float_dtype(out_dtype)) return INT8KV_E_BAD_DTYPE;
  ExchangeParams e;
  const int rc = exchange_params(exchange, batch, num_q_heads, head_dim, &e);
  if (rc != INT8KV_OK) return rc;
  if (batch == 0) return INT8KV_OK;
  if (!out || !out_strides) return INT8KV_E_NULLPTR;
  MergeParams m;
  std::memset(&m, 0, sizeof(m));
  const int64_t rank_floats = e.rows * e.row_floats;  // floats of one rank's rows
  m.parts = reinterpret_cast<const float*>(e.peer[e.rank] + kExchCtrlBytes) + rank_floats;  // slab 0 follows the staging
  m.R = e.world; m.rows = e.rows; m.Hq = num_q_heads; m.D = head_dim; m.row_floats = e.row_floats;
  m.out = out; m.out_dtype = out_dtype;
  for (int i = 0; i < 3; ++i) m.o_st[i] = out_strides[i];
  m.exchange_ctrl = reinterpret_cast<const int*>(e.peer[e.rank]);
  m.exchange_world = e.world;
  m.slab_floats = rank_floats * e.world;  // pairs per slab
  if (workspace != nullptr && workspace_bytes >= 16)
    m.status = reinterpret_cast<unsigned int*>(static_cast<char*>(workspace) + int8kv_workspace_status_offset(workspace_bytes));
  return launch_merge_exchanged(m, e, phase, static_cast<cudaStream_t>(stream));
}

int int8kv_selftest_bounded_wait(void* workspace, int64_t workspace_bytes, int attempts, void* stream) {
  if (workspace == nullptr || workspace_bytes < 16) return INT8KV_E_WORKSPACE;
  if (attempts <= 0 || attempts > (1 << 16)) return INT8KV_E_BAD_SHAPE;
  unsigned int* status =
      reinterpret_cast<unsigned int*>(static_cast<char*>(workspace) + int8kv_workspace_status_offset(workspace_bytes));
  return launch_bounded_wait_selftest(status, static_cast<unsigned int>(attempts), static_cast<cudaStream_t>(stream));
}

int int8kv_cache_write_dynamic(const void* key, const void* value, int in_dtype, int64_t num_tokens, int num_kv_heads,
                               int head_dim, const int64_t key_strides[3], const int64_t value_strides[3],
                               int8_t* key_cache, int8_t* value_cache, const int64_t key_cache_strides[4],
                               const int64_t value_cache_strides[4], float* k_scale_cache, float* v_scale_cache,
                               const int64_t k_scale_strides[3], const int64_t v_scale_strides[3], int64_t num_blocks,
                               int block_size, const void* slot_mapping, int slot_is_i64, void* stream) {
  if (num_tokens < 0 || num_kv_heads <= 0 || head_dim <= 0 || num_blocks < 0 || block_size <= 0)
    return INT8KV_E_BAD_SHAPE;
  if (!valid_float_dtype(in_dtype)) return INT8KV_E_BAD_DTYPE;
  if (num_tokens == 0) return INT8KV_OK;
  if (!key || !value || !key_cache || !value_cache || !k_scale_cache || !v_scale_cache || !slot_mapping ||
      !key_strides || !value_strides || !key_cache_strides || !value_cache_strides || !k_scale_strides ||
      !v_scale_strides)
    return INT8KV_E_NULLPTR;
  DynWriteParams p;
  std::memset(&p, 0, sizeof(p));
  p.key = key; p.value = value; p.in_dtype = in_dtype;
  p.T = num_tokens; p.Hkv = num_kv_heads; p.D = head_dim;
  for (int i = 0; i < 3; ++i) {
    p.k_st[i] = key_strides[i]; p.v_st[i] = value_strides[i];
    p.ks_st[i] = k_scale_strides[i]; p.vs_st[i] = v_scale_strides[i];
  }
  p.kc = key_cache; p.vc = value_cache; p.ks = k_scale_cache; p.vs = v_scale_cache;
  for (int i = 0; i < 4; ++i) { p.kc_st[i] = key_cache_strides[i]; p.vc_st[i] = value_cache_strides[i]; }
  p.num_slots = num_blocks * block_size;
  p.block_size = block_size;
  p.slots = slot_mapping; p.slot_is_i64 = slot_is_i64;
  return launch_cache_write_dynamic(p, static_cast<cudaStream_t>(stream));
}

int int8kv_decode_step(const void* key, const void* value, int kv_dtype, const int64_t key_strides[3],
                       const int64_t value_strides[3], const void* slot_mapping, int slot_is_i64,
                       const void* query, int q_dtype, const int64_t q_strides[3], int batch, int num_q_heads,
                       int num_kv_heads, int head_dim, int8_t* key_cache, int8_t* value_cache,
                       const int64_t key_cache_strides[4], const int64_t value_cache_strides[4], int64_t num_blocks,
                       int block_size, const void* block_tables, int bt_is_i64, const int64_t bt_strides[2],
                       int64_t bt_width, const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                       const float* k_scale, const float* v_scale, void* out, int out_dtype,
                       const int64_t out_strides[3], int num_splits, void* workspace, int64_t workspace_bytes,
                       int flags, void* stream) {
  if (!key || !value || !slot_mapping || !key_strides || !value_strides) return batch == 0 ? INT8KV_OK : INT8KV_E_NULLPTR;
  if (!valid_float_dtype(kv_dtype)) return INT8KV_E_BAD_DTYPE;
  // Shapes the tiled kernel covers: one launch does both.  For any other shape run_attention refuses with
  // INT8KV_E_UNSUPPORTED before launching anything, and the two-call form runs instead.
  AttnCall a{query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
             key_cache, value_cache, kCacheInt8, key_cache_strides, value_cache_strides, num_blocks, block_size,
             block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
             k_scale, v_scale, out, out_dtype, out_strides, nullptr,
             num_splits, workspace, workspace_bytes, flags, static_cast<cudaStream_t>(stream)};
  a.new_k = key; a.new_v = value; a.new_dtype = kv_dtype; a.nk_st = key_strides; a.nv_st = value_strides;
  a.new_slots = slot_mapping; a.new_slot_is_i64 = slot_is_i64;
  int rc = run_attention(a);
  if (rc != INT8KV_E_UNSUPPORTED) return rc;
  rc = int8kv_cache_write(key, value, kv_dtype, batch, num_kv_heads, head_dim, key_strides, value_strides,
                          key_cache, value_cache, key_cache_strides, value_cache_strides, num_blocks,
                          block_size, slot_mapping, slot_is_i64, k_scale, v_scale, stream);
  if (rc != INT8KV_OK) return rc;
  return int8kv_paged_attn_int8(query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim, key_cache,
                                value_cache, key_cache_strides, value_cache_strides, num_blocks, block_size,
                                block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64,
                                max_seq_len_hint, k_scale, v_scale, out, out_dtype, out_strides, num_splits,
                                workspace, workspace_bytes, flags & ~INT8KV_FLAG_INPUTS_READY, stream);
}

}  // extern "C"

namespace {

// The layers of one model step, INT8 caches (with or without the step's cache write) or float caches (attention
// only), behind one call.  With the inputs-ready promise and a workspace of at least twice one layer's need, the
// layers are CHAINED: layer l works in half l % 2 of the workspace and its split-KV merge is carried by the launch of
// layer l + 1, so a step is one launch per layer plus one closing merge, and a layer's page stream starts under the
// previous layer's tail.
int run_layers(const int8kv_layer_args* layers, int num_layers, int* failed_layer, int cache_kind, int kv_dtype,
               const int64_t* key_strides, const int64_t* value_strides, const void* slot_mapping, int slot_is_i64,
               int q_dtype, const int64_t* q_strides, int batch, int num_q_heads, int num_kv_heads, int head_dim,
               const int64_t* key_cache_strides, const int64_t* value_cache_strides, int64_t num_blocks,
               int block_size, const void* block_tables, int bt_is_i64, const int64_t* bt_strides, int64_t bt_width,
               const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint, int out_dtype,
               const int64_t* out_strides, int num_splits, void* workspace, int64_t workspace_bytes, int flags,
               void* stream) {
  if (failed_layer) *failed_layer = -1;
  if (num_layers < 0) return INT8KV_E_BAD_SHAPE;
  if (num_layers == 0) return INT8KV_OK;
  if (!layers) return INT8KV_E_NULLPTR;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto make_call = [&](const int8kv_layer_args& L, void* ws, int64_t ws_bytes, int lf) {
    AttnCall a{L.query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
               L.key_cache, L.value_cache, cache_kind, key_cache_strides, value_cache_strides, num_blocks, block_size,
               block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
               L.k_scale, L.v_scale, L.out, out_dtype, out_strides, nullptr,
               num_splits, ws, ws_bytes, lf, st};
    if (L.key != nullptr) {
      a.new_k = L.key; a.new_v = L.value; a.new_dtype = kv_dtype; a.nk_st = key_strides; a.nv_st = value_strides;
      a.new_slots = slot_mapping; a.new_slot_is_i64 = slot_is_i64;
    }
    return a;
  };
  Chain chain;
  char* ws = static_cast<char*>(workspace);
  int64_t half = 0;
  unsigned int* status = nullptr;
  if ((flags & INT8KV_FLAG_INPUTS_READY) && num_layers > 1 && ws != nullptr && workspace_bytes >= 1024 &&
      (reinterpret_cast<uintptr_t>(ws) & 255u) == 0) {
    half = (workspace_bytes / 2) & ~int64_t(255);
    status = reinterpret_cast<unsigned int*>(ws + int8kv_workspace_status_offset(workspace_bytes));
    AttnCall probe = make_call(layers[0], ws, half, flags);
    AttnPlan t;
    std::memset(&t, 0, sizeof(t));
    chain.active = batch > 0 && plan_attention(probe, t) == INT8KV_OK && t.tiled;  // else: one workspace, own merges
  }
  for (int l = 0; l < num_layers; ++l) {
    const int8kv_layer_args& L = layers[l];
    if (L.key != nullptr && (!L.value || !slot_mapping || !key_strides || !value_strides) && batch > 0) {
      flush_chain(&chain, st);
      if (failed_layer) *failed_layer = l;
      return INT8KV_E_NULLPTR;
    }
    if (L.key != nullptr && !valid_float_dtype(kv_dtype)) {
      flush_chain(&chain, st);
      if (failed_layer) *failed_layer = l;
      return INT8KV_E_BAD_DTYPE;
    }
    // the promise is about the layers of this call; what precedes the call on the stream is unknown here, so the
    // first layer orders itself behind it in the ordinary way
    const int lf = l == 0 ? (flags & ~INT8KV_FLAG_INPUTS_READY) : flags;
    AttnCall a = chain.active ? make_call(L, ws + (l & 1) * half, half, lf) : make_call(L, workspace, workspace_bytes, lf);
    if (chain.active) {
      a.status = status;
      a.chained = true;
    }
    int rc = run_attention(a, &chain);
    if (rc == INT8KV_E_UNSUPPORTED && L.key != nullptr) {
      // a shape outside the tiled kernel: the write and the attention as two calls (nothing was launched above)
      rc = flush_chain(&chain, st);
      if (rc == INT8KV_OK)
        rc = int8kv_cache_write(L.key, L.value, kv_dtype, batch, num_kv_heads, head_dim, key_strides, value_strides,
                                L.key_cache, L.value_cache, key_cache_strides, value_cache_strides, num_blocks,
                                block_size, slot_mapping, slot_is_i64, L.k_scale, L.v_scale, stream);
      if (rc == INT8KV_OK) {
        AttnCall b = make_call(L, workspace, workspace_bytes, lf & ~INT8KV_FLAG_INPUTS_READY);
        b.new_k = nullptr;
        rc = run_attention(b, nullptr);
      }
    }
    if (rc != INT8KV_OK) {
      flush_chain(&chain, st);
      if (failed_layer) *failed_layer = l;
      return rc;
    }
  }
  return flush_chain(&chain, st);
}

}  // namespace

extern "C" {

int int8kv_decode_step_layers(const int8kv_layer_args* layers, int num_layers, int* failed_layer, int kv_dtype,
                              const int64_t key_strides[3], const int64_t value_strides[3],
                              const void* slot_mapping, int slot_is_i64, int q_dtype, const int64_t q_strides[3],
                              int batch, int num_q_heads, int num_kv_heads, int head_dim,
                              const int64_t key_cache_strides[4], const int64_t value_cache_strides[4],
                              int64_t num_blocks, int block_size, const void* block_tables, int bt_is_i64,
                              const int64_t bt_strides[2], int64_t bt_width, const void* seq_lens, int sl_is_i64,
                              int64_t max_seq_len_hint, int out_dtype, const int64_t out_strides[3],
                              int num_splits, void* workspace, int64_t workspace_bytes, int flags, void* stream) {
  return run_layers(layers, num_layers, failed_layer, kCacheInt8, kv_dtype, key_strides, value_strides, slot_mapping,
                    slot_is_i64, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim, key_cache_strides,
                    value_cache_strides, num_blocks, block_size, block_tables, bt_is_i64, bt_strides, bt_width,
                    seq_lens, sl_is_i64, max_seq_len_hint, out_dtype, out_strides, num_splits, workspace,
                    workspace_bytes, flags, stream);
}

int int8kv_paged_attn_bf16_layers(const int8kv_layer_args* layers, int num_layers, int* failed_layer, int cache_dtype,
                                  int q_dtype, const int64_t q_strides[3], int batch, int num_q_heads,
                                  int num_kv_heads, int head_dim, const int64_t key_cache_strides[4],
                                  const int64_t value_cache_strides[4], int64_t num_blocks, int block_size,
                                  const void* block_tables, int bt_is_i64, const int64_t bt_strides[2],
                                  int64_t bt_width, const void* seq_lens, int sl_is_i64, int64_t max_seq_len_hint,
                                  int out_dtype, const int64_t out_strides[3], int num_splits, void* workspace,
                                  int64_t workspace_bytes, int flags, void* stream) {
  if (failed_layer) *failed_layer = -1;
  if (cache_dtype != INT8KV_BF16 && cache_dtype != INT8KV_FP16) return INT8KV_E_BAD_DTYPE;
  for (int l = 0; layers != nullptr && l < num_layers; ++l)
    if (layers[l].key != nullptr || layers[l].value != nullptr) {  // float caches have no quantising write
      if (failed_layer) *failed_layer = l;
      return INT8KV_E_UNSUPPORTED;
    }
  return run_layers(layers, num_layers, failed_layer, cache_dtype == INT8KV_BF16 ? kCacheBf16 : kCacheFp16, 0, nullptr,
                    nullptr, nullptr, 0, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
                    key_cache_strides, value_cache_strides, num_blocks, block_size, block_tables, bt_is_i64,
                    bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint, out_dtype, out_strides, num_splits,
                    workspace, workspace_bytes, flags, stream);
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant: the split-KV workspace is a buffer inside the library image.
// ---------------------------------------------------------------------------------------------------------
}  // extern "C"

// The workspace itself, at file scope.  In host code this name is only a handle for the runtime: it is NOT a
// device address and must never be handed to a kernel; the address the kernels use comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_ws[INT8KV_STATIC_WS_BYTES];

namespace {

// Device address of g_static_ws on each device, looked up on the first call made with that device current.
std::atomic<void*> g_static_ws_addr[kMaxDevices];

int static_ws_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return INT8KV_E_LAUNCH;
  void* p = g_static_ws_addr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_ws) != cudaSuccess || p == nullptr) return INT8KV_E_LAUNCH;
    g_static_ws_addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return INT8KV_OK;
}

}  // namespace

extern "C" {

int int8kv_paged_attn_int8_static_ws(const void* query, int q_dtype, const int64_t q_strides[3], int batch,
                                     int num_q_heads, int num_kv_heads, int head_dim, const int8_t* key_cache,
                                     const int8_t* value_cache, const int64_t key_cache_strides[4],
                                     const int64_t value_cache_strides[4], int64_t num_blocks, int block_size,
                                     const void* block_tables, int bt_is_i64, const int64_t bt_strides[2],
                                     int64_t bt_width, const void* seq_lens, int sl_is_i64,
                                     int64_t max_seq_len_hint, const float* k_scale, const float* v_scale,
                                     void* out, int out_dtype, const int64_t out_strides[3], int num_splits,
                                     int flags, void* stream) {
  // The same selection and the same checks as int8kv_paged_attn_int8 given a workspace of INT8KV_STATIC_WS_BYTES
  // bytes: run_attention picks the split count (the tiled or the untiled rule, or the device plan when its rows
  // and table fit) and refuses with INT8KV_E_WORKSPACE, before it launches anything, what does not fit.
  if (batch < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || block_size <= 0 || bt_width < 0 ||
      num_splits < INT8KV_SPLITS_PLANNED || num_splits > kMaxSplits)
    return INT8KV_E_BAD_SHAPE;
  void* ws = nullptr;
  const int rc = static_ws_address(&ws);
  if (rc != INT8KV_OK) return rc;
  AttnCall a{query, q_dtype, q_strides, batch, num_q_heads, num_kv_heads, head_dim,
             key_cache, value_cache, kCacheInt8, key_cache_strides, value_cache_strides, num_blocks, block_size,
             block_tables, bt_is_i64, bt_strides, bt_width, seq_lens, sl_is_i64, max_seq_len_hint,
             k_scale, v_scale, out, out_dtype, out_strides, nullptr,
             num_splits, ws, INT8KV_STATIC_WS_BYTES, flags, static_cast<cudaStream_t>(stream)};
  return run_attention(a);
}

int int8kv_static_ws_address(void** device_ptr) {
  if (device_ptr == nullptr) return INT8KV_E_NULLPTR;
  return static_ws_address(device_ptr);
}

int int8kv_static_ws_status(void* dst, int clear, void* stream) {
  if (dst == nullptr) return INT8KV_E_NULLPTR;
  void* ws = nullptr;
  const int rc = static_ws_address(&ws);
  if (rc != INT8KV_OK) return rc;
  char* word = static_cast<char*>(ws) + int8kv_workspace_status_offset(INT8KV_STATIC_WS_BYTES);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(dst, word, 4, cudaMemcpyDefault, st) != cudaSuccess) return INT8KV_E_LAUNCH;
  if (clear && cudaMemsetAsync(word, 0, 4, st) != cudaSuccess) return INT8KV_E_LAUNCH;
  return INT8KV_OK;
}

}  // extern "C"
