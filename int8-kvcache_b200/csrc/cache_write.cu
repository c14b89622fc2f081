// INT8 KV cache write for sm_100a: static per-KV-head symmetric quantisation of new K/V rows and a
// scatter through slot_mapping into the paged caches, one pass over the data.
//
// Arithmetic (bit-exact target): q = clamp(rint(float(x) / max(scale, 1e-6)), -127, 127) with an IEEE
// fp32 division and round-half-to-even, i.e. the result of the reference's torch oracle
// (src/quant.py:37-40) with the scale floor of its Triton kernel (src/triton_ops/int8_cache_write.py:50-51).
// No fast-math: a reciprocal multiply alone is not bit-identical to the division (see quant1).
//
// The kernel is a pure HBM stream (per token and KV head: 2*D*sizeof(in) bytes read, 2*D bytes written).
// Vector path: each thread owns 16 consecutive elements of one (token, head) row of K and of V: it
// issues all of its 16-byte loads first, then quantises and stores one 16-byte int8 vector per tensor,
// so a warp reads 1 KB (bf16) of consecutive input and writes 512 B of consecutive cache.
#include <algorithm>
#include <atomic>

#include "common.cuh"

namespace int8kv {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

// The exact form of one quantisation, out of line: IEEE division, clamp, round-half-even (what quant1 does inline
// for an element within a few ulp of a rounding tie, or huge, infinite or NaN).  About one element in ten thousand
// of real activations takes it, so its cost does not matter, while keeping a division sequence out of the streaming
// code behind each of a thread's 32 elements does: with it inline, the warps of this kernel waited for instruction
// fetch as often as for memory (13.4 us per 16384-token write against 12.9 us, same box).
__device__ __noinline__ int quant1_exact(float x, float scale) {
  const float q = fminf(fmaxf(x / scale, -127.f), 127.f);  // div.rn.f32; also maps +-inf
  float t = q + kRoundMagic;
  if (x != x) t = kRoundMagic;  // NaN -> 0, as a float-to-int8 cast of NaN gives on the CPU
  return __float_as_int(t) - kRoundMagicBits;
}

// 1 / scale for the streaming path, from the special-function unit alone (relative error at most 2^-23, against
// 2^-24 for the IEEE reciprocal, which costs a correction sequence per thread): the product x * (1 / scale) is then
// within 3 ulp of the true quotient instead of 2, i.e. within 2.3e-5 below 128, still well inside the 6.2e-5 around
// a tie inside which the exact division decides.
__device__ __forceinline__ float rcp_fast(float scale) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(scale));
  return r;
}

// Two quantisations at a time on the packed FP32 pipe (mul / add / fma on register pairs, sm_100): the same
// arithmetic as quant1 (common.cuh) element by element — q = x * (1/scale), t = q + 1.5 * 2^23, n = t - 1.5 * 2^23,
// exact division only when |q - n| comes within 6.2e-5 of one half — with two differences that save instructions,
// this kernel being bound by its instruction stream (18 per element before, against 7.7 us of HBM time for 13 us
// of issue slots):
//  * no separate test for huge quotients.  For q >= 2^22 the bits of t lie above those of 1.5 * 2^23 by at least
//    2^22 and the difference saturates to +127, as it must; for q <= -2^22 they lie below (t <= 2^23, down to zero)
//    and it saturates to -127; the one failure is t < 0, whose sign bit would wrap the integer subtraction, so
//    the bits are clamped from below first (one integer max).  Infinities and NaN make q - n NaN and take the exact
//    path through the comparison itself.
//  * the rare branch is out of line (quant1_exact).
__device__ __forceinline__ void quant2_stream(float x0, float x1, float scale, float2 rscale2, int& n0, int& n1) {
  const float2 q = __fmul2_rn(make_float2(x0, x1), rscale2);
  const float2 t = __fadd2_rn(q, make_float2(kRoundMagic, kRoundMagic));
  const float2 n = __fadd2_rn(t, make_float2(-kRoundMagic, -kRoundMagic));
  const float2 d = __ffma2_rn(n, make_float2(-1.f, -1.f), q);  // q - n, exact
  // The bits are clamped from below at those of 1.5 * 2^23 - 127 before the subtraction: -127 is the least result
  // (also for t < 0, whose sign bit would wrap the subtraction), so packing only has to saturate at +127 and the
  // four-byte maximum that raises -128 to -127 is not needed.  (A fused add-then-max would wrap for
  // -1.5 * 2^23 < t < 0.)
  n0 = max(__float_as_int(t.x), kRoundMagicBits - 127) - kRoundMagicBits;
  n1 = max(__float_as_int(t.y), kRoundMagicBits - 127) - kRoundMagicBits;
  if (!(fabsf(d.x) < 0.5f - 6.2e-5f)) n0 = quant1_exact(x0, scale);
  if (!(fabsf(d.y) < 0.5f - 6.2e-5f)) n1 = quant1_exact(x1, scale);
}

// Four integers >= -127 saturated at +127 and packed little-endian.
__device__ __forceinline__ uint32_t pack4_sat_upper(int n0, int n1, int n2, int n3) {
  uint32_t hi, w;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(n3), "r"(n2), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(n1), "r"(n0), "r"(hi));
  return w;
}

// Sixteen consecutive elements as raw 16-byte vectors (requested before anything depends on them) ...
template <typename T>
struct Raw16 {
  static constexpr int kVecs = 16 * sizeof(T) / 16;
  uint4 v[kVecs];
  __device__ __forceinline__ void load(const T* p) {
#pragma unroll
    for (int i = 0; i < kVecs; ++i) v[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  }
  // ... and their quantised bytes
  __device__ __forceinline__ uint4 quantise(float scale, float rscale) const {
    const T* e = reinterpret_cast<const T*>(v);
    const float2 r2 = make_float2(rscale, rscale);
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int n[4];
      quant2_stream(to_f32<T>(e[4 * i]), to_f32<T>(e[4 * i + 1]), scale, r2, n[0], n[1]);
      quant2_stream(to_f32<T>(e[4 * i + 2]), to_f32<T>(e[4 * i + 3]), scale, r2, n[2], n[3]);
      w[i] = pack4_sat_upper(n[0], n[1], n[2], n[3]);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Vector path: D % 16 == 0, unit innermost strides, 16-byte aligned rows on both sides.  One thread per 16
// elements of one (token, head) row of K and of V; index arithmetic in 32 bits (the launcher guarantees the
// unit count fits) and by shift where the sizes are powers of two.  128 threads and a register cap that fits 12
// CTAs = 48 warps per SM: finer waves and more resident warps than 256 threads x 5 CTAs (12.8 -> 11.8 us on the
// 16384-token write).
// DENSE: K and V rows and both caches are dense in their logical order and Hkv * D / 16 and D / 16 are powers of two
// (the launcher checks), so a unit's source is unit * 16 elements from the base and its destination slot * Hkv * D +
// (unit mod units-per-token) * 16: a handful of shifts instead of ten 64-bit stride products per thread.
constexpr int kVecThreads = 128;
template <typename T, bool DENSE>
__global__ void __launch_bounds__(kVecThreads, 12) cache_write_vec_kernel(const WriteParams p, const uint32_t total,
                                                              const int bs_shift, const int pt_shift, const int ch_shift) {
  const uint32_t chunks = static_cast<uint32_t>(p.D) >> 4;
  const uint32_t per_token = static_cast<uint32_t>(p.Hkv) * chunks;
  const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  grid_dependency_wait();    // the new rows and the slots may come from the kernel launched just before
  grid_launch_dependents();  // the next kernel in the stream waits for this grid before it reads the cache
  if constexpr (DENSE) {
    const uint32_t t = idx >> pt_shift;
    const uint32_t rem = idx & ((1u << pt_shift) - 1u);
    const uint32_t h = rem >> ch_shift;
    const int64_t slot = load_index(p.slots, p.slot_is_i64, t);
    Raw16<T> kr, vr;
    kr.load(reinterpret_cast<const T*>(p.key) + static_cast<int64_t>(idx) * 16);
    vr.load(reinterpret_cast<const T*>(p.value) + static_cast<int64_t>(idx) * 16);
    const float ks = fmaxf(__ldg(p.k_scale + h), 1e-6f);
    const float vs = fmaxf(__ldg(p.v_scale + h), 1e-6f);
    if (slot < 0 || slot >= p.num_slots) return;
    const int64_t dst = (slot << (pt_shift + 4)) + (rem << 4);
    *reinterpret_cast<uint4*>(p.kc + dst) = kr.quantise(ks, rcp_fast(ks));
    *reinterpret_cast<uint4*>(p.vc + dst) = vr.quantise(vs, rcp_fast(vs));
    return;
  }
  const uint32_t t = pt_shift >= 0 ? idx >> pt_shift : idx / per_token;
  const uint32_t rem = idx - t * per_token;
  const uint32_t h = ch_shift >= 0 ? rem >> ch_shift : rem / chunks;
  const uint32_t c = rem - h * chunks;
  // the slot and the K/V vectors are independent loads: all are in flight before the first use
  const int64_t slot = load_index(p.slots, p.slot_is_i64, t);
  Raw16<T> kr, vr;
  kr.load(reinterpret_cast<const T*>(p.key) + static_cast<int64_t>(t) * p.k_st[0] + h * p.k_st[1] + c * 16);
  vr.load(reinterpret_cast<const T*>(p.value) + static_cast<int64_t>(t) * p.v_st[0] + h * p.v_st[1] + c * 16);
  const float ks = fmaxf(__ldg(p.k_scale + h), 1e-6f);
  const float vs = fmaxf(__ldg(p.v_scale + h), 1e-6f);
  if (slot < 0 || slot >= p.num_slots) return;
  const int64_t blk = bs_shift >= 0 ? (slot >> bs_shift) : slot / p.block_size;
  const int64_t off = slot - blk * p.block_size;
  int8_t* kd = p.kc + blk * p.kc_st[0] + off * p.kc_st[1] + h * p.kc_st[2] + c * 16;
  int8_t* vd = p.vc + blk * p.vc_st[0] + off * p.vc_st[1] + h * p.vc_st[2] + c * 16;
  *reinterpret_cast<uint4*>(kd) = kr.quantise(ks, rcp_fast(ks));
  *reinterpret_cast<uint4*>(vd) = vr.quantise(vs, rcp_fast(vs));
}

// Element path: any D, any strides, any alignment.
__global__ void __launch_bounds__(256) cache_write_elem_kernel(const WriteParams p) {
  const int64_t per_token = static_cast<int64_t>(p.Hkv) * p.D;
  const int64_t total = p.T * per_token;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = idx / per_token;
    const int rem = static_cast<int>(idx - t * per_token);
    const int h = rem / p.D;
    const int d = rem - h * p.D;
    const int64_t slot = load_index(p.slots, p.slot_is_i64, t);
    if (slot < 0 || slot >= p.num_slots) continue;
    const float kx = load_as_float(p.key, p.in_dtype, t * p.k_st[0] + h * p.k_st[1] + d * p.k_st[2]);
    const float vx = load_as_float(p.value, p.in_dtype, t * p.v_st[0] + h * p.v_st[1] + d * p.v_st[2]);
    const float ks = fmaxf(__ldg(p.k_scale + h), 1e-6f);
    const float vs = fmaxf(__ldg(p.v_scale + h), 1e-6f);
    const int64_t blk = slot / p.block_size;
    const int64_t off = slot - blk * p.block_size;
    p.kc[blk * p.kc_st[0] + off * p.kc_st[1] + h * p.kc_st[2] + d * p.kc_st[3]] = static_cast<int8_t>(max(-127, min(127, quant1(kx, ks, __frcp_rn(ks)))));
    p.vc[blk * p.vc_st[0] + off * p.vc_st[1] + h * p.vc_st[2] + d * p.vc_st[3]] = static_cast<int8_t>(max(-127, min(127, quant1(vx, vs, __frcp_rn(vs)))));
  }
}

// Dynamic per-(token, head) quantisation (the reference's alternative scheme, vllm_int8/vllm_int8_cache_ops.py:13-131):
// scale = max(absmax / 127, 1e-6) over the head's D elements, q = round_half_away(clamp(x / scale, +-127)), INT8 row
// and fp32 scale are stored at the token's slot.  One warp per (token, head); rows up to 16 elements per lane are kept
// in registers, longer ones are read a second time.
__global__ void __launch_bounds__(256) cache_write_dynamic_kernel(const DynWriteParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= p.T * p.Hkv) return;
  const int64_t t = row / p.Hkv;
  const int h = static_cast<int>(row - t * p.Hkv);
  const int64_t slot = load_index(p.slots, p.slot_is_i64, t);
  if (slot < 0 || slot >= p.num_slots) return;
  const int64_t blk = slot / p.block_size;
  const int64_t off = slot - blk * p.block_size;
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const void* src = which ? p.value : p.key;
    const int64_t* st = which ? p.v_st : p.k_st;
    int8_t* cache = which ? p.vc : p.kc;
    const int64_t* cst = which ? p.vc_st : p.kc_st;
    float* scales = which ? p.vs : p.ks;
    const int64_t* sst = which ? p.vs_st : p.ks_st;
    const int64_t base = t * st[0] + h * st[1];
    constexpr int kKeep = 16;
    float x[kKeep];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int d = lane + 32 * i;
      x[i] = d < p.D ? load_as_float(src, p.in_dtype, base + d * st[2]) : 0.f;
      amax = fmaxf(amax, fabsf(x[i]));
    }
    for (int d = lane + 32 * kKeep; d < p.D; d += 32) amax = fmaxf(amax, fabsf(load_as_float(src, p.in_dtype, base + d * st[2])));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax / 127.f, 1e-6f);
    const int64_t cbase = blk * cst[0] + off * cst[1] + h * cst[2];
    auto quant = [scale](float v) {
      float q = fminf(fmaxf(v / scale, -127.f), 127.f);
      q = q >= 0.f ? floorf(q + 0.5f) : ceilf(q - 0.5f);
      return static_cast<int8_t>(static_cast<int>(q));
    };
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int d = lane + 32 * i;
      if (d < p.D) cache[cbase + d * cst[3]] = quant(x[i]);
    }
    for (int d = lane + 32 * kKeep; d < p.D; d += 32)
      cache[cbase + d * cst[3]] = quant(load_as_float(src, p.in_dtype, base + d * st[2]));
    if (lane == 0) scales[blk * sst[0] + off * sst[1] + h * sst[2]] = scale;
  }
}

// Vector path of the dynamic scheme: D / 16 (a power of two, at most 32) consecutive lanes share one
// (token, head) row; each holds 16 elements of K and of V, the row maxima are three to five shuffles, and the
// bytes leave as 16-byte stores.  Same conditions on strides and alignment as the static vector path.
template <typename T>
__global__ void __launch_bounds__(256) cache_write_dynamic_vec_kernel(const DynWriteParams p, const uint32_t total,
                                                                      const int chunk_shift) {
  const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = idx < total;  // whole row groups are valid or not: total is a multiple of the group size
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t chunks = 1u << chunk_shift;
  const uint32_t row = idx >> chunk_shift;
  const uint32_t c = idx & (chunks - 1);
  const uint32_t t = row / static_cast<uint32_t>(p.Hkv);
  const uint32_t h = row - t * static_cast<uint32_t>(p.Hkv);
  int64_t slot = -1;
  Raw16<T> kr, vr;
  if (valid) {
    slot = load_index(p.slots, p.slot_is_i64, t);
    kr.load(reinterpret_cast<const T*>(p.key) + static_cast<int64_t>(t) * p.k_st[0] + h * p.k_st[1] + c * 16);
    vr.load(reinterpret_cast<const T*>(p.value) + static_cast<int64_t>(t) * p.v_st[0] + h * p.v_st[1] + c * 16);
  } else {
#pragma unroll
    for (int i = 0; i < Raw16<T>::kVecs; ++i) kr.v[i] = vr.v[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  const T* ke = reinterpret_cast<const T*>(kr.v);
  const T* ve = reinterpret_cast<const T*>(vr.v);
  float kx[16], vx[16], kmax = 0.f, vmax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    kx[i] = to_f32<T>(ke[i]);
    vx[i] = to_f32<T>(ve[i]);
    kmax = fmaxf(kmax, fabsf(kx[i]));
    vmax = fmaxf(vmax, fabsf(vx[i]));
  }
  for (uint32_t o = 1; o < chunks; o <<= 1) {
    kmax = fmaxf(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
  }
  if (!valid || slot < 0 || slot >= p.num_slots) return;
  const float ks = fmaxf(__fdiv_rn(kmax, 127.f), 1e-6f), vs = fmaxf(__fdiv_rn(vmax, 127.f), 1e-6f);
  const float rk = __frcp_rn(ks), rv = __frcp_rn(vs);
  uint32_t kw[4], vw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    kw[i] = pack4_sat(quant_half_away(kx[4 * i], ks, rk), quant_half_away(kx[4 * i + 1], ks, rk),
                      quant_half_away(kx[4 * i + 2], ks, rk), quant_half_away(kx[4 * i + 3], ks, rk));
    vw[i] = pack4_sat(quant_half_away(vx[4 * i], vs, rv), quant_half_away(vx[4 * i + 1], vs, rv),
                      quant_half_away(vx[4 * i + 2], vs, rv), quant_half_away(vx[4 * i + 3], vs, rv));
  }
  const int64_t blk = slot / p.block_size;
  const int64_t off = slot - blk * p.block_size;
  *reinterpret_cast<uint4*>(p.kc + blk * p.kc_st[0] + off * p.kc_st[1] + h * p.kc_st[2] + c * 16) =
      make_uint4(kw[0], kw[1], kw[2], kw[3]);
  *reinterpret_cast<uint4*>(p.vc + blk * p.vc_st[0] + off * p.vc_st[1] + h * p.vc_st[2] + c * 16) =
      make_uint4(vw[0], vw[1], vw[2], vw[3]);
  if (c == 0) {
    p.ks[blk * p.ks_st[0] + off * p.ks_st[1] + h * p.ks_st[2]] = ks;
    p.vs[blk * p.vs_st[0] + off * p.vs_st[1] + h * p.vs_st[2]] = vs;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_cache_write_dynamic(const DynWriteParams& p, cudaStream_t stream) {
  const int64_t rows = p.T * p.Hkv;
  if (rows <= 0) return INT8KV_OK;
  const int esz = dtype_bytes(p.in_dtype);
  const int per16 = 16 / esz;
  const int chunks = p.D / 16;
  const int64_t units = rows * chunks;
  bool vec = (p.D % 16 == 0) && chunks >= 1 && chunks <= 32 && (chunks & (chunks - 1)) == 0 && p.k_st[2] == 1 &&
             p.v_st[2] == 1 && p.kc_st[3] == 1 && p.vc_st[3] == 1 && aligned16(p.key) && aligned16(p.value) &&
             aligned16(p.kc) && aligned16(p.vc) && units < (int64_t(1) << 31);
  for (int i = 0; i < 2 && vec; ++i) vec = (p.k_st[i] % per16 == 0) && (p.v_st[i] % per16 == 0);
  for (int i = 0; i < 3 && vec; ++i) vec = (p.kc_st[i] % 16 == 0) && (p.vc_st[i] % 16 == 0);
  if (vec) {
    int shift = 0;
    while ((1 << shift) < chunks) ++shift;
    const unsigned blocks = static_cast<unsigned>((units + 255) / 256);
    const uint32_t total = static_cast<uint32_t>(units);
    if (p.in_dtype == INT8KV_BF16) return launch_pdl(cache_write_dynamic_vec_kernel<__nv_bfloat16>, blocks, 256, 0, stream, p, total, shift);
    if (p.in_dtype == INT8KV_FP16) return launch_pdl(cache_write_dynamic_vec_kernel<__half>, blocks, 256, 0, stream, p, total, shift);
    return launch_pdl(cache_write_dynamic_vec_kernel<float>, blocks, 256, 0, stream, p, total, shift);
  }
  const int64_t blocks = (rows + 7) / 8;  // 8 warps per CTA
  cache_write_dynamic_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? INT8KV_OK : INT8KV_E_LAUNCH;
}

int launch_cache_write(const WriteParams& p, int sm_count, cudaStream_t stream) {
  if (p.T == 0) return INT8KV_OK;
  const int esz = dtype_bytes(p.in_dtype);
  const int per16 = 16 / esz;  // elements per 16 bytes
  const int64_t units = p.T * p.Hkv * (p.D / 16);
  bool vec = (p.D % 16 == 0) && p.k_st[2] == 1 && p.v_st[2] == 1 && p.kc_st[3] == 1 && p.vc_st[3] == 1 &&
             aligned16(p.key) && aligned16(p.value) && aligned16(p.kc) && aligned16(p.vc) &&
             units < (int64_t(1) << 31) && p.T < (int64_t(1) << 31);
  for (int i = 0; i < 2 && vec; ++i) vec = (p.k_st[i] % per16 == 0) && (p.v_st[i] % per16 == 0);
  for (int i = 0; i < 3 && vec; ++i) vec = (p.kc_st[i] % 16 == 0) && (p.vc_st[i] % 16 == 0);
  const int threads = vec ? kVecThreads : 256;
  if (vec) {
    auto shift_of = [](int64_t x) {
      if (x <= 0 || (x & (x - 1)) != 0) return -1;
      int sh = 0;
      while ((int64_t(1) << sh) < x) ++sh;
      return sh;
    };
    const int bs_shift = shift_of(p.block_size), ch_shift = shift_of(p.D / 16);
    const int pt_shift = shift_of(static_cast<int64_t>(p.Hkv) * (p.D / 16));
    const unsigned blocks = static_cast<unsigned>((units + threads - 1) / threads);
    const uint32_t total = static_cast<uint32_t>(units);
    const int64_t row = static_cast<int64_t>(p.Hkv) * p.D;
    bool dense = pt_shift >= 0 && ch_shift >= 0 && p.kc_st[2] == p.D && p.kc_st[1] == row &&
                 p.kc_st[0] == row * p.block_size;
    for (int i = 0; i < 4 && dense; ++i) dense = p.kc_st[i] == p.vc_st[i];
    for (int i = 0; i < 3 && dense; ++i) dense = p.k_st[i] == p.v_st[i];
    dense = dense && p.k_st[1] == p.D && p.k_st[0] == row;
    if (dense) {
      if (p.in_dtype == INT8KV_BF16) return launch_pdl(cache_write_vec_kernel<__nv_bfloat16, true>, blocks, threads, 0, stream, p, total, bs_shift, pt_shift, ch_shift);
      if (p.in_dtype == INT8KV_FP16) return launch_pdl(cache_write_vec_kernel<__half, true>, blocks, threads, 0, stream, p, total, bs_shift, pt_shift, ch_shift);
      return launch_pdl(cache_write_vec_kernel<float, true>, blocks, threads, 0, stream, p, total, bs_shift, pt_shift, ch_shift);
    }
    if (p.in_dtype == INT8KV_BF16) return launch_pdl(cache_write_vec_kernel<__nv_bfloat16, false>, blocks, threads, 0, stream, p, total, bs_shift, pt_shift, ch_shift);
    if (p.in_dtype == INT8KV_FP16) return launch_pdl(cache_write_vec_kernel<__half, false>, blocks, threads, 0, stream, p, total, bs_shift, pt_shift, ch_shift);
    return launch_pdl(cache_write_vec_kernel<float, false>, blocks, threads, 0, stream, p, total, bs_shift, pt_shift, ch_shift);
  } else {
    const int64_t work = p.T * p.Hkv * static_cast<int64_t>(p.D);
    int64_t blocks = (work + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(sm_count) * 32;  // grid-stride beyond 32 CTAs per SM
    if (blocks > cap) blocks = cap;
    cache_write_elem_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? INT8KV_OK : INT8KV_E_LAUNCH;
}

}  // namespace int8kv
