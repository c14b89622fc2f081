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
#include "common.cuh"

namespace int8kv {

// rint(x / scale) clamped to [-127, 127], bit-identical to IEEE division followed by round-half-even, at
// the cost of one multiply in the common case.  x * (1/scale) is within 2 ulp of the true quotient; its
// rounding to an integer can only differ from that of the correctly rounded quotient when the quotient is
// within a few ulp of a tie k + 0.5 (ulp <= 2^-17 below 128), so exactly those elements — and anything
// huge, infinite or NaN — take the real division.
__device__ __forceinline__ int quant1(float x, float scale, float rscale) {
  float q = x * rscale;
  float n = rintf(q);
  if (!(fabsf(q - n) < 0.5f - 6.2e-5f)) {
    q = x / scale;  // div.rn.f32
    n = rintf(q);
  }
  n = fminf(fmaxf(n, -127.f), 127.f);
  return (x != x) ? 0 : static_cast<int>(n);
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

// 16 consecutive elements as raw 16-byte vectors (issued before anything depends on them) ...
template <typename T>
struct Raw16 {
  static constexpr int kVecs = 16 * sizeof(T) / 16;
  uint4 v[kVecs];
  __device__ __forceinline__ void load(const T* p) {
#pragma unroll
    for (int i = 0; i < kVecs; ++i) v[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
  }
  // ... and their float values
  __device__ __forceinline__ void to_float(float (&x)[16]) const {
    const T* e = reinterpret_cast<const T*>(v);
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = to_f32<T>(e[i]);
  }
};

__device__ __forceinline__ uint4 quant16(const float (&x)[16], float scale, float rscale) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t b0 = static_cast<uint32_t>(quant1(x[4 * i + 0], scale, rscale)) & 0xffu;
    uint32_t b1 = static_cast<uint32_t>(quant1(x[4 * i + 1], scale, rscale)) & 0xffu;
    uint32_t b2 = static_cast<uint32_t>(quant1(x[4 * i + 2], scale, rscale)) & 0xffu;
    uint32_t b3 = static_cast<uint32_t>(quant1(x[4 * i + 3], scale, rscale)) & 0xffu;
    w[i] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Vector path: D % 16 == 0, unit innermost strides, 16-byte aligned rows on both sides.
template <typename T>
__global__ void __launch_bounds__(256) cache_write_vec_kernel(const WriteParams p) {
  const int chunks = p.D >> 4;
  const int64_t per_token = static_cast<int64_t>(p.Hkv) * chunks;
  const int64_t total = p.T * per_token;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = idx / per_token;
    const int rem = static_cast<int>(idx - t * per_token);
    const int h = rem / chunks;
    const int c = rem - h * chunks;
    // the slot and the K/V vectors are independent loads: all are in flight before the first use
    const int64_t slot = load_index(p.slots, p.slot_is_i64, t);
    const T* kp = reinterpret_cast<const T*>(p.key) + t * p.k_st[0] + h * p.k_st[1] + c * 16;
    const T* vp = reinterpret_cast<const T*>(p.value) + t * p.v_st[0] + h * p.v_st[1] + c * 16;
    Raw16<T> kr, vr;
    kr.load(kp);
    vr.load(vp);
    const float ks = fmaxf(__ldg(p.k_scale + h), 1e-6f);
    const float vs = fmaxf(__ldg(p.v_scale + h), 1e-6f);
    if (slot < 0 || slot >= p.num_slots) continue;
    float kx[16], vx[16];
    kr.to_float(kx);
    vr.to_float(vx);
    const int64_t blk = slot / p.block_size;
    const int64_t off = slot - blk * p.block_size;
    int8_t* kd = p.kc + blk * p.kc_st[0] + off * p.kc_st[1] + h * p.kc_st[2] + c * 16;
    int8_t* vd = p.vc + blk * p.vc_st[0] + off * p.vc_st[1] + h * p.vc_st[2] + c * 16;
    *reinterpret_cast<uint4*>(kd) = quant16(kx, ks, __frcp_rn(ks));
    *reinterpret_cast<uint4*>(vd) = quant16(vx, vs, __frcp_rn(vs));
  }
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
    p.kc[blk * p.kc_st[0] + off * p.kc_st[1] + h * p.kc_st[2] + d * p.kc_st[3]] = static_cast<int8_t>(quant1(kx, ks, __frcp_rn(ks)));
    p.vc[blk * p.vc_st[0] + off * p.vc_st[1] + h * p.vc_st[2] + d * p.vc_st[3]] = static_cast<int8_t>(quant1(vx, vs, __frcp_rn(vs)));
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int launch_cache_write(const WriteParams& p, int sm_count, cudaStream_t stream) {
  if (p.T == 0) return INT8KV_OK;
  const int esz = dtype_bytes(p.in_dtype);
  const int per16 = 16 / esz;  // elements per 16 bytes
  bool vec = (p.D % 16 == 0) && p.k_st[2] == 1 && p.v_st[2] == 1 && p.kc_st[3] == 1 && p.vc_st[3] == 1 &&
             aligned16(p.key) && aligned16(p.value) && aligned16(p.kc) && aligned16(p.vc);
  for (int i = 0; i < 2 && vec; ++i) vec = (p.k_st[i] % per16 == 0) && (p.v_st[i] % per16 == 0);
  for (int i = 0; i < 3 && vec; ++i) vec = (p.kc_st[i] % 16 == 0) && (p.vc_st[i] % 16 == 0);
  const int threads = 256;
  const int64_t work = vec ? p.T * p.Hkv * (p.D / 16) : p.T * p.Hkv * static_cast<int64_t>(p.D);
  int64_t blocks = (work + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(sm_count) * 32;  // grid-stride beyond 32 CTAs per SM
  if (blocks > cap) blocks = cap;
  if (vec) {
    if (p.in_dtype == INT8KV_BF16) cache_write_vec_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(p);
    else if (p.in_dtype == INT8KV_FP16) cache_write_vec_kernel<__half><<<blocks, threads, 0, stream>>>(p);
    else cache_write_vec_kernel<float><<<blocks, threads, 0, stream>>>(p);
  } else {
    cache_write_elem_kernel<<<blocks, threads, 0, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? INT8KV_OK : INT8KV_E_LAUNCH;
}

}  // namespace int8kv
