// Shared device helpers for the sm_100a paged-KV kernels: PTX wrappers for TMA tile loads,
// mbarrier pipelines with bounded waits, warp-level tensor-core MMA, and dtype conversion.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <cstring>
#include <utility>

#include "../../include/int8kv_b200.h"
#include "kernels.h"

namespace int8kv {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// ---------------------------------------------------------------------------------------------
// dtype helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_as_float(const void* base, int dtype, int64_t idx) {
  if (dtype == INT8KV_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  if (dtype == INT8KV_FP16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return reinterpret_cast<const float*>(base)[idx];
}

__device__ __forceinline__ void store_from_float(void* base, int dtype, int64_t idx, float v) {
  if (dtype == INT8KV_BF16) reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
  else if (dtype == INT8KV_FP16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else reinterpret_cast<float*>(base)[idx] = v;
}

__device__ __forceinline__ int64_t load_index(const void* base, int is_i64, int64_t idx) {
  return is_i64 ? reinterpret_cast<const int64_t*>(base)[idx]
                : static_cast<int64_t>(reinterpret_cast<const int32_t*>(base)[idx]);
}

// Four consecutive elements -> floats: one vector load when contiguous and aligned (a scalar load per element with
// its own dtype branch keeps the compiler from overlapping the loads).
__device__ __forceinline__ void load4_as_float(const void* base, int dtype, int64_t off, int64_t stride, float (&x)[4]) {
  const int esz = dtype == INT8KV_FP32 ? 4 : 2;
  const char* ptr = reinterpret_cast<const char*>(base) + off * esz;
  if (stride == 1 && (reinterpret_cast<uintptr_t>(ptr) & static_cast<uintptr_t>(4 * esz - 1)) == 0) {
    if (dtype == INT8KV_FP32) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(ptr));
      x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(ptr));
      float2 lo, hi;
      if (dtype == INT8KV_BF16) {
        lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
        hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
      } else {
        lo = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        hi = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
      }
      x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = load_as_float(base, dtype, off + i * stride);
  }
}

// 32 consecutive elements of a float tensor starting at element `off` (element stride `stride`) -> floats;
// 16-byte vector loads when the run is contiguous and aligned.  Any other layout goes element by element through
// `scratch` (shared memory, 128 bytes per lane, free at the time of the call) in a loop that is not unrolled: the
// rare path then costs a few dozen instructions of code instead of several hundred.
__device__ __forceinline__ void load32_as_float(const void* base, int dtype, int64_t off, int64_t stride, float (&x)[32],
                                                uint32_t scratch, int lane) {
  const int esz = dtype == INT8KV_FP32 ? 4 : 2;
  const char* ptr = reinterpret_cast<const char*>(base) + off * esz;
  if (stride == 1 && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) {
    if (dtype == INT8KV_FP32) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(ptr) + i);
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(ptr) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f;
          if (dtype == INT8KV_BF16) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
          else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
          x[8 * i + 2 * j] = f.x;
          x[8 * i + 2 * j + 1] = f.y;
        }
      }
    }
  } else {
    const uint32_t mine = scratch + lane * 128;
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      const float v = load_as_float(base, dtype, off + i * stride);
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(mine + 4 * i), "f"(v) : "memory");
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 v;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(mine + 16 * i) : "memory");
      x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
  }
}

// 16 consecutive output elements from floats; 16-byte vector stores when contiguous and aligned, else element by
// element through `scratch` (shared memory, 64 bytes per lane) in a rolled loop.
__device__ __forceinline__ void store16_from_float(void* base, int dtype, int64_t off, int64_t stride, const float (&x)[16],
                                                   uint32_t scratch, int lane) {
  const int esz = dtype == INT8KV_FP32 ? 4 : 2;
  char* ptr = reinterpret_cast<char*>(base) + off * esz;
  if (stride == 1 && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) {
    if (dtype == INT8KV_FP32) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        reinterpret_cast<float4*>(ptr)[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
    } else {
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (dtype == INT8KV_BF16) {
          __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
          w[i] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
          w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      reinterpret_cast<uint4*>(ptr)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(ptr)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
  } else {
    const uint32_t mine = scratch + lane * 64;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(mine + 16 * i), "f"(x[4 * i]), "f"(x[4 * i + 1]),
                   "f"(x[4 * i + 2]), "f"(x[4 * i + 3])
                   : "memory");
#pragma unroll 1
    for (int i = 0; i < 16; ++i) {
      float v;
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(mine + 4 * i) : "memory");
      store_from_float(base, dtype, off + i * stride, v);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// static INT8 quantisation shared by the cache-write kernels and the fused decode step
// ---------------------------------------------------------------------------------------------
// rint(x / scale) clamped to [-127, 127], bit-identical to IEEE division followed by round-half-even, at
// the cost of a few full-rate FP32 instructions in the common case:
//  * x * (1/scale) is within 2 ulp of the true quotient; its rounding to an integer can differ from that of
//    the correctly rounded quotient only when the quotient is within a few ulp of a tie k + 0.5 (ulp <= 2^-17
//    below 128), so exactly those elements — and anything huge, infinite or NaN — take the real division;
//  * rounding uses the 1.5 * 2^23 trick (adding and subtracting it rounds to nearest-even in the FP32 adder,
//    and the integer sits in the low mantissa bits), which keeps the work off the quarter-rate conversion unit.
// Returns the integer still unclamped for |n| < 2^22; the caller saturates when packing.
constexpr float kRoundMagic = 12582912.f;           // 1.5 * 2^23
constexpr int kRoundMagicBits = 0x4B400000;

__device__ __forceinline__ int quant1(float x, float scale, float rscale) {
  float q = x * rscale;
  float t = q + kRoundMagic;
  const float n = t - kRoundMagic;
  if (!(fabsf(q - n) < 0.5f - 6.2e-5f) || !(fabsf(q) < 4.0e6f)) {  // near a tie, beyond 2^22, infinite or NaN
    q = x / scale;                          // div.rn.f32
    q = fminf(fmaxf(q, -127.f), 127.f);     // also maps +-inf; NaN is handled below
    t = q + kRoundMagic;
    if (x != x) t = kRoundMagic;            // NaN -> 0, as a float-to-int8 cast of NaN gives on the CPU
  }
  return __float_as_int(t) - kRoundMagicBits;
}

// One element of the dynamic scheme and of the optional INT8 query: clamp(x / scale, +-127) rounded half away from zero, bit-identical to the
// fp32 sequence divide, clamp, floor(q + 0.5) / ceil(q - 0.5).  Away from a tie, rounding half away equals rounding
// to nearest, which the 1.5 * 2^23 addition does on a quotient formed with the reciprocal; within 1e-3 of a
// half-integer (where the few ulp between that quotient and the IEEE one could decide, and where the two rounding
// rules differ) the division and the reference sequence itself run.  The integer is returned unclamped; packing
// saturates it, which equals clamping the quotient first.
__device__ __forceinline__ int quant_half_away(float x, float scale, float rscale) {
  float q = x * rscale;
  const float t = q + kRoundMagic;
  const float n = t - kRoundMagic;
  if (!(fabsf(q - n) < 0.5f - 1e-3f) || !(fabsf(q) < 4.0e6f)) {
    q = fminf(fmaxf(__fdiv_rn(x, scale), -127.f), 127.f);
    const float r = q >= 0.f ? floorf(q + 0.5f) : ceilf(q - 0.5f);
    return x != x ? 0 : static_cast<int>(r);
  }
  return __float_as_int(t) - kRoundMagicBits;
}

// Four such integers saturated to int8 and packed little-endian; -128 is raised to -127.
__device__ __forceinline__ uint32_t pack4_sat(int n0, int n1, int n2, int n3) {
  uint32_t hi, w;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(n3), "r"(n2), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(n1), "r"(n0), "r"(hi));
  return __vmaxs4(w, 0x81818181u);
}

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may start while
// its predecessor drains; it must pass grid_dependency_wait() before touching memory the predecessor wrote.
// Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// INT8KV_PDL=0 in the environment turns programmatic dependent launch off (read once).
inline bool pdl_enabled() {
  static const bool on = []() {
    const char* e = std::getenv("INT8KV_PDL");
    return e == nullptr || std::atoi(e) != 0;
  }();
  return on;
}

// Launch with the programmatic-stream-serialisation attribute: the grid may be scheduled while the previous
// kernel in the stream drains; every kernel here calls grid_dependency_wait() before its first global access.
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t stream,
                      Args&&... args) {
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...) == cudaSuccess ? INT8KV_OK : INT8KV_E_LAUNCH;
}

// Flags that another GPU writes into this GPU's memory (and the other way round) are read and written with
// system-scope acquire / release, so that the rows stored before a flag are visible to whoever sees the flag.
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Attempts of a wait for another GPU's flag: 100 ns to 1 us apart, so the limit gives up after about a second.
constexpr uint32_t kFlagSpinLimit = 1u << 20;

__host__ __device__ __forceinline__ int dtype_bytes(int dtype) { return dtype == INT8KV_FP32 ? 4 : 2; }

// ---------------------------------------------------------------------------------------------
// shared-memory address, mbarrier, TMA
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  // make the initialised barriers visible to the async (TMA) proxy
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Orders this thread's earlier ordinary writes to shared memory before later writes of the async proxy (TMA) to the
// same bytes: a ring stage that lanes have written by hand must be fenced by those lanes before it is refilled.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 4-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// The calling thread's earlier cp.async copies arrive on the barrier when they complete (the arrival was counted
// when the barrier was initialised).
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One attempt to observe the completion of a phase: the hardware may suspend the thread for up to
// `hint_ns` nanoseconds while the phase is pending, then returns whether it completed.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}

// Wait for a phase of `bar` with an attempt limit (a wait that cannot finish must not hang the GPU): each
// attempt suspends for at most about a microsecond, so the default limit gives up after roughly a second.
// Returns false when the limit ran out.
constexpr uint32_t kWaitSpinLimit = 1u << 20;
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = kWaitSpinLimit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity, 1000u)) return true;
  }
  return false;
}

// L2 policy for data that is read exactly once (the KV pages): first in line for eviction, so that streaming a
// cache many times the size of the L2 does not push out what is read again shortly (the partial rows that the
// merge kernel needs, block tables, sequence lengths).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

// One 4-D tile load global -> shared through the tensor map; completion is counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, uint64_t l2_policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(l2_policy)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a 128-byte-swizzled tile of 128-byte rows
// (tile base aligned to 1024 bytes): the chunk index is XORed with the row index modulo 8.
__device__ __forceinline__ uint32_t swz128(int row, int chunk) {
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// ---------------------------------------------------------------------------------------------
// tensor-core MMA m16n8k16 (fp32 accumulate) and fragment movement
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// INT8 tensor-core MMA m16n8k32, int32 accumulate: A rows x 32 signed bytes, B 32 signed bytes x 8 columns.
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Transpose an 8x8 matrix of 16-bit elements held one row-pair per lane (the C/ldmatrix fragment layout).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Two bytes of `w` (already XORed with 0x80, i.e. value+128 as unsigned) -> half2 of the signed values.
// 0x6400 | u is the fp16 number 1024 + u exactly; subtracting 1152 = 1024 + 128 leaves the int8 value.
__device__ __forceinline__ uint32_t u8pair_to_half2(uint32_t w, uint32_t sel) {
  uint32_t h = prmt(w, 0x64646464u, sel);
  const uint32_t bias = 0x64806480u;
  __half2 r = __hsub2(*reinterpret_cast<__half2*>(&h), *reinterpret_cast<const __half2*>(&bias));
  return *reinterpret_cast<uint32_t*>(&r);
}

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace int8kv
