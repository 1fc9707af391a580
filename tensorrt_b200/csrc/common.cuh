// Shared device helpers for the b200q kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200q.h"
#include "exact_div.h"

namespace b200q {

constexpr float kE4M3Max = 448.0f;
constexpr float kE2M1Max = 6.0f;

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? B200Q_OK : B200Q_ERR_CUDA;
}

// Programmatic dependent launch.  A kernel launched through `launch_pdl` may start while the kernel
// before it on the stream is still running, once every CTA of that kernel has called
// `pdl_launch_dependents()` (or exited).  It must call `pdl_wait()` before it touches global
// memory that an earlier kernel may still read or write; the wait returns when the preceding
// kernel has completed and its writes are visible.  Kernels that do neither behave as usual.
bool pdl_enabled();  // environment variable B200Q_PDL, default on

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// fused_ops.cu: dynamic per-token FP8 quantize of many long bf16 rows by persistent CTAs fed through a
// shared-memory ring; 1 = shape does not qualify, else a B200Q status.
#ifdef __CUDACC__
int launch_fp8_rows_stream(const __nv_bfloat16* x, uint8_t* codes, float* scales, int64_t rows, int64_t cols, cudaStream_t st);
#endif

// Device must be compute capability 10.x; cached per device.
int check_arch();
int sm_count();

// ---------------------------------------------------------------- global memory vectors
struct alignas(32) U32x8 {
  uint32_t v[8];
};

__device__ __forceinline__ U32x8 ld_nc_256(const void* p) {
  U32x8 r;
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]),
                 "=r"(r.v[6]), "=r"(r.v[7])
               : "l"(p));
  return r;
}

__device__ __forceinline__ uint4 ld_nc_128(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ void st_256(void* p, const U32x8& r) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.v[0]), "r"(r.v[1]),
               "r"(r.v[2]), "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7])
               : "memory");
}

// ---------------------------------------------------------------- element types
// Elem<T>::load8 reads 8 consecutive elements (16-byte aligned for 2-byte types,
// 32-byte aligned for float) and widens them to fp32; store8 narrows with RNE.
template <typename T>
struct Elem;

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kDtype = B200Q_BF16;
  __device__ static __forceinline__ void unpack(const uint4& w, float* f) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  }
  __device__ static __forceinline__ void load8(const __nv_bfloat16* p, float* f) { unpack(ld_nc_128(p), f); }
  __device__ static __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
    uint4 w;
    uint32_t* u = &w.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = w;
  }
};

template <>
struct Elem<__half> {
  static constexpr int kDtype = B200Q_F16;
  __device__ static __forceinline__ void unpack(const uint4& w, float* f) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static __forceinline__ void load8(const __half* p, float* f) { unpack(ld_nc_128(p), f); }
  __device__ static __forceinline__ void store8(__half* p, const float* f) {
    uint4 w;
    uint32_t* u = &w.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = w;
  }
};

template <>
struct Elem<float> {
  static constexpr int kDtype = B200Q_F32;
  __device__ static __forceinline__ void load8(const float* p, float* f) {
    uint4 a = ld_nc_128(p), b = ld_nc_128(p + 4);
    f[0] = __uint_as_float(a.x), f[1] = __uint_as_float(a.y), f[2] = __uint_as_float(a.z), f[3] = __uint_as_float(a.w);
    f[4] = __uint_as_float(b.x), f[5] = __uint_as_float(b.y), f[6] = __uint_as_float(b.z), f[7] = __uint_as_float(b.w);
  }
  __device__ static __forceinline__ void store8(float* p, const float* f) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// ---------------------------------------------------------------- number formats
// two fp32 -> two E4M3 bytes (RNE, saturate to +-448); low byte = a.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float a, float b) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(b), "f"(a));
  return r;
}

// two E4M3 bytes (low 16 bits) -> two fp32; exact.
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t v) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(static_cast<uint16_t>(v)));
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

__device__ __forceinline__ float e4m3_to_f32(uint32_t code) { return e4m3x2_to_f32x2(code & 0xffu).x; }

// two fp32 -> two E2M1 nibbles in one byte (RNE, saturate to +-6); low nibble = a.
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float a, float b) {
  uint32_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}" : "=r"(r) : "f"(b), "f"(a));
  return r;
}

// one byte holding two E2M1 nibbles -> two fp32; exact.
__device__ __forceinline__ float2 e2m1x2_to_f32x2(uint32_t byte) {
  uint32_t h;
  asm("{\n\t.reg .b8 t;\n\tcvt.u8.u32 t, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h) : "r"(byte));
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

// copysign(mag >= 0, sign source)
__device__ __forceinline__ float with_sign_of(float mag, float src) {
  return __uint_as_float((__float_as_uint(mag) & 0x7fffffffu) | (__float_as_uint(src) & 0x80000000u));
}

// Quotient x / d by one of three routes, all bit-identical to IEEE division wherever the
// result can influence a code:
//   kDivFast     shared-divisor sequence on the signed numerator; needs b200q_div_fast_ok(d)
//                and a quotient that cannot overflow (|x| bounded by a multiple of d)
//   kDivClamped  same, on |x| clamped to `lim` (any value whose quotient already saturates),
//                sign restored afterwards; for numerators that may be arbitrarily large
//   kDivTrue     IEEE division on the clamped numerator; for extreme divisors
enum DivPath { kDivFast = 0, kDivClamped = 1, kDivTrue = 2 };

template <int PATH>
__device__ __forceinline__ float div_path(float x, float d, float y, float lim) {
  if constexpr (PATH == kDivFast) {
    return b200q_div_by_shared(x, d, y);
  } else if constexpr (PATH == kDivClamped) {
    return with_sign_of(b200q_div_by_shared(fminf(fabsf(x), lim), d, y), x);
  } else {
    return with_sign_of(__fdiv_rn(fminf(fabsf(x), lim), d), x);
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the CTA (THREADS threads); `smem` holds THREADS / 32 floats and is free again on return.
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (lane < THREADS / 32) ? smem[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

// silu(a) * b = a / (1 + exp(-a)) * b with the hardware exponential and reciprocal (a few ulp in fp32,
// below the bf16 rounding that follows).  Every kernel that applies the activation uses exactly this
// expression, so the fused and the separate forms give the same bits.
__device__ __forceinline__ float silu_mul_f32(float a, float b) { return __fdividef(a, 1.0f + __expf(-a)) * b; }

// fp8 scale from amax: amax / 448, zero -> 1 (true division, as the CPU restatement).
__device__ __forceinline__ float fp8_scale_from_amax(float amax) {
  float s = __fdiv_rn(amax, kE4M3Max);
  return s == 0.0f ? 1.0f : s;
}

__device__ __forceinline__ float nvfp4_global_from_amax(float amax) {
  float g = __fdiv_rn(__fdiv_rn(amax, kE2M1Max), kE4M3Max);
  return g == 0.0f ? 1.0f : g;
}

}  // namespace b200q
