// NVFP4 dynamic block quantize: E2M1 codes (two per byte), E4M3 block scales written
// straight into the 128x4 swizzled layout the block-scaled tensor-core MMA reads, fp32
// global scale.  Fake-quantize and dequantize share the arithmetic.
//
// HBM-bound streaming kernel.  One thread owns one 16-element block: a single 256-bit
// load (bf16/fp16) brings it in, the block abs-max needs no cross-lane traffic, the 16
// codes leave as one 64-bit store, and four neighbouring lanes (four consecutive blocks
// of one row = one 4-byte word of the swizzled scale layout) merge their scale bytes with
// two shuffles into one 32-bit store.  A warp therefore reads 1 KiB and writes 256 B of
// codes + 32 B of scales per step, all fully coalesced.
//
// Arithmetic contract (identical to the CPU restatement the tests compare against):
//   global = (amax / 6) / 448, 0 -> 1
//   s_blk  = e4m3_rne(min((amax_blk / 6) / global, 448));  d = fp32(s_blk) * global
//   code   = e2m1_rne_sat(x_fp32 / d); all codes of a block with s_blk == 0 are 0
//   x_hat  = e2m1 * d, rounded (RNE) to the input dtype.
#include "common.cuh"

namespace b200q {
namespace {

constexpr int kThreads = 256;

template <typename T>
struct Block16;

template <>
struct Block16<__nv_bfloat16> {
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    U32x8 w = ld_nc_256(p);
    Elem<__nv_bfloat16>::unpack(make_uint4(w.v[0], w.v[1], w.v[2], w.v[3]), f);
    Elem<__nv_bfloat16>::unpack(make_uint4(w.v[4], w.v[5], w.v[6], w.v[7]), f + 8);
  }
  __device__ static __forceinline__ void store(__nv_bfloat16* p, const float* f) {
    U32x8 w;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w.v[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_256(p, w);
  }
};

template <>
struct Block16<__half> {
  __device__ static __forceinline__ void load(const __half* p, float* f) {
    U32x8 w = ld_nc_256(p);
    Elem<__half>::unpack(make_uint4(w.v[0], w.v[1], w.v[2], w.v[3]), f);
    Elem<__half>::unpack(make_uint4(w.v[4], w.v[5], w.v[6], w.v[7]), f + 8);
  }
  __device__ static __forceinline__ void store(__half* p, const float* f) {
    U32x8 w;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w.v[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_256(p, w);
  }
};

template <>
struct Block16<float> {
  __device__ static __forceinline__ void load(const float* p, float* f) {
    U32x8 a = ld_nc_256(p), b = ld_nc_256(p + 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(a.v[i]), f[8 + i] = __uint_as_float(b.v[i]);
  }
  __device__ static __forceinline__ void store(float* p, const float* f) {
    U32x8 a, b;
#pragma unroll
    for (int i = 0; i < 8; ++i) a.v[i] = __float_as_uint(f[i]), b.v[i] = __float_as_uint(f[8 + i]);
    st_256(p, a);
    st_256(p + 8, b);
  }
};

// byte offset of the 4-byte scale word holding scale columns [4*(c/4), 4*(c/4)+4) of row r
__device__ __forceinline__ int64_t swizzled_word_offset(int64_t r, int64_t c, int64_t col_tiles) {
  const int64_t tile = (r >> 7) * col_tiles + (c >> 2);
  return tile * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4;
}

// Quantize one block held in f[16]: returns the 8-bit scale, writes 16 codes as two words.
__device__ __forceinline__ uint32_t quantize_block(const float* f, float g, uint32_t& c_lo, uint32_t& c_hi, float& d_out) {
  float a = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) a = fmaxf(a, fabsf(f[i]));
  const float s = fminf(__fdiv_rn(__fdiv_rn(a, kE2M1Max), g), kE4M3Max);
  const uint32_t sb = f32x2_to_e4m3x2(s, 0.0f) & 0xffu;
  const float d = __fmul_rn(e4m3_to_f32(sb), g);
  d_out = d;
  c_lo = 0u;
  c_hi = 0u;
  if (sb != 0u) {
    const SharedDivisor dv(d);
    const float lim = __fmul_rn(d, 8.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      c_lo |= f32x2_to_e2m1x2(dv.div(f[2 * i], lim), dv.div(f[2 * i + 1], lim)) << (8 * i);
      c_hi |= f32x2_to_e2m1x2(dv.div(f[8 + 2 * i], lim), dv.div(f[8 + 2 * i + 1], lim)) << (8 * i);
    }
  }
  return sb;
}

// FAKE = false: codes + swizzled scales.  FAKE = true: dequantized values in T.
// One warp covers 32 consecutive blocks (512 elements) of one row per step.
template <typename T, bool FAKE>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const T* __restrict__ x, const float* __restrict__ amax, uint8_t* __restrict__ codes,
                      uint8_t* __restrict__ sf, T* __restrict__ fake, float* __restrict__ gout, int64_t rows,
                      int64_t cols, int64_t spans_per_row, int64_t total_spans) {
  const float g = nvfp4_global_from_amax(__ldg(amax));
  if (gout != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *gout = g;
  const int lane = threadIdx.x & 31;
  const int64_t blocks_per_row = cols >> 4;
  const int64_t col_tiles = (blocks_per_row + 3) >> 2;
  const int64_t warp0 = (blockIdx.x * (int64_t)kThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kThreads) >> 5;
  for (int64_t span = warp0; span < total_spans; span += nwarps) {
    const int64_t row = span / spans_per_row;
    const int64_t blk = (span - row * spans_per_row) * 32 + lane;
    const bool live = blk < blocks_per_row;
    float f[16];
    uint32_t sb = 0u, c_lo = 0u, c_hi = 0u;
    float d = 0.0f;
    if (live) {
      Block16<T>::load(x + row * cols + blk * 16, f);
      sb = quantize_block(f, g, c_lo, c_hi, d);
    }
    if constexpr (!FAKE) {
      if (live) *reinterpret_cast<uint2*>(codes + row * (cols >> 1) + blk * 8) = make_uint2(c_lo, c_hi);
      uint32_t w = sb << (8 * (lane & 3));
      w |= __shfl_xor_sync(0xffffffffu, w, 1);
      w |= __shfl_xor_sync(0xffffffffu, w, 2);
      if ((lane & 3) == 0 && live) *reinterpret_cast<uint32_t*>(sf + swizzled_word_offset(row, blk, col_tiles)) = w;
    } else {
      if (live) {
        float o[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 p = e2m1x2_to_f32x2((c_lo >> (8 * i)) & 0xffu);
          o[2 * i] = __fmul_rn(p.x, d), o[2 * i + 1] = __fmul_rn(p.y, d);
          p = e2m1x2_to_f32x2((c_hi >> (8 * i)) & 0xffu);
          o[8 + 2 * i] = __fmul_rn(p.x, d), o[8 + 2 * i + 1] = __fmul_rn(p.y, d);
        }
        Block16<T>::store(fake + row * cols + blk * 16, o);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
nvfp4_dequantize_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf, const float* __restrict__ gptr,
                        T* __restrict__ out, int64_t rows, int64_t cols) {
  const float g = __ldg(gptr);
  const int64_t blocks_per_row = cols >> 4;
  const int64_t col_tiles = (blocks_per_row + 3) >> 2;
  const int64_t total = rows * blocks_per_row;
  for (int64_t b = blockIdx.x * (int64_t)kThreads + threadIdx.x; b < total; b += (int64_t)gridDim.x * kThreads) {
    const int64_t row = b / blocks_per_row, blk = b - row * blocks_per_row;
    const uint32_t sb = sf[swizzled_word_offset(row, blk, col_tiles) + (blk & 3)];
    const float d = __fmul_rn(e4m3_to_f32(sb), g);
    const uint2 c = *reinterpret_cast<const uint2*>(codes + b * 8);
    float o[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 p = e2m1x2_to_f32x2((c.x >> (8 * i)) & 0xffu);
      o[2 * i] = __fmul_rn(p.x, d), o[2 * i + 1] = __fmul_rn(p.y, d);
      p = e2m1x2_to_f32x2((c.y >> (8 * i)) & 0xffu);
      o[8 + 2 * i] = __fmul_rn(p.x, d), o[8 + 2 * i + 1] = __fmul_rn(p.y, d);
    }
    Block16<T>::store(out + b * 16, o);
  }
}

template <typename T, bool FAKE>
int launch(const void* x, const float* amax, uint8_t* codes, uint8_t* sf, void* fake, float* gout, int64_t rows,
           int64_t cols, cudaStream_t st) {
  const int64_t blocks_per_row = cols >> 4;
  const int64_t spans_per_row = (blocks_per_row + 31) >> 5;
  const int64_t total_spans = rows * spans_per_row;
  const int64_t warps_per_cta = kThreads / 32;
  int64_t ctas = (total_spans + warps_per_cta - 1) / warps_per_cta;
  // a few steps per warp keep several 256-bit loads in flight per SM without a tail
  const int64_t cap = (int64_t)sm_count() * 8 * 8;
  if (ctas > cap) ctas = cap;
  nvfp4_quantize_kernel<T, FAKE><<<static_cast<unsigned>(ctas), kThreads, 0, st>>>(
      static_cast<const T*>(x), amax, codes, sf, static_cast<T*>(fake), gout, rows, cols, spans_per_row, total_spans);
  return check_launch();
}

int validate(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax) {
  if (rows < 0 || cols < 0) return B200Q_ERR_INVALID;
  if (rows == 0 || cols == 0) return B200Q_OK;  // empty tensors are a valid no-op, whatever the pointers
  if (x == nullptr || amax == nullptr) return B200Q_ERR_INVALID;
  if (dtype != B200Q_F32 && dtype != B200Q_F16 && dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (cols % 16 != 0) return B200Q_ERR_INVALID;
  if (!aligned(x, 32)) return B200Q_ERR_ALIGN;
  return B200Q_OK;
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

size_t b200q_nvfp4_scale_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  const int64_t rt = (rows + 127) / 128, ct = (cols / 16 + 3) / 4;
  return static_cast<size_t>(rt * ct * 512);
}

int b200q_nvfp4_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax, uint8_t* codes_out,
                         uint8_t* scales_out, float* global_scale_out, b200q_stream_t stream) {
  if (int rc = validate(x, dtype, rows, cols, amax)) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  if (codes_out == nullptr || scales_out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(codes_out, 8) || !aligned(scales_out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // rows that only exist as padding of the last 128-row tile are never visited by the
  // kernel: clear the last row tile first so the padding reads as zero.
  if (rows % 128 != 0) {
    const int64_t ct = (cols / 16 + 3) / 4;
    const int64_t last = (rows / 128) * ct * 512;
    if (cudaMemsetAsync(scales_out + last, 0, static_cast<size_t>(ct * 512), st) != cudaSuccess) return B200Q_ERR_CUDA;
  }
  switch (dtype) {
    case B200Q_BF16: return launch<__nv_bfloat16, false>(x, amax, codes_out, scales_out, nullptr, global_scale_out, rows, cols, st);
    case B200Q_F16: return launch<__half, false>(x, amax, codes_out, scales_out, nullptr, global_scale_out, rows, cols, st);
    default: return launch<float, false>(x, amax, codes_out, scales_out, nullptr, global_scale_out, rows, cols, st);
  }
}

int b200q_nvfp4_fake_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax, void* out,
                              b200q_stream_t stream) {
  if (int rc = validate(x, dtype, rows, cols, amax)) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  if (out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(out, 32)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200Q_BF16: return launch<__nv_bfloat16, true>(x, amax, nullptr, nullptr, out, nullptr, rows, cols, st);
    case B200Q_F16: return launch<__half, true>(x, amax, nullptr, nullptr, out, nullptr, rows, cols, st);
    default: return launch<float, true>(x, amax, nullptr, nullptr, out, nullptr, rows, cols, st);
  }
}

int b200q_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales_swizzled, const float* global_scale, int64_t rows,
                           int64_t cols, void* out, int dtype, b200q_stream_t stream) {
  if (codes == nullptr || scales_swizzled == nullptr || global_scale == nullptr || out == nullptr || rows < 0 || cols < 0 ||
      cols % 16 != 0)
    return B200Q_ERR_INVALID;
  if (!aligned(codes, 8) || !aligned(out, 32)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * (cols >> 4);
  int64_t ctas = (total + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (ctas > cap) ctas = cap;
  const unsigned grid = static_cast<unsigned>(ctas);
  switch (dtype) {
    case B200Q_BF16: nvfp4_dequantize_kernel<<<grid, kThreads, 0, st>>>(codes, scales_swizzled, global_scale, static_cast<__nv_bfloat16*>(out), rows, cols); break;
    case B200Q_F16: nvfp4_dequantize_kernel<<<grid, kThreads, 0, st>>>(codes, scales_swizzled, global_scale, static_cast<__half*>(out), rows, cols); break;
    case B200Q_F32: nvfp4_dequantize_kernel<<<grid, kThreads, 0, st>>>(codes, scales_swizzled, global_scale, static_cast<float*>(out), rows, cols); break;
    default: return B200Q_ERR_INVALID;
  }
  return check_launch();
}

}  // extern "C"
