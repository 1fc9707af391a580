// NVFP4 dynamic block quantize: E2M1 codes (two per byte), E4M3 block scales written
// straight into the 128x4 swizzled layout the block-scaled tensor-core MMA reads, fp32
// global scale.  Fake-quantize and dequantize share the arithmetic.
//
// HBM-bound streaming kernel.  One thread owns one 16-element block: a single 256-bit
// load (bf16/fp16) brings it in, the block abs-max needs no cross-lane traffic, the 16
// codes leave as one 64-bit store, and four neighbouring lanes (four consecutive blocks
// of one row = one 4-byte word of the swizzled scale layout) merge their scale bytes with
// two shuffles into one 32-bit store.  A warp therefore reads 1 KiB and writes 256 B of
// codes + 32 B of scales per step, all fully coalesced.  The kernel is only HBM-bound if
// it issues few instructions per element (~14 issue slots per element are available at
// full bandwidth): divisions go through the shared-divisor sequence of exact_div.h, the
// grid is (row, chunk) so no index division is needed, and each lane has two loads in
// flight before it starts computing.
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

// Block16<T>: one 16-element block.  `Raw` is what a lane keeps in registers while its loads
// are in flight; `widen` turns it into 16 fp32 values.
template <typename T>
struct Block16;

template <>
struct Block16<__nv_bfloat16> {
  struct Raw { U32x8 w; };
  __device__ static __forceinline__ Raw load_raw(const __nv_bfloat16* p) { return Raw{ld_nc_256(p)}; }
  __device__ static __forceinline__ void widen(const Raw& r, float* f) {
    Elem<__nv_bfloat16>::unpack(make_uint4(r.w.v[0], r.w.v[1], r.w.v[2], r.w.v[3]), f);
    Elem<__nv_bfloat16>::unpack(make_uint4(r.w.v[4], r.w.v[5], r.w.v[6], r.w.v[7]), f + 8);
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
  struct Raw { U32x8 w; };
  __device__ static __forceinline__ Raw load_raw(const __half* p) { return Raw{ld_nc_256(p)}; }
  __device__ static __forceinline__ void widen(const Raw& r, float* f) {
    Elem<__half>::unpack(make_uint4(r.w.v[0], r.w.v[1], r.w.v[2], r.w.v[3]), f);
    Elem<__half>::unpack(make_uint4(r.w.v[4], r.w.v[5], r.w.v[6], r.w.v[7]), f + 8);
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
  struct Raw { U32x8 a, b; };
  __device__ static __forceinline__ Raw load_raw(const float* p) { return Raw{ld_nc_256(p), ld_nc_256(p + 8)}; }
  __device__ static __forceinline__ void widen(const Raw& r, float* f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r.a.v[i]), f[8 + i] = __uint_as_float(r.b.v[i]);
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

// eight fp32 -> eight E2M1 nibbles in one word (RNE, saturating), element 0 in the lowest nibble
__device__ __forceinline__ uint32_t pack8_e2m1(float a0, float a1, float a2, float a3, float a4, float a5, float a6, float a7) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(a0), "f"(a1), "f"(a2), "f"(a3), "f"(a4), "f"(a5), "f"(a6), "f"(a7));
  return r;
}

constexpr float kRcp6 = 0.16666667163372039794921875f;   // RN(1/6)
constexpr float kRcp448 = 0.002232142956927418708801269531f;  // RN(1/448)

// Per-launch constants of the scale computation: global scale, its reciprocal, and whether
// the shared-divisor sequence may be used for divisions by it.
struct GlobalScale {
  float g, yg;
  bool fast;
  __device__ __forceinline__ explicit GlobalScale(float amax) {
    // (amax / 6) / 448 as exact IEEE quotients; the shared-divisor sequence is exact for a
    // numerator in the normal range away from its ends, anything else takes true divisions
    const uint32_t e = (__float_as_uint(amax) >> 23) & 0xffu;
    if (e >= 64u && e <= 190u) {
      g = b200q_div_by_shared(b200q_div_by_shared(amax, kE2M1Max, kRcp6), kE4M3Max, kRcp448);
    } else {
      g = nvfp4_global_from_amax(amax);
    }
    yg = b200q_rcp_rn(g);
    fast = b200q_div_fast_ok(g);
  }
};


// Quantize one block held in f[16]: returns the 8-bit scale, writes 16 codes as two words and
// the effective divisor d = fp32(scale) * global.
__device__ __forceinline__ uint32_t quantize_block(const float* f, const GlobalScale& gs, uint32_t& c_lo, uint32_t& c_hi,
                                                   float& d_out) {
  float m[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) m[i] = fmaxf(fabsf(f[2 * i]), fabsf(f[2 * i + 1]));
  const float a = fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), fmaxf(fmaxf(m[4], m[5]), fmaxf(m[6], m[7])));
  // s = (a / 6) / g, both as exact IEEE quotients
  float s;
  if (gs.fast) {
    s = b200q_div_by_shared(b200q_div_by_shared(a, kE2M1Max, kRcp6), gs.g, gs.yg);
  } else {
    s = __fdiv_rn(__fdiv_rn(a, kE2M1Max), gs.g);
  }
  const bool clamped = s > kE4M3Max;
  const uint32_t sb = f32x2_to_e4m3x2(s, 0.0f) & 0xffu;  // saturates to 448
  const float d = __fmul_rn(e4m3_to_f32(sb), gs.g);
  d_out = d;
  if (sb != 0u && !clamped && b200q_div_fast_ok(d)) {
    // common case: |x| <= 6.5 d, so the quotient can neither overflow nor need a clamp
    const float y = b200q_rcp_rn(d);
    float q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = b200q_div_by_shared(f[i], d, y);
    c_lo = pack8_e2m1(q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7]);
    c_hi = pack8_e2m1(q[8], q[9], q[10], q[11], q[12], q[13], q[14], q[15]);
  } else if (sb != 0u) {
    // stored scale saturated at 448 (amax input below the data) or an extreme divisor:
    // true division on a numerator clamped to 8 d, which still saturates to +-6
    const float lim = __fmul_rn(d, 8.0f);
    float q[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) q[i] = with_sign_of(__fdiv_rn(fminf(fabsf(f[i]), lim), d), f[i]);
    c_lo = pack8_e2m1(q[0], q[1], q[2], q[3], q[4], q[5], q[6], q[7]);
    c_hi = pack8_e2m1(q[8], q[9], q[10], q[11], q[12], q[13], q[14], q[15]);
  } else {
    c_lo = 0u;
    c_hi = 0u;
  }
  return sb;
}

// FAKE = false: codes + swizzled scales.  FAKE = true: dequantized values in T.
// Grid: x = row, y = chunk of the row.  A warp covers U spans of 32 consecutive blocks
// (512 elements each); all U 256-bit loads of a lane are issued before any arithmetic.
template <typename T, bool FAKE, int U>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const T* __restrict__ x, const float* __restrict__ amax, uint8_t* __restrict__ codes,
                      uint8_t* __restrict__ sf, T* __restrict__ fake, float* __restrict__ gout, uint32_t cols,
                      uint32_t blocks_per_row, uint32_t col_tiles) {
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x;
  const uint32_t blk0 = ((blockIdx.y * (blockDim.x >> 5) + warp) * U) * 32u + lane;
  const T* xr = x + row * cols;
  typename Block16<T>::Raw raw[U];
#pragma unroll
  for (int u = 0; u < U; ++u)
    if (blk0 + u * 32u < blocks_per_row) raw[u] = Block16<T>::load_raw(xr + (blk0 + u * 32u) * 16u);
  const GlobalScale gs(__ldg(amax));
  if (gout != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *gout = gs.g;
  uint8_t* code_row = codes + row * (cols >> 1);
  uint8_t* sf_row = sf + ((row >> 7) * col_tiles) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const uint32_t blk = blk0 + u * 32u;
    const bool live = blk < blocks_per_row;
    uint32_t sb = 0u, c_lo = 0u, c_hi = 0u;
    float d = 0.0f;
    if (live) {
      float f[16];
      Block16<T>::widen(raw[u], f);
      sb = quantize_block(f, gs, c_lo, c_hi, d);
    }
    if constexpr (!FAKE) {
      if (live) *reinterpret_cast<uint2*>(code_row + blk * 8u) = make_uint2(c_lo, c_hi);
      uint32_t w = sb << (8u * (lane & 3u));
      w |= __shfl_xor_sync(0xffffffffu, w, 1);
      w |= __shfl_xor_sync(0xffffffffu, w, 2);
      if ((lane & 3u) == 0u && live) *reinterpret_cast<uint32_t*>(sf_row + (blk >> 2) * 512u) = w;
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
        Block16<T>::store(fake + row * cols + blk * 16u, o);
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
  constexpr int U = sizeof(T) == 4 ? 2 : 4;  // 128 bytes of loads in flight per lane
  const uint32_t blocks_per_row = static_cast<uint32_t>(cols >> 4);
  const uint32_t spans_per_row = (blocks_per_row + 31u) >> 5;
  const uint32_t warps_needed = (spans_per_row + U - 1) / U;
  // up to 8 warps per CTA; short rows get smaller CTAs instead of idle warps
  const uint32_t warps = warps_needed < 8u ? warps_needed : 8u;
  const uint32_t chunks = (warps_needed + warps - 1) / warps;
  if (chunks > 65535u) return B200Q_ERR_INVALID;
  dim3 grid(static_cast<unsigned>(rows), chunks), block(warps * 32u);
  nvfp4_quantize_kernel<T, FAKE, U><<<grid, block, 0, st>>>(static_cast<const T*>(x), amax, codes, sf, static_cast<T*>(fake),
                                                             gout, static_cast<uint32_t>(cols), blocks_per_row,
                                                             (blocks_per_row + 3u) >> 2);
  return check_launch();
}

int validate(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax) {
  if (rows < 0 || cols < 0) return B200Q_ERR_INVALID;
  if (rows == 0 || cols == 0) return B200Q_OK;  // empty tensors are a valid no-op, whatever the pointers
  if (x == nullptr || amax == nullptr) return B200Q_ERR_INVALID;
  if (dtype != B200Q_F32 && dtype != B200Q_F16 && dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (cols % 16 != 0 || rows > 0x7fffffffLL || cols > 0x7fffffffLL) return B200Q_ERR_INVALID;
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
