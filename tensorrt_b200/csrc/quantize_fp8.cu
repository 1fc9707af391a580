// FP8 E4M3 quantize / fake-quantize / dequantize and the abs-max reductions.
//
// All kernels are HBM-bound streaming kernels: 128-bit coalesced loads, warp-shuffle
// abs-max reductions, the row kept in registers between the amax pass and the quantize
// pass so that every input byte is read from DRAM once.
//
// Arithmetic contract (identical to the CPU restatement the tests compare against):
//   scale = amax / 448 (fp32 division; 0 -> 1)
//   code  = e4m3_rne_sat(x_fp32 / scale)
//   fake-quant output = fp32(code) * scale, rounded (RNE) to the input dtype.
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace b200q {

namespace {

constexpr int kRowThreads = 256;
constexpr int kMaxItems = 8;  // 8-element groups a thread keeps in registers between the two passes

// ---------------------------------------------------------------- block reduce
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* smem) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = (lane < THREADS / 32) ? smem[lane] : 0.0f;
  r = warp_max(r);
  __syncthreads();
  return r;
}

// ---------------------------------------------------------------- row kernels
enum class Out { Codes, Fake };

// One CTA per row.  ITEMS groups of 8 elements per thread stay in registers when the row
// fits (cols <= THREADS * 8 * ITEMS); otherwise (ITEMS == 0) the row is streamed twice and
// the second pass hits L2.
//   AMAX_MODE 0: dynamic (reduce the row), 1: amax[0], 2: amax[row]
template <typename T, int ITEMS, int AMAX_MODE, Out OUT>
__global__ void __launch_bounds__(kRowThreads)
fp8_rows_kernel(const T* __restrict__ x, const float* __restrict__ amax, uint8_t* __restrict__ codes,
                T* __restrict__ fake, float* __restrict__ scales, int64_t rows, int64_t cols) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  const int groups = static_cast<int>(cols >> 3);

  float v[ITEMS > 0 ? ITEMS : 1][8];
  float local = 0.0f;
  if constexpr (ITEMS > 0) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kRowThreads;
      if (g < groups) {
        Elem<T>::load8(xr + (int64_t)g * 8, v[i]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
      }
    }
    if constexpr (AMAX_MODE == 0) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) local = fmaxf(local, fabsf(v[i][j]));
    }
  } else if constexpr (AMAX_MODE == 0) {
    for (int g = threadIdx.x; g < groups; g += kRowThreads) {
      float t[8];
      Elem<T>::load8(xr + (int64_t)g * 8, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) local = fmaxf(local, fabsf(t[j]));
    }
  }

  float a;
  if constexpr (AMAX_MODE == 0) {
    a = block_max<kRowThreads>(local, red);
  } else if constexpr (AMAX_MODE == 1) {
    a = __ldg(amax);
  } else {
    a = __ldg(amax + row);
  }
  const float scale = fp8_scale_from_amax(a);
  if (threadIdx.x == 0 && scales != nullptr && (AMAX_MODE != 1 || row == 0)) scales[AMAX_MODE == 1 ? 0 : row] = scale;

  const float y = b200q_rcp_rn(scale);
  const float lim = __fmul_rn(scale, 512.0f);  // |x| >= 512 * scale saturates to 448 anyway
  // With the amax reduced in this kernel every quotient is <= 448 (1 + 2^-23) and the plain
  // sequence is safe; a supplied amax may lie below the data, so the numerator is clamped.
  const int path = !b200q_div_fast_ok(scale) ? kDivTrue : (AMAX_MODE == 0 ? kDivFast : kDivClamped);

  auto emit = [&](int g, const float* t, auto path_tag) {
    constexpr int P = decltype(path_tag)::value;
    float q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = div_path<P>(t[j], scale, y, lim);
    uint32_t lo = f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16);
    uint32_t hi = f32x2_to_e4m3x2(q[4], q[5]) | (f32x2_to_e4m3x2(q[6], q[7]) << 16);
    if constexpr (OUT == Out::Codes) {
      *reinterpret_cast<uint2*>(codes + row * cols + (int64_t)g * 8) = make_uint2(lo, hi);
    } else {
      float o[8];
      float2 p;
      p = e4m3x2_to_f32x2(lo), o[0] = __fmul_rn(p.x, scale), o[1] = __fmul_rn(p.y, scale);
      p = e4m3x2_to_f32x2(lo >> 16), o[2] = __fmul_rn(p.x, scale), o[3] = __fmul_rn(p.y, scale);
      p = e4m3x2_to_f32x2(hi), o[4] = __fmul_rn(p.x, scale), o[5] = __fmul_rn(p.y, scale);
      p = e4m3x2_to_f32x2(hi >> 16), o[6] = __fmul_rn(p.x, scale), o[7] = __fmul_rn(p.y, scale);
      Elem<T>::store8(fake + row * cols + (int64_t)g * 8, o);
    }
  };

  auto emit_all = [&](auto path_tag) {
    if constexpr (ITEMS > 0) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = threadIdx.x + i * kRowThreads;
        if (g < groups) emit(g, v[i], path_tag);
      }
    } else {
      for (int g = threadIdx.x; g < groups; g += kRowThreads) {
        float t[8];
        Elem<T>::load8(xr + (int64_t)g * 8, t);
        emit(g, t, path_tag);
      }
    }
  };

  if (path == kDivFast) emit_all(std::integral_constant<int, kDivFast>{});
  else if (path == kDivClamped) emit_all(std::integral_constant<int, kDivClamped>{});
  else emit_all(std::integral_constant<int, kDivTrue>{});
}

template <typename T, int AMAX_MODE, Out OUT>
int launch_rows_items(const T* x, const float* amax, uint8_t* codes, T* fake, float* scales, int64_t rows,
                      int64_t cols, cudaStream_t st) {
  const int64_t groups = cols >> 3;
  const int items = static_cast<int>((groups + kRowThreads - 1) / kRowThreads);
  dim3 grid(static_cast<unsigned>(rows)), block(kRowThreads);
#define B200Q_ROWS(I) launch_pdl(fp8_rows_kernel<T, I, AMAX_MODE, OUT>, grid, block, 0, st, x, amax, codes, fake, scales, rows, cols)
  if (items <= 1) B200Q_ROWS(1);
  else if (items <= 2) B200Q_ROWS(2);
  else if (items <= 4) B200Q_ROWS(4);
  else if (items <= kMaxItems) B200Q_ROWS(8);
  else B200Q_ROWS(0);
#undef B200Q_ROWS
  return check_launch();
}

template <typename T, Out OUT>
int launch_rows(const void* x, const float* amax, int64_t amax_numel, uint8_t* codes, void* fake, float* scales,
                int64_t rows, int64_t cols, cudaStream_t st) {
  const T* xt = static_cast<const T*>(x);
  T* ft = static_cast<T*>(fake);
  if (amax_numel == 0) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value && OUT == Out::Codes) {
      // many long rows: persistent CTAs fed through a shared-memory ring (fused_ops.cu)
      const int rc = launch_fp8_rows_stream(xt, codes, scales, rows, cols, st);
      if (rc != 1) return rc;
    }
    return launch_rows_items<T, 0, OUT>(xt, amax, codes, ft, scales, rows, cols, st);
  }
  if (amax_numel == 1) return launch_rows_items<T, 1, OUT>(xt, amax, codes, ft, scales, rows, cols, st);
  return launch_rows_items<T, 2, OUT>(xt, amax, codes, ft, scales, rows, cols, st);
}

int validate_rows(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax, int64_t amax_numel,
                  const void* out, int64_t col_multiple) {
  if (rows < 0 || cols < 0) return B200Q_ERR_INVALID;
  if (rows == 0 || cols == 0) return B200Q_OK;  // empty tensors are a valid no-op, whatever the pointers
  if (x == nullptr || out == nullptr) return B200Q_ERR_INVALID;
  if (dtype != B200Q_F32 && dtype != B200Q_F16 && dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (amax_numel != 0 && amax_numel != 1 && amax_numel != rows) return B200Q_ERR_INVALID;
  if (amax_numel != 0 && amax == nullptr) return B200Q_ERR_INVALID;
  if (cols % col_multiple != 0) return B200Q_ERR_INVALID;
  if (rows > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (!aligned(x, 16) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  return B200Q_OK;
}

// ---------------------------------------------------------------- dequantize
template <typename T>
__global__ void __launch_bounds__(256)
fp8_dequant_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scales, int per_row, T* __restrict__ out,
                   int64_t rows, int64_t cols) {
  const int64_t groups_per_row = cols >> 3;
  const int64_t total = rows * groups_per_row;
  for (int64_t g = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = g / groups_per_row;
    const float s = __ldg(scales + (per_row ? row : 0));
    const uint2 c = *reinterpret_cast<const uint2*>(codes + g * 8);
    float o[8];
    float2 p;
    p = e4m3x2_to_f32x2(c.x), o[0] = __fmul_rn(p.x, s), o[1] = __fmul_rn(p.y, s);
    p = e4m3x2_to_f32x2(c.x >> 16), o[2] = __fmul_rn(p.x, s), o[3] = __fmul_rn(p.y, s);
    p = e4m3x2_to_f32x2(c.y), o[4] = __fmul_rn(p.x, s), o[5] = __fmul_rn(p.y, s);
    p = e4m3x2_to_f32x2(c.y >> 16), o[6] = __fmul_rn(p.x, s), o[7] = __fmul_rn(p.y, s);
    Elem<T>::store8(out + g * 8, o);
  }
}

// ---------------------------------------------------------------- amax reductions
constexpr int kAmaxBlocks = 148 * 8;
constexpr int kAmaxThreads = 256;

// Single-pass tensor abs-max.  Every CTA folds its maximum into one running word (atomicMax on the
// bit pattern) and takes a ticket; the CTA that draws the last ticket writes the result and re-arms the
// ticket counter (so the workspace is zero again when the kernel ends).
// Running abs-max over 32-byte chunks as they come from memory.  16-bit types stay packed: the
// maximum of absolute values is exact in the input format, so two elements cost one instruction.
template <typename T>
struct ChunkMax;
template <>
struct ChunkMax<__nv_bfloat16> {
  static constexpr int kElems = 16;
  __nv_bfloat162 m = __floats2bfloat162_rn(0.0f, 0.0f);
  __device__ __forceinline__ void add(const U32x8& r) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&r.v[i])));
  }
  __device__ __forceinline__ float get() const { return fmaxf(__low2float(m), __high2float(m)); }
};
template <>
struct ChunkMax<__half> {
  static constexpr int kElems = 16;
  __half2 m = __floats2half2_rn(0.0f, 0.0f);
  __device__ __forceinline__ void add(const U32x8& r) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __half2*>(&r.v[i])));
  }
  __device__ __forceinline__ float get() const { return fmaxf(__low2float(m), __high2float(m)); }
};
template <>
struct ChunkMax<float> {
  static constexpr int kElems = 8;
  float m = 0.0f;
  __device__ __forceinline__ void add(const U32x8& r) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(__uint_as_float(r.v[i])));
  }
  __device__ __forceinline__ float get() const { return m; }
};

// `wide`: x is 32-byte aligned; the bulk then goes through 256-bit loads, four in flight per thread.
template <typename T>
__global__ void __launch_bounds__(kAmaxThreads)
amax_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ out, float* __restrict__ partials,
            unsigned int* __restrict__ ticket, bool wide) {
  __shared__ float red[kAmaxThreads / 32];
  pdl_launch_dependents();   // no-ops unless launched with the programmatic-serialization attribute
  pdl_wait();
  float local = 0.0f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  int64_t done = 0;  // elements covered by the wide part
  if (wide) {
    constexpr int kE = ChunkMax<T>::kElems;
    const int64_t chunks = n / kE;
    ChunkMax<T> acc;
    int64_t c = tid;
    for (; c + 3 * stride < chunks; c += 4 * stride) {
      const U32x8 r0 = ld_nc_256(x + c * kE);
      const U32x8 r1 = ld_nc_256(x + (c + stride) * kE);
      const U32x8 r2 = ld_nc_256(x + (c + 2 * stride) * kE);
      const U32x8 r3 = ld_nc_256(x + (c + 3 * stride) * kE);
      acc.add(r0);
      acc.add(r1);
      acc.add(r2);
      acc.add(r3);
    }
    for (; c < chunks; c += stride) acc.add(ld_nc_256(x + c * kE));
    local = acc.get();
    done = chunks * kE;
  }
  const int64_t groups = n >> 3;
  for (int64_t g = (done >> 3) + tid; g < groups; g += stride) {
    float t[8];
    Elem<T>::load8(x + g * 8, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) local = fmaxf(local, fabsf(t[j]));
  }
  if (blockIdx.x == 0) {  // ragged tail (n % 8 elements), scalar
    for (int64_t i = (groups << 3) + threadIdx.x; i < n; i += blockDim.x) local = fmaxf(local, fabsf(static_cast<float>(x[i])));
  }
  const float m = block_max<kAmaxThreads>(local, red);
  // CTA maxima meet in one word next to the ticket: values are >= 0 and never NaN here, so their bit patterns
  // order like unsigned integers.  The CTA that draws the last ticket hands the result out and re-arms both words.
  if (threadIdx.x == 0) {
    unsigned int* running = ticket + 1;
    atomicMax(running, __float_as_uint(m));
    __threadfence();
    const unsigned int t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      __threadfence();
      out[0] = __uint_as_float(atomicExch(running, 0u));
      *ticket = 0u;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
row_amax_kernel(const T* __restrict__ x, float* __restrict__ out, int64_t rows, int64_t cols) {
  __shared__ float red[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * cols;
  const int groups = static_cast<int>(cols >> 3);
  float local = 0.0f;
  for (int g = threadIdx.x; g < groups; g += kRowThreads) {
    float t[8];
    Elem<T>::load8(xr + (int64_t)g * 8, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) local = fmaxf(local, fabsf(t[j]));
  }
  const float m = block_max<kRowThreads>(local, red);
  if (threadIdx.x == 0) out[row] = m;
}

}  // namespace

// launcher used by the entry points below and by the no-scratch variants elsewhere
int launch_amax(const void* x, int dtype, int64_t n, float* out, float* partials, unsigned int* ticket,
                cudaStream_t st) {
  const bool wide = aligned(x, 32);
  // one CTA per kAmaxThreads x 4 chunks of 32 bytes (16 bytes without the alignment), up to 8 CTAs per SM
  int blocks = static_cast<int>((n >> 3) / (kAmaxThreads * (wide ? 8 : 1)));
  blocks = blocks < 1 ? 1 : (blocks > kAmaxBlocks ? kAmaxBlocks : blocks);
  // launched with the programmatic-serialization attribute: back-to-back launches overlap the next one's
  // start-up with this one's tail (the kernel waits for its predecessor before its first load)
  const dim3 grid(static_cast<unsigned>(blocks)), block(kAmaxThreads);
  switch (dtype) {
    case B200Q_BF16:
      launch_pdl(amax_kernel<__nv_bfloat16>, grid, block, 0, st, static_cast<const __nv_bfloat16*>(x), n, out, partials, ticket, wide);
      break;
    case B200Q_F16:
      launch_pdl(amax_kernel<__half>, grid, block, 0, st, static_cast<const __half*>(x), n, out, partials, ticket, wide);
      break;
    case B200Q_F32:
      launch_pdl(amax_kernel<float>, grid, block, 0, st, static_cast<const float*>(x), n, out, partials, ticket, wide);
      break;
    default:
      return B200Q_ERR_INVALID;
  }
  return check_launch();
}

// ---------------------------------------------------------------- abs-max without a caller workspace
// Scratch of b200q_amax_static: the ticket counter and the running maximum live in the first 256
// bytes (the rest is spare).  Zero at module load; the kernel re-arms both words when it ends.
constexpr int kStaticAmaxMaxBlocks = 1024;
constexpr int64_t kStaticAmaxElemsPerBlock = 1 << 18;
static __device__ __align__(256) unsigned char g_amax_static_scratch[256 + kStaticAmaxMaxBlocks * sizeof(float)];

namespace {
std::mutex g_static_mu;
unsigned char* g_static_scratch_addr[64] = {};

// Device address of the scratch array on the current device.  In host code the array's name
// is only a handle for the runtime, so the address is asked for once per device.
int static_scratch_address(unsigned char** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200Q_ERR_CUDA;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_scratch_addr[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_amax_static_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return B200Q_ERR_CUDA;
    }
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return B200Q_OK;
}

int launch_amax_static(const void* x, int dtype, int64_t n, float* out, float* partials, unsigned int* ticket,
                       cudaStream_t st) {
  const bool wide = aligned(x, 32);
  int blocks = static_cast<int>((n + kStaticAmaxElemsPerBlock - 1) / kStaticAmaxElemsPerBlock);
  if (blocks < 1) blocks = 1;
  switch (dtype) {
    case B200Q_BF16:
      amax_kernel<<<blocks, kAmaxThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, out, partials, ticket, wide);
      break;
    case B200Q_F16:
      amax_kernel<<<blocks, kAmaxThreads, 0, st>>>(static_cast<const __half*>(x), n, out, partials, ticket, wide);
      break;
    case B200Q_F32:
      amax_kernel<<<blocks, kAmaxThreads, 0, st>>>(static_cast<const float*>(x), n, out, partials, ticket, wide);
      break;
    default:
      return B200Q_ERR_INVALID;
  }
  return check_launch();
}
}  // namespace

}  // namespace b200q

using namespace b200q;

extern "C" {

size_t b200q_amax_workspace_bytes(void) { return (kAmaxBlocks + 64) * sizeof(float); }

int b200q_amax(const void* x, int dtype, int64_t n, float* amax_out, void* workspace, size_t workspace_bytes,
               b200q_stream_t stream) {
  if (x == nullptr || amax_out == nullptr || n < 0) return B200Q_ERR_INVALID;
  if (workspace == nullptr || workspace_bytes < b200q_amax_workspace_bytes()) return B200Q_ERR_WORKSPACE;
  if (!aligned(x, 16) || !aligned(workspace, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  // layout: [0, 64) floats reserved for the ticket counter (first word), then the partials
  unsigned int* ticket = static_cast<unsigned int*>(workspace);
  float* partials = static_cast<float*>(workspace) + 64;
  return launch_amax(x, dtype, n, amax_out, partials, ticket, static_cast<cudaStream_t>(stream));
}

int b200q_row_amax(const void* x, int dtype, int64_t rows, int64_t cols, float* amax_out, b200q_stream_t stream) {
  if (x == nullptr || amax_out == nullptr || rows < 0 || cols < 0 || cols % 8 != 0 || rows > 0x7fffffffLL)
    return B200Q_ERR_INVALID;
  if (!aligned(x, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (rows == 0) return B200Q_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(static_cast<unsigned>(rows)), block(kRowThreads);
  switch (dtype) {
    case B200Q_BF16: row_amax_kernel<<<grid, block, 0, st>>>(static_cast<const __nv_bfloat16*>(x), amax_out, rows, cols); break;
    case B200Q_F16: row_amax_kernel<<<grid, block, 0, st>>>(static_cast<const __half*>(x), amax_out, rows, cols); break;
    case B200Q_F32: row_amax_kernel<<<grid, block, 0, st>>>(static_cast<const float*>(x), amax_out, rows, cols); break;
    default: return B200Q_ERR_INVALID;
  }
  return check_launch();
}

int b200q_fp8_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax, int64_t amax_numel,
                       uint8_t* codes_out, float* scales_out, b200q_stream_t stream) {
  if (int rc = validate_rows(x, dtype, rows, cols, amax, amax_numel, codes_out, 16)) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  if (amax_numel != 1 && scales_out == nullptr) return B200Q_ERR_INVALID;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200Q_BF16: return launch_rows<__nv_bfloat16, Out::Codes>(x, amax, amax_numel, codes_out, nullptr, scales_out, rows, cols, st);
    case B200Q_F16: return launch_rows<__half, Out::Codes>(x, amax, amax_numel, codes_out, nullptr, scales_out, rows, cols, st);
    default: return launch_rows<float, Out::Codes>(x, amax, amax_numel, codes_out, nullptr, scales_out, rows, cols, st);
  }
}

int b200q_fp8_fake_quantize(const void* x, int dtype, int64_t rows, int64_t cols, const float* amax,
                            int64_t amax_numel, void* out, b200q_stream_t stream) {
  if (int rc = validate_rows(x, dtype, rows, cols, amax, amax_numel, out, 8)) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200Q_BF16: return launch_rows<__nv_bfloat16, Out::Fake>(x, amax, amax_numel, nullptr, out, nullptr, rows, cols, st);
    case B200Q_F16: return launch_rows<__half, Out::Fake>(x, amax, amax_numel, nullptr, out, nullptr, rows, cols, st);
    default: return launch_rows<float, Out::Fake>(x, amax, amax_numel, nullptr, out, nullptr, rows, cols, st);
  }
}

int b200q_fp8_dequantize(const uint8_t* codes, const float* scales, int64_t scales_numel, int64_t rows, int64_t cols,
                         void* out, int dtype, b200q_stream_t stream) {
  if (codes == nullptr || scales == nullptr || out == nullptr || rows < 0 || cols < 0 || cols % 8 != 0)
    return B200Q_ERR_INVALID;
  if (scales_numel != 1 && scales_numel != rows) return B200Q_ERR_INVALID;
  if (!aligned(codes, 8) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  if (rows == 0 || cols == 0) return B200Q_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * (cols >> 3);
  int blocks = static_cast<int>((total + 255) / 256);
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  const int per_row = (scales_numel == rows && scales_numel != 1) ? 1 : 0;
  switch (dtype) {
    case B200Q_BF16: fp8_dequant_kernel<<<blocks, 256, 0, st>>>(codes, scales, per_row, static_cast<__nv_bfloat16*>(out), rows, cols); break;
    case B200Q_F16: fp8_dequant_kernel<<<blocks, 256, 0, st>>>(codes, scales, per_row, static_cast<__half*>(out), rows, cols); break;
    case B200Q_F32: fp8_dequant_kernel<<<blocks, 256, 0, st>>>(codes, scales, per_row, static_cast<float*>(out), rows, cols); break;
    default: return B200Q_ERR_INVALID;
  }
  return check_launch();
}

int64_t b200q_amax_static_max_elements(void) { return kStaticAmaxMaxBlocks * kStaticAmaxElemsPerBlock; }

int b200q_amax_static(const void* x, int dtype, int64_t n, float* amax_out, b200q_stream_t stream) {
  if (x == nullptr || amax_out == nullptr || n < 0) return B200Q_ERR_INVALID;
  if (dtype != B200Q_F32 && dtype != B200Q_F16 && dtype != B200Q_BF16) return B200Q_ERR_INVALID;
  if (n > b200q_amax_static_max_elements()) return B200Q_ERR_TOO_LARGE;
  if (!aligned(x, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  unsigned char* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch);
  float* partials = reinterpret_cast<float*>(scratch + 256);
  return launch_amax_static(x, dtype, n, amax_out, partials, ticket, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
