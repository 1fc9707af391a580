// Elementwise / row-wise kernels either side of the quantized linears in the decoder
// linear stack: RMSNorm, silu(gate) * up, residual add, and the "attention = identity on V"
// head expansion.  All are HBM-bound streaming kernels over bf16 with 128-bit accesses.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"

namespace b200q {
namespace gemm {
int* device_status_word();
}
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// float at the same shared-memory address in CTA `rank` of the cluster
__device__ __forceinline__ float ld_cluster_f32(const float* p, int rank) {
  uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(p)), remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// y = x * rsqrt(mean(x^2) + eps) * w, fp32 math, bf16 in/out; one CTA per row, the row stays
// in registers (ITEMS groups of 8 per thread) or is re-read (ITEMS == 0).
template <int ITEMS>
__global__ void __launch_bounds__(kThreads)
rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                int64_t cols, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[kThreads / 32];
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * cols;
  __nv_bfloat16* yr = y + row * cols;
  const int groups = static_cast<int>(cols >> 3);
  float v[ITEMS > 0 ? ITEMS : 1][8];
  float ss = 0.0f;
  if constexpr (ITEMS > 0) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kThreads;
      if (g < groups) {
        Elem<__nv_bfloat16>::load8(xr + (int64_t)g * 8, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
      }
    }
  } else {
    for (int g = threadIdx.x; g < groups; g += kThreads) {
      float t[8];
      Elem<__nv_bfloat16>::load8(xr + (int64_t)g * 8, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(t[j], t[j], ss);
    }
  }
  const float total = block_sum<kThreads>(ss, red);
  const float inv = rsqrtf(total / static_cast<float>(cols) + eps);
  auto emit = [&](int g, const float* t) {
    float wv[8], o[8];
    Elem<__nv_bfloat16>::load8(w + (int64_t)g * 8, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = t[j] * inv * wv[j];
    Elem<__nv_bfloat16>::store8(yr + (int64_t)g * 8, o);
  };
  if constexpr (ITEMS > 0) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kThreads;
      if (g < groups) emit(g, v[i]);
    }
  } else {
    for (int g = threadIdx.x; g < groups; g += kThreads) {
      float t[8];
      Elem<__nv_bfloat16>::load8(xr + (int64_t)g * 8, t);
      emit(g, t);
    }
  }
}

// Residual add + RMSNorm + per-token FP8 quantize of one row per CTA, the row held in registers:
//   h_new = bf16(h + delta)            (delta may be null: h_new = h, nothing is written back)
//   x     = bf16(h_new * rsqrt(mean(h_new^2) + eps) * w)
//   scale = max|x| / 448 (0 -> 1);  code = e4m3(x / scale)
// Same arithmetic and rounding points as add -> rms_norm -> fp8 quantize run one after the
// other, with 1.75 bytes of traffic per element and step instead of 3.25.
// PARTS > 1: a cluster of PARTS CTAs shares one token (few tokens: a decode step); the slices'
// sums of squares and maxima meet through distributed shared memory, summed in rank order.
template <int ITEMS, int PARTS>
__global__ void __launch_bounds__(kThreads)
add_norm_quant_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out, uint8_t* __restrict__ codes,
                      float* __restrict__ scales, int64_t cols, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[kThreads / 32];
  __shared__ float part_val[2];
  const int64_t row = blockIdx.x / PARTS;
  const int part = PARTS > 1 ? static_cast<int>(blockIdx.x % PARTS) : 0;   // == rank in the cluster
  const int groups = static_cast<int>(cols >> 3);
  const int per_part = (groups + PARTS - 1) / PARTS;
  const int g_begin = part * per_part, g_end = min(groups, g_begin + per_part);
  // few-token form: the norm weights are requested together with the row, ahead of the first
  // reduction; many-token form: loaded after it (fewer live registers, more CTAs per SM)
  constexpr bool kEarlyW = PARTS > 1;
  float v[ITEMS][8];
  float wv[kEarlyW ? ITEMS : 1][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = g_begin + threadIdx.x + i * kThreads;
    if (g < g_end) {
      Elem<__nv_bfloat16>::load8(h + row * cols + (int64_t)g * 8, v[i]);
      if constexpr (kEarlyW) Elem<__nv_bfloat16>::load8(w + (int64_t)g * 8, wv[i]);
      if (delta != nullptr) {
        float d[8];
        Elem<__nv_bfloat16>::load8(delta + row * cols + (int64_t)g * 8, d);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] + d[j]));
        Elem<__nv_bfloat16>::store8(h_out + row * cols + (int64_t)g * 8, v[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
    }
  }
  float total = block_sum<kThreads>(ss, red);
  if constexpr (PARTS > 1) {
    if (threadIdx.x == 0) part_val[0] = total;
    cluster_barrier();
    total = 0.0f;
#pragma unroll
    for (int r = 0; r < PARTS; ++r) total += ld_cluster_f32(&part_val[0], r);
  }
  const float inv = rsqrtf(total / static_cast<float>(cols) + eps);
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = g_begin + threadIdx.x + i * kThreads;
    if (g < g_end) {
      float wl[8];
      if constexpr (!kEarlyW) Elem<__nv_bfloat16>::load8(w + (int64_t)g * 8, wl);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float wj = kEarlyW ? wv[kEarlyW ? i : 0][j] : wl[j];
        v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] * inv * wj));
        amax = fmaxf(amax, fabsf(v[i][j]));
      }
    }
  }
  // block max (values are >= 0): reuse the sum scratch
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = (threadIdx.x & 31) < kThreads / 32 ? red[threadIdx.x & 31] : 0.0f;
  amax = warp_max(amax);
  if constexpr (PARTS > 1) {
    if (threadIdx.x == 0) part_val[1] = amax;
    cluster_barrier();
    float other = 0.0f;
    if ((threadIdx.x & 31) < PARTS) other = ld_cluster_f32(&part_val[1], threadIdx.x & 31);
    amax = warp_max(other);
    cluster_barrier();  // nobody leaves while a peer may still read its shared memory
  }
  const float scale = fp8_scale_from_amax(amax);
  if (threadIdx.x == 0 && part == 0) scales[row] = scale;
  const float y = b200q_rcp_rn(scale);
  const bool fast = b200q_div_fast_ok(scale);
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = g_begin + threadIdx.x + i * kThreads;
    if (g < g_end) {
      float q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = fast ? b200q_div_by_shared(v[i][j], scale, y) : __fdiv_rn(v[i][j], scale);
      const uint32_t lo = f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16);
      const uint32_t hi = f32x2_to_e4m3x2(q[4], q[5]) | (f32x2_to_e4m3x2(q[6], q[7]) << 16);
      *reinterpret_cast<uint2*>(codes + row * cols + (int64_t)g * 8) = make_uint2(lo, hi);
    }
  }
}

// Many-token form of add_norm_quant_kernel: persistent CTAs (two per SM) walk the rows with a stride
// of the grid, and the rows of h and delta arrive through a ring of shared-memory stages filled by
// bulk asynchronous copies that one thread issues `stages` rows ahead.  One CTA per row keeps too few
// bytes in flight to cover the HBM latency (its loads stop while it reduces and stores); here the
// copies of the next rows run during all of that.  Thread-to-element mapping, arithmetic and
// reduction order are those of add_norm_quant_kernel, so the results are bit-identical.
constexpr int kStreamStagesMax = 8;
constexpr int kStreamRingBytes = 96 * 1024;

template <int ITEMS, bool HAS_DELTA>
__global__ void __launch_bounds__(kThreads, 2)
add_norm_quant_stream_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                             const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out, uint8_t* __restrict__ codes,
                             float* __restrict__ scales, int rows, int cols, float eps, int stages, int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ uint64_t full[kStreamStagesMax];
  __shared__ float red[kThreads / 32];
  const uint32_t row_bytes = static_cast<uint32_t>(cols) * 2u;
  const uint32_t stage_bytes = row_bytes * (HAS_DELTA ? 2u : 1u);
  const int groups = cols >> 3;
  const int step = static_cast<int>(gridDim.x);
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) ptx::mbar_init(&full[s], 1);
    ptx::fence_barrier_init();
  }
  __syncthreads();
  auto issue = [&](int row, int s) {
    ptx::mbar_arrive_expect_tx(&full[s], stage_bytes);
    ptx::bulk_load(ring + (size_t)s * stage_bytes, h + (int64_t)row * cols, row_bytes, &full[s]);
    if constexpr (HAS_DELTA) ptx::bulk_load(ring + (size_t)s * stage_bytes + row_bytes, delta + (int64_t)row * cols, row_bytes, &full[s]);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      const int64_t row = (int64_t)blockIdx.x + (int64_t)s * step;
      if (row < rows) issue(static_cast<int>(row), s);
    }
  }
  // the norm weights of this thread's groups are the same for every row
  uint4 wp[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = threadIdx.x + i * kThreads;
    wp[i] = g < groups ? ld_nc_128(w + (int64_t)g * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  int k = 0;
  for (int64_t row = blockIdx.x; row < rows; row += step, ++k) {
    const int s = k % stages;
    const bool arrived = ptx::mbar_wait(&full[s], static_cast<uint32_t>(k / stages) & 1u);
    // also separates this row's use of `red` from the previous row's last read of it
    if (__syncthreads_or(!arrived)) {
      if (threadIdx.x == 0) atomicCAS(status, 0, 81);
      break;
    }
    const unsigned char* st = ring + (size_t)s * stage_bytes;
    float v[ITEMS][8];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kThreads;
      if (g < groups) {
        Elem<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(st + (size_t)g * 16), v[i]);
        if constexpr (HAS_DELTA) {
          float d[8];
          Elem<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(st + row_bytes + (size_t)g * 16), d);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] + d[j]));
          Elem<__nv_bfloat16>::store8(h_out + row * cols + (int64_t)g * 8, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[i][j], v[i][j], ss);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
      }
    }
    const float total = block_sum<kThreads>(ss, red);
    // every thread has taken its part of the stage: refill it with the row `stages` steps ahead
    if (threadIdx.x == 0) {
      const int64_t next = row + (int64_t)stages * step;
      if (next < rows) issue(static_cast<int>(next), s);
    }
    const float inv = rsqrtf(total / static_cast<float>(cols) + eps);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kThreads;
      if (g < groups) {
        float wl[8];
        Elem<__nv_bfloat16>::unpack(wp[i], wl);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] * inv * wl[j]));
          amax = fmaxf(amax, fabsf(v[i][j]));
        }
      }
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = (threadIdx.x & 31) < kThreads / 32 ? red[threadIdx.x & 31] : 0.0f;
    amax = warp_max(amax);
    const float scale = fp8_scale_from_amax(amax);
    if (threadIdx.x == 0) scales[row] = scale;
    const float y = b200q_rcp_rn(scale);
    auto emit = [&](auto fast_tag) {
      constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = threadIdx.x + i * kThreads;
        if (g < groups) {
          float q[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) q[j] = kFast ? b200q_div_by_shared(v[i][j], scale, y) : __fdiv_rn(v[i][j], scale);
          const uint32_t lo = f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16);
          const uint32_t hi = f32x2_to_e4m3x2(q[4], q[5]) | (f32x2_to_e4m3x2(q[6], q[7]) << 16);
          *reinterpret_cast<uint2*>(codes + row * cols + (int64_t)g * 8) = make_uint2(lo, hi);
        }
      }
    };
    if (b200q_div_fast_ok(scale)) emit(std::true_type{});   // one branch per row, not one select per element
    else emit(std::false_type{});
  }
}

// act[t, j] = silu(gu[t, j]) * gu[t, F + j], gu is [T, 2F] (gate columns first)
__global__ void __launch_bounds__(kThreads)
silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int64_t rows, int64_t f) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t groups_per_row = f >> 3;
  const int64_t total = rows * groups_per_row;
  for (int64_t g = blockIdx.x * (int64_t)kThreads + threadIdx.x; g < total; g += (int64_t)gridDim.x * kThreads) {
    const int64_t row = g / groups_per_row, c = (g - row * groups_per_row) * 8;
    float a[8], b[8], o[8];
    Elem<__nv_bfloat16>::load8(gu + row * 2 * f + c, a);
    Elem<__nv_bfloat16>::load8(gu + row * 2 * f + f + c, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = silu_mul_f32(a[j], b[j]);
    Elem<__nv_bfloat16>::store8(act + row * f + c, o);
  }
}

// silu(gate) * up fused with the per-token FP8 quantize that feeds the down projection: the
// bf16 activation [T, F] is never written.  One CTA per token; the row stays in registers as
// packed bf16 (ITEMS groups of 8 per thread), rounded exactly as silu_mul_kernel stores it, so
// codes and scales equal those of the two separate kernels.
// PARTS > 1: a cluster of PARTS CTAs shares one token (few tokens, long rows: a decode step would
// otherwise run on a handful of SMs); each CTA takes a contiguous slice of the row and the slice
// maxima meet through distributed shared memory.
template <int ITEMS, int PARTS>
__global__ void __launch_bounds__(kThreads)
silu_mul_quant_kernel(const __nv_bfloat16* __restrict__ gu, uint8_t* __restrict__ codes, float* __restrict__ scales, int64_t f) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[kThreads / 32];
  __shared__ float part_max;
  const int64_t row = blockIdx.x / PARTS;
  const int part = PARTS > 1 ? static_cast<int>(blockIdx.x % PARTS) : 0;   // == rank in the cluster
  const int groups = static_cast<int>(f >> 3);
  const int per_part = (groups + PARTS - 1) / PARTS;
  const int g_begin = part * per_part, g_end = min(groups, g_begin + per_part);
  uint4 y[ITEMS];
  __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);   // running max |.| of the packed results (exact in bf16)
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = g_begin + threadIdx.x + i * kThreads;
    y[i] = make_uint4(0u, 0u, 0u, 0u);
    if (g < g_end) {
      float a[8], b[8];
      Elem<__nv_bfloat16>::load8(gu + row * 2 * f + (int64_t)g * 8, a);
      Elem<__nv_bfloat16>::load8(gu + row * 2 * f + f + (int64_t)g * 8, b);
      uint32_t* u = &y[i].x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul_f32(a[2 * j], b[2 * j]), silu_mul_f32(a[2 * j + 1], b[2 * j + 1]));
        u[j] = *reinterpret_cast<const uint32_t*>(&h);
        m2 = __hmax2(m2, __habs2(h));
      }
    }
  }
  float amax = fmaxf(__low2float(m2), __high2float(m2));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = (threadIdx.x & 31) < kThreads / 32 ? red[threadIdx.x & 31] : 0.0f;
  amax = warp_max(amax);
  if constexpr (PARTS > 1) {
    if (threadIdx.x == 0) part_max = amax;
    cluster_barrier();
    float other = 0.0f;
    if ((threadIdx.x & 31) < PARTS) other = ld_cluster_f32(&part_max, threadIdx.x & 31);
    amax = warp_max(other);
    cluster_barrier();  // nobody leaves (or rewrites part_max) while a peer may still read it
  }
  const float scale = fp8_scale_from_amax(amax);
  if (threadIdx.x == 0 && part == 0) scales[row] = scale;
  const float rcp = b200q_rcp_rn(scale);
  auto emit = [&](auto fast_tag) {
    constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = g_begin + threadIdx.x + i * kThreads;
      if (g < g_end) {
        float v[8], q[8];
        Elem<__nv_bfloat16>::unpack(y[i], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = kFast ? b200q_div_by_shared(v[j], scale, rcp) : __fdiv_rn(v[j], scale);
        const uint32_t lo = f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16);
        const uint32_t hi = f32x2_to_e4m3x2(q[4], q[5]) | (f32x2_to_e4m3x2(q[6], q[7]) << 16);
        *reinterpret_cast<uint2*>(codes + row * f + (int64_t)g * 8) = make_uint2(lo, hi);
      }
    }
  };
  // one branch per row, not one select per element: the true division is an order of magnitude longer
  if (b200q_div_fast_ok(scale)) emit(std::true_type{});
  else emit(std::false_type{});
}

// Many-token form of silu_mul_quant_kernel: persistent CTAs (two per SM), one row per iteration, the
// gate and up halves of the row arriving in chunks of 2 * kThreads groups (8 KB each) through a ring of
// shared-memory stages that one thread keeps filled with bulk asynchronous copies, across rows.  The
// row's results wait in registers, packed as bf16, for the row maximum.  Same expression, rounding
// points and thread-to-element mapping per chunk as the per-row kernels: same codes and scales.
constexpr int kSiluChunkGroups = 2 * kThreads;                // groups of 8 elements per chunk and half
constexpr int kSiluChunkBytes = kSiluChunkGroups * 16;        // per half
constexpr int kSiluStages = 6;                                // 6 x 16 KB

// GATED = false: the same machine as a plain per-token FP8 quantize of bf16 rows [rows, f] (one source, chunks of
// 8 KB): rows too long to stay in registers with one CTA per row would otherwise be read twice.
template <int CHUNKS, bool GATED>
__global__ void __launch_bounds__(kThreads, 2)
silu_mul_quant_stream_kernel(const __nv_bfloat16* __restrict__ gu, uint8_t* __restrict__ codes, float* __restrict__ scales, int rows,
                             int f, int* __restrict__ status) {
  constexpr int kStageBytes = (GATED ? 2 : 1) * kSiluChunkBytes;
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ uint64_t full[kSiluStages];
  __shared__ float red[kThreads / 32];
  const int groups = f >> 3;
  const int nch = (groups + kSiluChunkGroups - 1) / kSiluChunkGroups;    // chunks per row (<= CHUNKS)
  const int step = static_cast<int>(gridDim.x);
  const int my_rows = (rows - static_cast<int>(blockIdx.x) + step - 1) / step;
  const int total = my_rows * nch;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSiluStages; ++s) ptx::mbar_init(&full[s], 1);
    ptx::fence_barrier_init();
  }
  __syncthreads();
  // copy number q of this CTA: chunk q % nch of its row number q / nch; gate half first, up half behind it
  auto issue = [&](int q) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(q / nch) * step;
    const int c = q % nch;
    const int g0 = c * kSiluChunkGroups;
    const uint32_t bytes = static_cast<uint32_t>(min(kSiluChunkGroups, groups - g0)) * 16u;
    const __nv_bfloat16* gate = gu + row * (GATED ? 2 : 1) * f + static_cast<int64_t>(g0) * 8;
    const int s = q % kSiluStages;
    unsigned char* dst = ring + static_cast<size_t>(s) * kStageBytes;
    ptx::mbar_arrive_expect_tx(&full[s], (GATED ? 2u : 1u) * bytes);
    ptx::bulk_load(dst, gate, bytes, &full[s]);
    if constexpr (GATED) ptx::bulk_load(dst + kSiluChunkBytes, gate + f, bytes, &full[s]);
  };
  if (threadIdx.x == 0)
    for (int q = 0; q < kSiluStages && q < total; ++q) issue(q);
  bool arrived = true;   // after one wait gave up the rest are not waited for: the status word says the result is void
  int q = 0;
  for (int64_t row = blockIdx.x; row < rows; row += step) {
    uint4 y[CHUNKS][2];
    __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      if (c < nch) {
        const int s = q % kSiluStages;
        if (arrived && !ptx::mbar_wait(&full[s], static_cast<uint32_t>(q / kSiluStages) & 1u)) {
          arrived = false;
          atomicCAS(status, 0, 82);
        }
        const unsigned char* st = ring + static_cast<size_t>(s) * kStageBytes;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int gl = threadIdx.x + i * kThreads;              // group inside the chunk
          y[c][i] = make_uint4(0u, 0u, 0u, 0u);
          if (c * kSiluChunkGroups + gl < groups) {
            if constexpr (!GATED) {
              y[c][i] = *reinterpret_cast<const uint4*>(st + static_cast<size_t>(gl) * 16);
              const uint32_t* u = &y[c][i].x;
#pragma unroll
              for (int j = 0; j < 4; ++j) m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&u[j])));
              continue;
            }
            float a[8], b[8];
            Elem<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(st + static_cast<size_t>(gl) * 16), a);
            Elem<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(st + kSiluChunkBytes + static_cast<size_t>(gl) * 16), b);
            uint32_t* u = &y[c][i].x;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 hh = __floats2bfloat162_rn(silu_mul_f32(a[2 * j], b[2 * j]), silu_mul_f32(a[2 * j + 1], b[2 * j + 1]));
              u[j] = *reinterpret_cast<const uint32_t*>(&hh);
              m2 = __hmax2(m2, __habs2(hh));
            }
          }
        }
        __syncthreads();                                           // the whole CTA has taken its part of the stage
        if (threadIdx.x == 0 && q + kSiluStages < total) issue(q + kSiluStages);
        ++q;
      }
    }
    float amax = fmaxf(__low2float(m2), __high2float(m2));
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = (threadIdx.x & 31) < kThreads / 32 ? red[threadIdx.x & 31] : 0.0f;
    amax = warp_max(amax);
    const float scale = fp8_scale_from_amax(amax);
    if (threadIdx.x == 0) scales[row] = scale;
    const float rcp = b200q_rcp_rn(scale);
    auto emit = [&](auto fast_tag) {
      constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int g = c * kSiluChunkGroups + threadIdx.x + i * kThreads;
          if (c < nch && g < groups) {
            float v[8], qv[8];
            Elem<__nv_bfloat16>::unpack(y[c][i], v);
#pragma unroll
            for (int j = 0; j < 8; ++j) qv[j] = kFast ? b200q_div_by_shared(v[j], scale, rcp) : __fdiv_rn(v[j], scale);
            const uint32_t lo = f32x2_to_e4m3x2(qv[0], qv[1]) | (f32x2_to_e4m3x2(qv[2], qv[3]) << 16);
            const uint32_t hi = f32x2_to_e4m3x2(qv[4], qv[5]) | (f32x2_to_e4m3x2(qv[6], qv[7]) << 16);
            *reinterpret_cast<uint2*>(codes + row * f + static_cast<int64_t>(g) * 8) = make_uint2(lo, hi);
          }
        }
      }
    };
    if (b200q_div_fast_ok(scale)) emit(std::true_type{});
    else emit(std::false_type{});
    // `red` is written again only after the next row's chunk barriers
  }
}

// out = a + b (bf16, fp32 add)
__global__ void __launch_bounds__(kThreads)
add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ out, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t groups = n >> 3;
  for (int64_t g = blockIdx.x * (int64_t)kThreads + threadIdx.x; g < groups; g += (int64_t)gridDim.x * kThreads) {
    float x[8], y[8];
    Elem<__nv_bfloat16>::load8(a + g * 8, x);
    Elem<__nv_bfloat16>::load8(b + g * 8, y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    Elem<__nv_bfloat16>::store8(out + g * 8, x);
  }
}

// out[t, h * hd + d] = src[t, src_col0 + (h / rep) * hd + d]: every kv head repeated `rep` times
__global__ void __launch_bounds__(kThreads)
expand_heads_kernel(const __nv_bfloat16* __restrict__ src, int64_t src_stride, int64_t src_col0, __nv_bfloat16* __restrict__ out,
                    int64_t rows, int heads_out, int rep, int head_dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t groups_per_head = head_dim >> 3;
  const int64_t groups_per_row = heads_out * groups_per_head;
  const int64_t total = rows * groups_per_row;
  for (int64_t g = blockIdx.x * (int64_t)kThreads + threadIdx.x; g < total; g += (int64_t)gridDim.x * kThreads) {
    const int64_t row = g / groups_per_row, r = g - row * groups_per_row;
    const int64_t h = r / groups_per_head, d = (r - h * groups_per_head) * 8;
    const uint4 v = *reinterpret_cast<const uint4*>(src + row * src_stride + src_col0 + (h / rep) * head_dim + d);
    *reinterpret_cast<uint4*>(out + row * groups_per_row * 8 + h * head_dim + d) = v;
  }
}

// expand_heads followed by the per-token FP8 quantize, in one pass over the kv slice: a repeated head does
// not change the token's abs-max, so the token is quantized once (one warp per token, its slice in
// registers) and every code group is stored `rep` times.  The same codes and scales as
// b200q_expand_heads + b200q_fp8_quantize with dynamic per-row amax; the expanded bf16 tensor is never written.
template <int ITEMS>
__global__ void __launch_bounds__(kThreads)
expand_heads_quant_kernel(const __nv_bfloat16* __restrict__ src, int64_t src_stride, int64_t src_col0, uint8_t* __restrict__ codes,
                          float* __restrict__ scales, int64_t rows, int heads_out, int rep, int head_dim) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(kThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int kv_heads = heads_out / rep;
  const int groups = (kv_heads * head_dim) >> 3;            // groups of 8 elements in the token's kv slice
  const int64_t out_cols = static_cast<int64_t>(heads_out) * head_dim;
  float v[ITEMS][8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = lane + i * 32;
    if (g < groups) {
      Elem<__nv_bfloat16>::load8(src + row * src_stride + src_col0 + (int64_t)g * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    }
  }
  amax = warp_max(amax);
  const float scale = fp8_scale_from_amax(amax);
  if (lane == 0) scales[row] = scale;
  const float y = b200q_rcp_rn(scale);
  const bool fast = b200q_div_fast_ok(scale);
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = lane + i * 32;
    if (g < groups) {
      float q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = fast ? b200q_div_by_shared(v[i][j], scale, y) : __fdiv_rn(v[i][j], scale);
      const uint2 packed = make_uint2(f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16),
                                      f32x2_to_e4m3x2(q[4], q[5]) | (f32x2_to_e4m3x2(q[6], q[7]) << 16));
      const int e = g * 8, kvh = e / head_dim, d = e - kvh * head_dim;
      uint8_t* dst = codes + row * out_cols + static_cast<int64_t>(kvh) * rep * head_dim + d;
      for (int r = 0; r < rep; ++r) *reinterpret_cast<uint2*>(dst + static_cast<int64_t>(r) * head_dim) = packed;
    }
  }
}

int grid_for(int64_t work_items) {
  int64_t ctas = (work_items + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  return static_cast<int>(ctas < 1 ? 1 : (ctas > cap ? cap : ctas));
}

}  // namespace

// Dynamic per-token FP8 quantize of many long bf16 rows through the ring-fed persistent kernel
// (silu_mul_quant_stream_kernel<.., false>).  Returns 1 when the shape does not qualify (the caller
// then takes its one-CTA-per-row kernels), else the launch status.
int launch_fp8_rows_stream(const __nv_bfloat16* x, uint8_t* codes, float* scales, int64_t rows, int64_t cols, cudaStream_t st) {
  static const bool enabled = [] {
    const char* e = std::getenv("B200Q_ROWS_STREAM");   // 0 = always one CTA per row (A/B measurements)
    return e == nullptr || e[0] != '0';
  }();
  if (!enabled) return 1;
  const int64_t groups = cols >> 3;
  // rows of up to 16384 elements stay in registers with one CTA per row, which is faster (0.82-0.91 of HBM against
  // 0.54-0.72 here); beyond that the one-CTA form reads the row twice and this one wins (0.81)
  if (cols % 8 != 0 || rows < 8 * sm_count() || rows > 0x7fffffffLL || cols <= 16384 || groups > 8 * kSiluChunkGroups) return 1;
  if (!aligned(x, 16) || !aligned(codes, 8)) return 1;
  int* status = gemm::device_status_word();
  if (status == nullptr) return B200Q_ERR_CUDA;
  const int nch = static_cast<int>((groups + kSiluChunkGroups - 1) / kSiluChunkGroups);
  const size_t smem = static_cast<size_t>(kSiluStages) * kSiluChunkBytes;
  const dim3 grid(static_cast<unsigned>(2 * sm_count()));
  const int r32 = static_cast<int>(rows), f32 = static_cast<int>(cols);
#define B200Q_ROWS_STREAM(C)                                                                                                 \
  do {                                                                                                                        \
    cudaFuncSetAttribute(silu_mul_quant_stream_kernel<C, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    launch_pdl(silu_mul_quant_stream_kernel<C, false>, grid, dim3(kThreads), smem, st, x, codes, scales, r32, f32, status);           \
  } while (0)
  if (nch <= 2) B200Q_ROWS_STREAM(2);
  else if (nch <= 4) B200Q_ROWS_STREAM(4);
  else B200Q_ROWS_STREAM(8);
#undef B200Q_ROWS_STREAM
  return check_launch();
}
}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_rms_norm(const void* x, const void* weight, void* out, int64_t rows, int64_t cols, float eps, b200q_stream_t stream) {
  if (rows < 0 || cols < 0 || cols % 8 != 0 || rows > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (rows == 0 || cols == 0) return B200Q_OK;
  if (x == nullptr || weight == nullptr || out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(x, 16) || !aligned(weight, 16) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* wp = static_cast<const __nv_bfloat16*>(weight);
  auto* yp = static_cast<__nv_bfloat16*>(out);
  const int items = static_cast<int>(((cols >> 3) + kThreads - 1) / kThreads);
  dim3 grid(static_cast<unsigned>(rows));
  if (items <= 1) launch_pdl(rms_norm_kernel<1>, dim3(grid), dim3(kThreads), 0, st, xp, wp, yp, cols, eps);
  else if (items <= 2) launch_pdl(rms_norm_kernel<2>, dim3(grid), dim3(kThreads), 0, st, xp, wp, yp, cols, eps);
  else if (items <= 4) launch_pdl(rms_norm_kernel<4>, dim3(grid), dim3(kThreads), 0, st, xp, wp, yp, cols, eps);
  else launch_pdl(rms_norm_kernel<0>, dim3(grid), dim3(kThreads), 0, st, xp, wp, yp, cols, eps);
  return check_launch();
}

int b200q_add_rms_norm_fp8_quantize(const void* h, const void* delta, const void* weight, void* h_out, uint8_t* codes_out,
                                    float* scales_out, int64_t rows, int64_t cols, float eps, b200q_stream_t stream) {
  if (rows < 0 || cols < 0 || cols % 16 != 0 || rows > 0x7fffffffLL || cols > kThreads * 8 * 8) return B200Q_ERR_INVALID;
  if (rows == 0 || cols == 0) return B200Q_OK;
  if (h == nullptr || weight == nullptr || codes_out == nullptr || scales_out == nullptr) return B200Q_ERR_INVALID;
  if (delta != nullptr && h_out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(h, 16) || !aligned(weight, 16) || !aligned(codes_out, 8) || (delta != nullptr && (!aligned(delta, 16) || !aligned(h_out, 16))))
    return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto* hp = static_cast<const __nv_bfloat16*>(h);
  const auto* dp = static_cast<const __nv_bfloat16*>(delta);
  const auto* wp = static_cast<const __nv_bfloat16*>(weight);
  auto* op = static_cast<__nv_bfloat16*>(h_out);
  const int64_t groups = cols >> 3;
  int parts = 1;   // few tokens: split every row over a cluster so that the launch covers more SMs
  while (parts < 8 && rows * parts < 2 * sm_count() && groups / (parts * 2) >= kThreads / 2) parts *= 2;
  const int items = static_cast<int>(((groups + parts - 1) / parts + kThreads - 1) / kThreads);
  // many tokens: persistent CTAs fed through a shared-memory ring of rows
  const int64_t stage_bytes = cols * 2 * (delta != nullptr ? 2 : 1);
  if (parts == 1 && items <= 4 && rows >= 8 * sm_count() && kStreamRingBytes / stage_bytes >= 2) {
    int stages = static_cast<int>(kStreamRingBytes / stage_bytes);
    if (stages > kStreamStagesMax) stages = kStreamStagesMax;
    int* status = gemm::device_status_word();
    if (status == nullptr) return B200Q_ERR_CUDA;
    const size_t smem = static_cast<size_t>(stages) * static_cast<size_t>(stage_bytes);
    const dim3 grid(static_cast<unsigned>(2 * sm_count()));
    const int r32 = static_cast<int>(rows), c32 = static_cast<int>(cols);
#define B200Q_ANQS(I, D)                                                                                                     \
  do {                                                                                                                        \
    cudaFuncSetAttribute(add_norm_quant_stream_kernel<I, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamRingBytes); \
    launch_pdl(add_norm_quant_stream_kernel<I, D>, grid, dim3(kThreads), smem, st, hp, dp, wp, op, codes_out, scales_out,     \
               r32, c32, eps, stages, status);                                                                                \
  } while (0)
    if (delta != nullptr) {
      if (items <= 1) B200Q_ANQS(1, true);
      else if (items <= 2) B200Q_ANQS(2, true);
      else B200Q_ANQS(4, true);
    } else {
      if (items <= 1) B200Q_ANQS(1, false);
      else if (items <= 2) B200Q_ANQS(2, false);
      else B200Q_ANQS(4, false);
    }
#undef B200Q_ANQS
    return check_launch();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows * parts));
  cfg.blockDim = dim3(kThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(parts);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
#define B200Q_ANQ(I, P) cudaLaunchKernelEx(&cfg, add_norm_quant_kernel<I, P>, hp, dp, wp, op, codes_out, scales_out, cols, eps)
  if (parts == 1) {
    if (items <= 1) B200Q_ANQ(1, 1);
    else if (items <= 2) B200Q_ANQ(2, 1);
    else if (items <= 4) B200Q_ANQ(4, 1);
    else B200Q_ANQ(8, 1);
  } else if (parts == 2) {
    if (items <= 1) B200Q_ANQ(1, 2);
    else if (items <= 2) B200Q_ANQ(2, 2);
    else B200Q_ANQ(4, 2);
  } else if (parts == 4) {
    if (items <= 1) B200Q_ANQ(1, 4);
    else B200Q_ANQ(2, 4);
  } else {
    B200Q_ANQ(1, 8);
  }
#undef B200Q_ANQ
  return check_launch();
}

int b200q_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t f, b200q_stream_t stream) {
  if (rows < 0 || f < 0 || f % 8 != 0) return B200Q_ERR_INVALID;
  if (rows == 0 || f == 0) return B200Q_OK;
  if (gate_up == nullptr || out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(gate_up, 16) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  launch_pdl(silu_mul_kernel, dim3(grid_for(rows * (f >> 3))), dim3(kThreads), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), rows, f);
  return check_launch();
}

int b200q_silu_mul_fp8_quantize(const void* gate_up, uint8_t* codes_out, float* scales_out, int64_t rows, int64_t f,
                                b200q_stream_t stream) {
  if (rows < 0 || f < 0 || f % 8 != 0 || rows > 0x7fffffffLL || f > kThreads * 8 * 16) return B200Q_ERR_INVALID;
  if (rows == 0 || f == 0) return B200Q_OK;
  if (gate_up == nullptr || codes_out == nullptr || scales_out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(gate_up, 16) || !aligned(codes_out, 8)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto* gp = static_cast<const __nv_bfloat16*>(gate_up);
  const int64_t groups = f >> 3;
  // many tokens, rows of at least one chunk: persistent CTAs fed through a shared-memory ring
  if (rows >= 8 * sm_count() && groups >= kSiluChunkGroups) {
    int* status = gemm::device_status_word();
    if (status == nullptr) return B200Q_ERR_CUDA;
    const int nch = static_cast<int>((groups + kSiluChunkGroups - 1) / kSiluChunkGroups);
    const size_t smem = static_cast<size_t>(kSiluStages) * 2 * kSiluChunkBytes;
    const dim3 grid(static_cast<unsigned>(2 * sm_count()));
    const int r32 = static_cast<int>(rows), f32 = static_cast<int>(f);
#define B200Q_SILUS(C)                                                                                              \
  do {                                                                                                               \
    cudaFuncSetAttribute(silu_mul_quant_stream_kernel<C, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    launch_pdl(silu_mul_quant_stream_kernel<C, true>, grid, dim3(kThreads), smem, st, gp, codes_out, scales_out, r32, f32, status);   \
  } while (0)
    if (nch <= 2) B200Q_SILUS(2);
    else if (nch <= 4) B200Q_SILUS(4);
    else B200Q_SILUS(8);
#undef B200Q_SILUS
    return check_launch();
  }
  // few tokens: split every row over a cluster so that the launch covers the SMs
  int parts = 1;
  while (parts < 8 && rows * parts < 2 * sm_count() && groups / (parts * 2) >= kThreads / 2) parts *= 2;
  // long rows: 16 groups per thread cost 92 registers (two CTAs per SM) and the kernel turns
  // compute-bound on the exponentials; two CTAs per row at 8 groups per thread double the warps per SM
  if (parts == 1 && groups > 8 * kThreads) parts = 2;
  const int items = static_cast<int>(((groups + parts - 1) / parts + kThreads - 1) / kThreads);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows * parts));
  cfg.blockDim = dim3(kThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(parts);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
#define B200Q_SILU(I, P) cudaLaunchKernelEx(&cfg, silu_mul_quant_kernel<I, P>, gp, codes_out, scales_out, f)
  if (parts == 1) {
    if (items <= 1) B200Q_SILU(1, 1);
    else if (items <= 2) B200Q_SILU(2, 1);
    else if (items <= 4) B200Q_SILU(4, 1);
    else if (items <= 8) B200Q_SILU(8, 1);
    else B200Q_SILU(16, 1);
  } else if (parts == 2) {
    if (items <= 1) B200Q_SILU(1, 2);
    else if (items <= 2) B200Q_SILU(2, 2);
    else if (items <= 4) B200Q_SILU(4, 2);
    else B200Q_SILU(8, 2);
  } else if (parts == 4) {
    if (items <= 1) B200Q_SILU(1, 4);
    else if (items <= 2) B200Q_SILU(2, 4);
    else B200Q_SILU(4, 4);
  } else {
    if (items <= 1) B200Q_SILU(1, 8);
    else B200Q_SILU(2, 8);
  }
#undef B200Q_SILU
  return check_launch();
}

int b200q_add(const void* a, const void* b, void* out, int64_t n, b200q_stream_t stream) {
  if (n < 0 || n % 8 != 0) return B200Q_ERR_INVALID;
  if (n == 0) return B200Q_OK;
  if (a == nullptr || b == nullptr || out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(a, 16) || !aligned(b, 16) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  launch_pdl(add_kernel, dim3(grid_for(n >> 3)), dim3(kThreads), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(out), n);
  return check_launch();
}

int b200q_expand_heads(const void* src, int64_t src_stride, int64_t src_col0, void* out, int64_t rows, int heads_out, int rep,
                       int head_dim, b200q_stream_t stream) {
  if (rows < 0 || heads_out <= 0 || rep <= 0 || head_dim <= 0 || head_dim % 8 != 0 || heads_out % rep != 0 || src_stride % 8 != 0 ||
      src_col0 % 8 != 0)
    return B200Q_ERR_INVALID;
  if (rows == 0) return B200Q_OK;
  if (src == nullptr || out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(src, 16) || !aligned(out, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  launch_pdl(expand_heads_kernel, dim3(grid_for(rows * heads_out * (head_dim >> 3))), dim3(kThreads), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(src), src_stride, src_col0, static_cast<__nv_bfloat16*>(out), rows, heads_out, rep, head_dim);
  return check_launch();
}

int b200q_expand_heads_fp8_quantize(const void* src, int64_t src_stride, int64_t src_col0, uint8_t* codes_out, float* scales_out,
                                    int64_t rows, int heads_out, int rep, int head_dim, b200q_stream_t stream) {
  if (rows < 0 || heads_out <= 0 || rep <= 0 || head_dim <= 0 || head_dim % 8 != 0 || heads_out % rep != 0 || src_stride % 8 != 0 ||
      src_col0 % 8 != 0 || rows > 0x7fffffffLL)
    return B200Q_ERR_INVALID;
  const int64_t kv_width = static_cast<int64_t>(heads_out / rep) * head_dim;
  if (kv_width > 32 * 8 * 8) return B200Q_ERR_INVALID;       // the slice of a token stays in one warp's registers
  if (rows == 0) return B200Q_OK;
  if (src == nullptr || codes_out == nullptr || scales_out == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(src, 16) || !aligned(codes_out, 8)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const int items = static_cast<int>(((kv_width >> 3) + 31) / 32);
  const dim3 grid(static_cast<unsigned>((rows + kThreads / 32 - 1) / (kThreads / 32)));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto* sp = static_cast<const __nv_bfloat16*>(src);
#define B200Q_EHQ(I) launch_pdl(expand_heads_quant_kernel<I>, grid, dim3(kThreads), 0, st, sp, src_stride, src_col0, codes_out, scales_out, rows, heads_out, rep, head_dim)
  if (items <= 1) B200Q_EHQ(1);
  else if (items <= 2) B200Q_EHQ(2);
  else if (items <= 4) B200Q_EHQ(4);
  else B200Q_EHQ(8);
#undef B200Q_EHQ
  return check_launch();
}

}  // extern "C"
