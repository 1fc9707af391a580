// Small-M variant of the quantized GEMM (decode steps, M <= 128 tokens).
//
// With M <= 128 the problem is a stream of weights: it is HBM-bound, the activations are tiny,
// and there are only N / 128 output tiles.  Two changes against the persistent kernel:
//
//   * operands swapped: the 128 weight rows of a tile are the tcgen05 "M" side and the tokens
//     are the "N" side, padded to a multiple of 16 only (not to 128).  A pipeline stage is then
//     16 KiB of weights plus at most 16 KiB of activations, so the shared-memory ring holds up
//     to 12 K tiles of weights in flight per SM, and the tensor core does no work on padding.
//   * K split over a cluster: S CTAs (S = 1, 2, 4, 8) share one output tile, CTA r runs the
//     TMA / tcgen05 main loop over its own slice of K, so S times as many SMs pull weights.
//     Each CTA parks its fp32 partial tile [token][weight row] in its own shared memory; after
//     a cluster barrier CTA r sums the tokens it owns over all S partials with 16-byte
//     ld.shared::cluster loads, applies the dequantization scales and the bias and stores
//     bf16 rows.  No global workspace, no atomics, fixed summation order.
#pragma once

#include "gemm_kernel.cuh"

namespace b200q {
namespace gemm {

constexpr int kSmallWRows = 128;    // weight rows per tile
constexpr int kSmallMaxStages = 12;
constexpr int kSmallTailBytes = 2048;
constexpr int kSmallHalfSmem = (233472 - 2 * 1024) / 2;  // dynamic shared memory of a CTA when two share an SM

// Shared-memory and tensor-memory budget of a launch (host and device agree through these).
template <bool NVF4>
struct SmallCfg {
  static constexpr int kWBytes = kSmallWRows * kBKBytes;             // 16 KiB
  static constexpr int kSfBytes = NVF4 ? 4096 : 0;                   // weight + token scale atoms of one K tile
  static constexpr int kSfCols = NVF4 ? 32 : 0;                      // tensor-memory columns per stage (16 + 16)
  __host__ __device__ static constexpr int stage_bytes(int bt) { return kWBytes + bt * kBKBytes + kSfBytes; }
  __host__ __device__ static constexpr int smem_bytes(int bt, int stages) { return 1024 + stages * stage_bytes(bt) + kSmallTailBytes; }
  __host__ __device__ static constexpr int tmem_cols(int stages) {
    const int need = 128 + stages * kSfCols;
    return need <= 128 ? 128 : (need <= 256 ? 256 : 512);
  }
  // deepest ring that fits `budget` bytes of shared memory and 512 tensor-memory columns
  static int max_stages(int bt, int budget) {
    int s = (budget - 1024 - kSmallTailBytes) / stage_bytes(bt);
    if (s > kSmallMaxStages) s = kSmallMaxStages;
    return s;
  }
};

__device__ __forceinline__ float4 ld_shared_cluster_v4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// Sum tokens [t0, t1) of the S partial tiles of the cluster, scale, add bias, store bf16.
// partial tile layout: float [token][128 weight rows]; thread item = (token, group of 8 rows).
template <int S>
__device__ __forceinline__ void small_reduce_store(uint32_t partial_u32, int t0, int t1, int n_base, const float* xscale,
                                                   const float* wscale, const float* wbias, const Params& p) {
  const bool vec_ok = (p.N % 8) == 0;
  const int items = (t1 - t0) * 16;
  for (int i = threadIdx.x; i < items; i += kThreads) {
    const int tok = t0 + (i >> 4), g = i & 15;
    const uint32_t off = partial_u32 + static_cast<uint32_t>((tok * kSmallWRows + g * 8) * 4);
    float4 lo[S], hi[S];
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const uint32_t remote = ptx::mapa_u32(off, static_cast<uint32_t>(s));
      lo[s] = ld_shared_cluster_v4(remote);
      hi[s] = ld_shared_cluster_v4(remote + 16);
    }
    float acc[8] = {lo[0].x, lo[0].y, lo[0].z, lo[0].w, hi[0].x, hi[0].y, hi[0].z, hi[0].w};
#pragma unroll
    for (int s = 1; s < S; ++s) {
      acc[0] += lo[s].x, acc[1] += lo[s].y, acc[2] += lo[s].z, acc[3] += lo[s].w;
      acc[4] += hi[s].x, acc[5] += hi[s].y, acc[6] += hi[s].z, acc[7] += hi[s].w;
    }
    const float xs = xscale[tok];
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = g * 8 + 2 * j;
      const float x0 = fmaf(acc[2 * j] * xs, wscale[c], wbias[c]);
      const float x1 = fmaf(acc[2 * j + 1] * xs, wscale[c + 1], wbias[c + 1]);
      __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    const int n = n_base + g * 8;
    __nv_bfloat16* dst = p.out + static_cast<int64_t>(tok) * p.N + n;
    if (vec_ok && n + 8 <= p.N) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (n + j < p.N)
          reinterpret_cast<uint16_t*>(dst)[j] = (j & 1) ? static_cast<uint16_t>(w[j >> 1] >> 16) : static_cast<uint16_t>(w[j >> 1] & 0xffffu);
    }
  }
}

// tmap_w: weights [N, k_bytes], box 128 rows; tmap_x: activations [M, k_bytes], box `bt` rows
// (bt = M rounded up to 16).  `splits` = cluster size, `stages` = depth of the operand ring.
template <bool NVF4>
__global__ void __launch_bounds__(kThreads, 1)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const Params p,
                   const int splits, const int stages, const int bt) {
  using C = SmallCfg<NVF4>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int stage_bytes = C::stage_bytes(bt);
  const int x_bytes = bt * kBKBytes;
  uint8_t* tail = smem + stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_bar = full_bar + kSmallMaxStages;
  uint64_t* acc_full = empty_bar + kSmallMaxStages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tail + 256);
  volatile int* failed = reinterpret_cast<volatile int*>(tail + 260);
  uint64_t* sft_full = reinterpret_cast<uint64_t*>(tail + 384);   // NVFP4: a stage's scales are in tensor memory (4 warps)
  float* wscale = reinterpret_cast<float*>(tail + 512);   // [128] dequantization scale of each weight row
  float* wbias = wscale + 128;                            // [128]
  float* xscale = wbias + 128;                            // [128] dequantization scale of each token

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(ptx::cluster_ctarank());
  const int nb = blockIdx.x / splits;                     // one cluster per tile of 128 weight rows
  const int n_base = nb * kSmallWRows;
  const int k_tiles = (p.k_bytes + kBKBytes - 1) / kBKBytes;
  const int per = (k_tiles + splits - 1) / splits;
  const int kt0 = min(rank * per, k_tiles), kt1 = min(kt0 + per, k_tiles);
  const uint32_t tmem_cols = static_cast<uint32_t>(C::tmem_cols(stages));

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
      ptx::mbar_init(sft_full + s, 4);
    }
    ptx::mbar_init(acc_full, 1);
    *failed = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_w);
    ptx::prefetch_tmap(&tmap_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(tmem_holder, tmem_cols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_launch_dependents();   // the next kernel may be scheduled; it waits for this one before touching memory

  if (warp == 0 && lane == 0) {
    // ------------------------------------------------------------ TMA producer
    // Under programmatic dependent launch this kernel may start while the kernel before it on the
    // stream still runs.  When the caller promised that the weights are older than that kernel
    // (static_weights), the first ring of weight tiles is requested before waiting for it and only
    // the activation tiles (which it may still be writing) after; otherwise everything waits.
    const uint8_t* sfw_src = NVF4 ? p.sfb + static_cast<int64_t>(nb) * p.sf_col_tiles * 512 : nullptr;
    const uint8_t* sfx_src = NVF4 ? p.sfa : nullptr;
    auto sf_bytes_of = [&](int kt) -> uint32_t {
      return NVF4 ? static_cast<uint32_t>(min(4, p.sf_col_tiles - kt * 4)) * 512u : 0u;
    };
    auto issue_w = [&](int kt, int stage) {
      uint8_t* sw = smem + stage * stage_bytes;
      const uint32_t sfb = sf_bytes_of(kt);
      ptx::mbar_arrive_expect_tx(full_bar + stage, static_cast<uint32_t>(C::kWBytes + x_bytes) + 2u * sfb);
      ptx::tma_load_2d(sw, &tmap_w, full_bar + stage, kt * kBKBytes, n_base);
      if constexpr (NVF4) ptx::bulk_load(sw + C::kWBytes + x_bytes, sfw_src + kt * 2048, sfb, full_bar + stage);
    };
    auto issue_x = [&](int kt, int stage) {
      uint8_t* sx = smem + stage * stage_bytes + C::kWBytes;
      ptx::tma_load_2d(sx, &tmap_x, full_bar + stage, kt * kBKBytes, 0);
      if constexpr (NVF4) ptx::bulk_load(sx + x_bytes + 2048, sfx_src + kt * 2048, sf_bytes_of(kt), full_bar + stage);
    };
    const int pre = min(stages, kt1 - kt0);
    if (!p.static_weights) {   // the weights may come from the kernel before this one: wait first
      pdl_wait();
      ptx::fence_proxy_async_all();
    }
    for (int i = 0; i < pre; ++i) issue_w(kt0 + i, i);
    if (p.static_weights) {
      pdl_wait();
      ptx::fence_proxy_async_all();
    }
    for (int i = 0; i < pre; ++i) issue_x(kt0 + i, i);
    int stage = pre == stages ? 0 : pre;
    uint32_t phase = pre == stages ? 1u : 0u;
    for (int kt = kt0 + pre; kt < kt1; ++kt) {
      if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1u)) {
        raise_timeout(p.status, 31);
        *failed = 1;
        break;
      }
      issue_w(kt, stage);
      issue_x(kt, stage);
      if (++stage == stages) stage = 0, phase ^= 1u;
    }
  } else if (warp == 1 && lane == 0) {
    // ------------------------------------------------------------ MMA issuer (weights = A, tokens = B)
    const uint32_t idesc = NVF4 ? ptx::idesc_nvf4(kSmallWRows, bt) : ptx::idesc_f8(kSmallWRows, bt);
    const uint32_t smem_u = ptx::smem_u32(smem);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kt = kt0; kt < kt1; ++kt) {
      if (!ptx::mbar_wait(full_bar + stage, phase)) {
        raise_timeout(p.status, 32);
        *failed = 1;
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t sw = smem_u + stage * stage_bytes;
      const uint32_t w_lo = ptx::desc_lo_sw128(sw), x_lo = w_lo + (C::kWBytes >> 4);
      const uint32_t tmem_sfw = tmem_base + 128 + stage * C::kSfCols, tmem_sfx = tmem_sfw + 16;
      int kblocks = 4;
      if constexpr (NVF4) {
        kblocks = min(4, p.sf_col_tiles - kt * 4);
        // the stage's block scales are put into tensor memory by warps 2-5 (tcgen05.st from registers): a
        // tcgen05.cp costs about 50 tensor-pipe clocks and does not overlap MMAs, and a stage would need 8
        if (!ptx::mbar_wait(sft_full + stage, phase)) {
          raise_timeout(p.status, 34);
          *failed = 1;
          ok = false;
          break;
        }
        ptx::tc_fence_after();
      }
      for (int kb = 0; kb < kblocks; ++kb) {
        const uint32_t accum = (kt > kt0 || kb > 0) ? 1u : 0u;
        const uint64_t dw = ptx::desc_join(w_lo + kb * 2, ptx::kDescHiSw128);
        const uint64_t dx = ptx::desc_join(x_lo + kb * 2, ptx::kDescHiSw128);
        if constexpr (NVF4)
          ptx::mma_nvf4<1>(tmem_base, dw, dx, idesc, accum, tmem_sfw + kb * 4, tmem_sfx + kb * 4);
        else
          ptx::mma_f8<1>(tmem_base, dw, dx, idesc, accum);
      }
      ptx::tc_commit<1>(empty_bar + stage);
      if (++stage == stages) stage = 0, phase ^= 1u;
    }
    if (ok) ptx::tc_commit<1>(acc_full);
  } else if (warp >= 2) {
    // ------------------------------------------------------------ scales to shared memory, then park the partial tile
    const int q = warp & 3;
    const int wrow = q * 32 + lane;                      // weight row of the tile = tensor-memory lane
    {
      const int n = n_base + wrow;
      float ws = 1.0f, wb = 0.0f, xs = 0.0f;
      if (!p.static_weights) pdl_wait();
      if (n < p.N) {
        if constexpr (!NVF4) ws = __ldg(p.b_scales + static_cast<int64_t>(n) * p.b_scale_stride);
        if (p.bias != nullptr) wb = __bfloat162float(p.bias[n]);
      }
      pdl_wait();  // the activation scales come from the kernel before this one
      if (wrow < p.M) {
        if constexpr (NVF4) xs = __fmul_rn(__ldg(p.a_scales), __ldg(p.b_scales));
        else xs = __ldg(p.a_scales + static_cast<int64_t>(wrow) * p.a_scale_stride);
      }
      wscale[wrow] = ws;
      wbias[wrow] = wb;
      xscale[wrow] = xs;
    }
    if constexpr (NVF4) {
      // main loop: shared memory -> tensor memory for the scale tiles of every stage.  Lane l of each
      // lane quarter holds, per 512-byte scale tile, the 16 bytes at offset 16 l (4 columns): the layout
      // the block-scaled MMA reads, replicated in the four quarters.
      const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
      int stage = 0;
      uint32_t phase = 0;
      for (int kt = kt0; kt < kt1; ++kt) {
        if (!ptx::mbar_wait(full_bar + stage, phase)) {
          raise_timeout(p.status, 33);
          *failed = 1;
          break;
        }
        const uint8_t* sfw = smem + stage * stage_bytes + C::kWBytes + x_bytes + lane * 16;
        const uint8_t* sfx = sfw + 2048;
        uint32_t rw[16], rx[16];
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
          const uint4 a = *reinterpret_cast<const uint4*>(sfw + kb * 512);
          const uint4 b = *reinterpret_cast<const uint4*>(sfx + kb * 512);
          rw[kb * 4 + 0] = a.x, rw[kb * 4 + 1] = a.y, rw[kb * 4 + 2] = a.z, rw[kb * 4 + 3] = a.w;
          rx[kb * 4 + 0] = b.x, rx[kb * 4 + 1] = b.y, rx[kb * 4 + 2] = b.z, rx[kb * 4 + 3] = b.w;
        }
        const uint32_t dst = tmem_base + 128 + stage * C::kSfCols + lane_base;
        ptx::tmem_st_32x32_x16(dst, rw);
        ptx::tmem_st_32x32_x16(dst + 16, rx);
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(sft_full + stage);
        if (++stage == stages) stage = 0, phase ^= 1u;
      }
    }
    float* partial = reinterpret_cast<float*>(smem);     // [token][128 weight rows]: lanes hit consecutive banks
    const bool have = kt1 > kt0;
    bool ok = true;
    if (have) {
      ok = ptx::mbar_wait(acc_full, 0);
      if (!ok) {
        raise_timeout(p.status, 33);
        *failed = 1;
      }
    }
    ptx::tc_fence_after();
#pragma unroll 1
    for (int c = 0; c * 32 < p.M; ++c) {
      uint32_t r[32];
      if (have && ok) {
        ptx::tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + c * 32, r);
        ptx::tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c * 32 + j < p.M) partial[(c * 32 + j) * kSmallWRows + wrow] = __uint_as_float(r[j]);
    }
  }

  // all MMAs of this CTA have retired (the epilogue warps waited for them), the ring is idle:
  // partial tiles are complete cluster-wide after this barrier
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  pdl_wait();  // every thread stores to global memory below (returns at once: the producer already waited)

  if (*failed == 0) {
    // ------------------------------------------------------------ reduce my tokens over the cluster, scale, store
    const int per_rank = (p.M + splits - 1) / splits;
    const int t0 = min(rank * per_rank, p.M), t1 = min(t0 + per_rank, p.M);
    const uint32_t partial_u32 = ptx::smem_u32(smem);
    switch (splits) {
      case 1: small_reduce_store<1>(partial_u32, t0, t1, n_base, xscale, wscale, wbias, p); break;
      case 2: small_reduce_store<2>(partial_u32, t0, t1, n_base, xscale, wscale, wbias, p); break;
      case 4: small_reduce_store<4>(partial_u32, t0, t1, n_base, xscale, wscale, wbias, p); break;
      default: small_reduce_store<8>(partial_u32, t0, t1, n_base, xscale, wscale, wbias, p); break;
    }
  }

  __syncthreads();
  ptx::cluster_sync();  // nobody leaves while a peer may still read its partial tile
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, tmem_cols);
  }
}

}  // namespace gemm
}  // namespace b200q
