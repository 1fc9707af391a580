// CTA-pair variant of the quantized GEMM (tcgen05 cta_group::2), used when the problem has
// enough 256 x 256 output tiles to keep every SM pair busy.
//
// Two CTAs of a cluster (ranks 0 = leader, 1 = peer; two neighbouring SMs) share one 256 x 256
// output tile.  CTA r owns rows [128 r, 128 r + 128) of the tile: it loads that half of A and
// the half [128 r, 128 r + 128) of B's rows, and keeps its 128 x 256 slice of the accumulator
// in its own tensor memory.  One tcgen05.mma.cta_group::2 issued by the leader multiplies the
// pair's A halves with both B halves, so each CTA moves 32 KiB per K tile instead of the
// 48 KiB a single-CTA 128 x 256 tile needs, and one instruction stream feeds two SMs.
//
//   - TMA loads are issued by both CTAs into their own shared memory (cta_group::2, no
//     multicast); their byte counts are credited to the LEADER's `full` barrier.
//   - The leader's MMA thread releases a stage with a commit that arrives on the `empty`
//     barrier of both CTAs, and publishes a finished accumulator the same way.
//   - Epilogue warps of both CTAs arrive on the leader's `acc_empty` barrier (8 arrivals).
//   - NVFP4: each CTA loads the scale tiles of its own A rows and of all 256 B rows (3-D
//     tensor maps over the swizzled layout, zero fill past the end), tcgen05.cp
//     (cta_group::2) moves them to tensor memory in both CTAs.
//   - Both CTAs pass a cluster barrier before they free tensor memory and exit, so neither
//     leaves while the other can still touch its shared memory or barriers.
// Every wait is bounded exactly as in the single-CTA kernel.
#pragma once

#include "gemm_kernel.cuh"

namespace b200q {
namespace gemm {

constexpr int kPairM = 256;
constexpr int kPairN = 256;

template <bool NVF4>
struct Cfg2 {
  static constexpr int kABytes = 128 * kBKBytes;                    // this CTA's 128 rows of A
  static constexpr int kBBytes = (kPairN / 2) * kBKBytes;           // this CTA's 128 rows of B
  static constexpr int kSfaBytes = NVF4 ? 2048 : 0;
  static constexpr int kSfbBytes = NVF4 ? 4096 : 0;                 // scales of all 256 B rows
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kAccStages = NVF4 ? 1 : 2;
  static constexpr int kSfCols = NVF4 ? 48 : 0;
  static constexpr int kTailBytes = 2048;
  static constexpr int kEpiBytes = 2 * 2 * kPairN * 4;
  static constexpr int kPanelBytes = 32 * 128;
  static constexpr int kFixed = 1024 + kTailBytes + kEpiBytes;
  static constexpr int kStages2 = (kSmemLimit - kFixed - 4 * 2 * kPanelBytes) / kStageBytes;
  static constexpr int kStages1 = (kSmemLimit - kFixed - 4 * 1 * kPanelBytes) / kStageBytes;
  static constexpr int kEpiBufs = (kStages2 >= 5 || kStages2 == kStages1) ? 2 : 1;
  static constexpr int kStoreBytes = 4 * kEpiBufs * kPanelBytes;
  static constexpr int kStagesRaw = kEpiBufs == 2 ? kStages2 : kStages1;
  static constexpr int kStagesCap = NVF4 ? (512 - kAccStages * kPairN) / 48 : 8;   // tensor-memory columns for scales
  static constexpr int kStages = kStagesRaw > kStagesCap ? kStagesCap : kStagesRaw;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStoreBytes + kEpiBytes + kTailBytes;
  static constexpr int kColsNeeded = kAccStages * kPairN + kStages * kSfCols;
  static constexpr int kTmemCols = 512;
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert(kColsNeeded <= 512, "tensor memory overflow");
};

// SILU (FP8 only): the tile's B rows are 128 gate rows (loaded by the leader) and the matching 128 up rows
// (loaded by the peer, F rows further on), so accumulator columns 0..127 / 128..255 are a gate / up pair
// and the epilogue writes silu(gate) * up into out[M, F] (Params::silu_f = F): SILU = 1 as bf16, SILU = 2 as E4M3
// codes at the static per-tensor scale Params::act_amax / 448.
template <bool NVF4, int SILU = 0>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ OutMaps tmap_out, const __grid_constant__ CUtensorMap tmap_sfa,
                 const __grid_constant__ CUtensorMap tmap_sfb, const Params p) {
  using C = Cfg2<NVF4>;
  constexpr int BN = kPairN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* store_stage = smem + C::kStages * C::kStageBytes;
  float* epi = reinterpret_cast<float*>(store_stage + C::kStoreBytes);
  uint8_t* tail = store_stage + C::kStoreBytes + C::kEpiBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full = empty_bar + C::kStages;
  uint64_t* acc_empty = acc_full + C::kAccStages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + C::kAccStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int m_blocks = (p.M + kPairM - 1) / kPairM;
  const int n_blocks = SILU ? (p.silu_f + kPairN / 2 - 1) / (kPairN / 2) : (p.N + kPairN - 1) / kPairN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_tiles = (p.k_bytes + kBKBytes - 1) / kBKBytes;
  constexpr int kGroupM = 8;

  auto tile_coord = [&](int t, int& mb, int& nb) {
    const int per_group = kGroupM * n_blocks;
    const int g = t / per_group, r = t - g * per_group;
    const int rows_in_group = min(kGroupM, m_blocks - g * kGroupM);
    nb = r / rows_in_group;
    mb = g * kGroupM + (r - nb * rows_in_group);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
    }
    for (int s = 0; s < C::kAccStages; ++s) {
      ptx::mbar_init(acc_full + s, 1);
      ptx::mbar_init(acc_empty + s, 8);  // one arrival per epilogue warp of both CTAs
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    if (p.tma_store) ptx::prefetch_tmap(&tmap_out.m[0]);
  }
  if (warp == 1) {
    ptx::tmem_alloc<2>(tmem_holder, C::kTmemCols);
    ptx::tmem_relinquish<2>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // the peer's barriers are initialised before anything can arrive on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int mb, nb;
        tile_coord(t, mb, nb);
        const int32_t m0 = mb * kPairM + static_cast<int>(cta_rank) * 128;
        const int32_t n0 = SILU ? nb * (kPairN / 2) + static_cast<int>(cta_rank) * p.silu_f
                                : nb * kPairN + static_cast<int>(cta_rank) * (kPairN / 2);
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1u)) {
            raise_timeout(p.status, 11);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          const uint32_t leader_full = ptx::mapa_u32(ptx::smem_u32(full_bar + stage), 0);
          if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar + stage, 2u * C::kStageBytes);
          ptx::tma_load_2d_pair(sa, &tmap_a, leader_full, kt * kBKBytes, m0);
          ptx::tma_load_2d_pair(sb, &tmap_b, leader_full, kt * kBKBytes, n0);
          if constexpr (NVF4) {
            uint8_t* ssfa = sb + C::kBBytes;
            uint8_t* ssfb = ssfa + C::kSfaBytes;
            // [128 u32 of one 512-byte scale tile, column tile, row tile]: 4 column tiles of one
            // row tile of A, 4 x 2 of B; tiles past the end read as zero
            ptx::tma_load_3d_pair(ssfa, &tmap_sfa, leader_full, 0, kt * 4, mb * 2 + static_cast<int>(cta_rank));
            ptx::tma_load_3d_pair(ssfb, &tmap_sfb, leader_full, 0, kt * 4, nb * 2);
          }
          if (++stage == C::kStages) stage = 0, phase ^= 1u;
        }
      }
      for (int s = 0; s < C::kStages; ++s) {  // drain: all loads landed and were consumed
        const int st = (stage + s) % C::kStages;
        const uint32_t ph = (st >= stage) ? phase : (phase ^ 1u);
        if (!ptx::mbar_wait(empty_bar + st, ph ^ 1u)) {
          raise_timeout(p.status, 12);
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = NVF4 ? ptx::idesc_nvf4(kPairM, BN) : ptx::idesc_f8(kPairM, BN);
      constexpr uint32_t kStageStep = C::kStageBytes >> 4;
      const uint32_t smem_u = ptx::smem_u32(smem);
      const uint32_t a_lo0 = ptx::desc_lo_sw128(smem_u);
      const uint32_t tmem_sf0 = tmem_base + C::kAccStages * BN;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!ptx::mbar_wait(acc_empty + acc, acc_phase ^ 1u)) {
          raise_timeout(p.status, 13);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbar_wait(full_bar + stage, phase)) {
            raise_timeout(p.status, 14);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * kStageStep;
          const uint32_t b_lo = a_lo + (C::kABytes >> 4);
          const uint32_t tmem_sfa = tmem_sf0 + stage * C::kSfCols;
          const uint32_t tmem_sfb = tmem_sfa + 16;
          if constexpr (NVF4) {
            const uint32_t sfa_lo = (b_lo & 0x3fffu) + (C::kBBytes >> 4);
            const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
              ptx::tmem_cp_sf<2>(tmem_sfa + kb * 4, ptx::desc_join(sfa_lo + kb * 32, ptx::kDescHiSf));
#pragma unroll
              for (int j = 0; j < 2; ++j)
                ptx::tmem_cp_sf<2>(tmem_sfb + kb * 8 + j * 4, ptx::desc_join(sfb_lo + j * 128 + kb * 32, ptx::kDescHiSf));
            }
          }
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            const uint32_t accum = (kt > 0 || kb > 0) ? 1u : 0u;
            const uint64_t da = ptx::desc_join(a_lo + kb * 2, ptx::kDescHiSw128);
            const uint64_t db = ptx::desc_join(b_lo + kb * 2, ptx::kDescHiSw128);
            if constexpr (NVF4)
              ptx::mma_nvf4<2>(tmem_d, da, db, idesc, accum, tmem_sfa + kb * 4, tmem_sfb + kb * 8);
            else
              ptx::mma_f8<2>(tmem_d, da, db, idesc, accum);
          }
          ptx::tc_commit_pair(empty_bar + stage, 3);
          if (++stage == C::kStages) stage = 0, phase ^= 1u;
        }
        if (ok) ptx::tc_commit_pair(acc_full + acc, 3);
        if (++acc == C::kAccStages) acc = 0, acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    int sbuf = 0;
    bool dead = false;
    float gscale = 1.0f;
    if constexpr (NVF4) gscale = __fmul_rn(__ldg(p.a_scales), __ldg(p.b_scales));
    const bool vec_ok = (p.N % 8) == 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int mb, nb;
      tile_coord(t, mb, nb);
      const int n0 = SILU ? nb * (BN / 2) : nb * BN;     // first output column of the tile
      float* colscale = epi + buf * 2 * BN;
      float* colbias = colscale + BN;
      for (int i = et; i < BN; i += 128) {
        int n = n0 + i;
        bool valid = n < p.N;
        if constexpr (SILU) {                                // columns 0..127: gate rows n0 + i; 128..255: up rows F + n0 + i - 128
          n = i < BN / 2 ? n0 + i : p.silu_f + n0 + (i - BN / 2);
          valid = n0 + (i & (BN / 2 - 1)) < p.silu_f;
        }
        float s = 1.0f, b = 0.0f;
        if (valid) {
          if constexpr (!NVF4) s = __ldg(p.b_scales + static_cast<int64_t>(n) * p.b_scale_stride);
          if (p.bias != nullptr) b = __bfloat162float(p.bias[n]);
        }
        colscale[i] = s;
        colbias[i] = b;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      buf ^= 1;
      if (dead) continue;
      if (!ptx::mbar_wait(acc_full + acc, acc_phase)) {
        raise_timeout(p.status, 15);
        dead = true;
        continue;
      }
      ptx::tc_fence_after();
      const int row0 = mb * kPairM + static_cast<int>(cta_rank) * 128 + q * 32;
      const int row = row0 + lane;
      float rscale = gscale;
      if constexpr (!NVF4) rscale = (row < p.M) ? __ldg(p.a_scales + static_cast<int64_t>(row) * p.a_scale_stride) : 0.0f;
      __nv_bfloat16* orow = p.out + static_cast<int64_t>(row) * p.N + n0;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      // Row-parallel reduce-scatter mode: the 32-row panel goes to the rank that owns these rows,
      // into the slot of its receive buffer reserved for this rank.
      const CUtensorMap* omap = &tmap_out.m[0];
      int store_y = row0;
      if (p.rs_world > 1) {
        const int owner = row0 / p.rs_rows;
        omap = &tmap_out.m[owner];
        store_y = p.rs_rank * p.rs_rows + (row0 - owner * p.rs_rows);
      }
      uint64_t* release_bar = acc_empty + acc;
      if constexpr (SILU == 2) {
        const float qscale = fp8_scale_from_amax(__ldg(p.act_amax));
        if (t == 0 && cta_rank == 0 && et == 0 && p.act_scale_out != nullptr) p.act_scale_out[0] = qscale;
        uint8_t* crow = reinterpret_cast<uint8_t*>(p.out) + static_cast<int64_t>(row) * p.silu_f + n0;
        epilogue_tile_silu_quant(taddr, rscale, colscale, colbias, crow, row < p.M, n0, p.silu_f, qscale, b200q_rcp_rn(qscale),
                                 __fmul_rn(qscale, 512.0f), b200q_div_fast_ok(qscale), lane,
                                 [release_bar]() { ptx::mbar_arrive_cluster(release_bar, 0); });
      } else if constexpr (SILU == 1)
        epilogue_tile_silu<C::kEpiBufs, C::kPanelBytes>(taddr, rscale, colscale, colbias, store_stage + q * C::kEpiBufs * C::kPanelBytes,
                                                        sbuf, omap, store_y, row0, n0, p.M, p.silu_f, lane,
                                                        [release_bar]() { ptx::mbar_arrive_cluster(release_bar, 0); });
      else
        epilogue_tile<BN, C::kEpiBufs, C::kPanelBytes>(taddr, rscale, colscale, colbias, store_stage + q * C::kEpiBufs * C::kPanelBytes,
                                                       sbuf, omap, store_y, p.tma_store != 0, orow, row, row0, n0, p.M, p.N, vec_ok, lane,
                                                       [release_bar]() { ptx::mbar_arrive_cluster(release_bar, 0); });
      if (++acc == C::kAccStages) acc = 0, acc_phase ^= 1u;
    }
    if (lane == 0) {
      ptx::bulk_wait_group_read<0>();
      if (p.rs_world > 1) ptx::bulk_wait_group_all();  // stores to peers are complete before the kernel retires
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // neither CTA leaves while the other may still reach into it
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<2>(tmem_base, C::kTmemCols);
  }
}

}  // namespace gemm
}  // namespace b200q
