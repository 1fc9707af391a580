// NVFP4 CTA-pair GEMM (tcgen05.mma.cta_group::2 kind::mxf4nvf4.block_scale.block16), 256 x 256 tiles.
//
// Two CTAs of a cluster share one 256 x 256 output tile as in gemm_kernel_2cta.cuh: CTA r loads
// rows [128 r, 128 r + 128) of the A tile and of the B tile (32 KiB per 256-element K tile, against
// the 48 KiB of a single-CTA 128 x 256 tile) and keeps its 128 x 256 accumulator slice in its own
// tensor memory.  What differs from the generic pair kernel is everything the block scales need.
//
// The block scales reach tensor memory through ordinary warps (tcgen05.st), not through tcgen05.cp.
// Measured on this kernel shape: every tcgen05.cp (32x128b.warpx4, cta_group::2) takes about 50
// clocks of the tensor pipe and does not overlap the MMAs, whether it is issued in front of them,
// between them or a K tile ahead; the 12 copies of a K tile cost more than its four MMAs (512
// clocks).  Without the copies the same MMAs run at 124 clocks each.  So:
//
//   - Scales travel in their OWN shared-memory ring (6 KiB per K tile: this CTA's A-row scale
//     tiles and the scale tiles of all 256 B rows, two 3-D TMA loads over the swizzled layout, each
//     CTA on its own barrier); the operand ring holds plain 32 KiB stages, six of them.
//   - Four scale warps per CTA (one per tensor-memory lane quarter) read a K tile's scale tiles from
//     shared memory (16 bytes per lane and tile: exactly what tcgen05.cp 32x128b would put into that
//     lane) and store them into one of five scale buffers in tensor memory (48 columns each: all
//     256 columns the accumulator leaves free), up to four K tiles ahead of the MMAs.  The tensor
//     pipe executes MMAs only.
//   - One accumulator (256 columns).  Eight epilogue warps (two per lane quarter, 128 columns each)
//     pull it into registers in one go and hand tensor memory back BEFORE converting and storing,
//     so the next tile's MMAs wait for the loads only.  Registers are re-balanced between the
//     warpgroups (setmaxnreg) so that an epilogue thread can hold its 128 values.
//   - Signals whose payload is already complete (tensor-memory stores after tcgen05.wait::st,
//     tensor-memory loads after tcgen05.wait::ld) cross to the leader CTA with a RELAXED remote
//     arrive: a release at cluster scope costs on the order of a thousand clocks per arrive, which
//     at one arrive per K tile was the whole difference between 3.5 and 4.8 PFLOP/s.
//   - Output leaves in 32-byte row segments straight from registers (full sectors, no staging).
//   - K tails need no special path: the operand and scale loads zero-fill past the end, a zero
//     scale byte is 0.0, so the surplus MMAs add zeros.
//   warpgroup 0: warp 0 TMA producer, warp 1 MMA issue (leader CTA) and tensor-memory allocation
//   warpgroup 1: scale warps (lane quarter = warp & 3)
//   warpgroups 2, 3: epilogue (lane quarter = warp & 3, column half = warpgroup - 2)
// No TMA multicast; every wait is bounded as in the other kernels.
#pragma once

#include "gemm_kernel_2cta.cuh"

namespace b200q {
namespace gemm {

constexpr int kNvPairThreads = 512;

struct CfgNvPair {
  static constexpr int kABytes = 128 * kBKBytes;
  static constexpr int kBBytes = 128 * kBKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;                 // 32 KiB
  static constexpr int kSfaBytes = 2048;                                // 4 column tiles x 512 B (this CTA's 128 A rows)
  static constexpr int kSfbBytes = 4096;                                // the same for the two row tiles of B
  static constexpr int kSfEntryBytes = kSfaBytes + kSfbBytes;
  static constexpr int kSfEntries = 4;
  static constexpr int kTailBytes = 1024;
  static constexpr int kStages = (kSmemLimit - 1024 - kTailBytes - kSfEntries * kSfEntryBytes) / kStageBytes;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kSfEntries * kSfEntryBytes + kTailBytes;
  static constexpr int kSfCols = 48;                                    // 16 (A) + 32 (B, N = 256) per K tile
  static constexpr int kSfTmemBufs = 256 / kSfCols;                     // every column the accumulator leaves free
  static_assert(kStages >= 4, "pipeline too shallow");
};

// (a template only so that the definition may live in a header included by several translation units)
template <int kVariant = 0>
__global__ void __launch_bounds__(kNvPairThreads, 1)
gemm_nvf4_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb, const Params p) {
  using P = CfgNvPair;
  using C = CfgNvPair;
  constexpr int BN = kPairN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sf_smem = smem + C::kStages * P::kStageBytes;
  uint8_t* tail = sf_smem + C::kSfEntries * P::kSfEntryBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);           // leader: operands of both CTAs landed
  uint64_t* empty_bar = full_bar + C::kStages;                      // both: stage consumed (commit, multicast)
  uint64_t* sf_full = empty_bar + C::kStages;                       // own: scale entry landed in this CTA's shared memory
  uint64_t* sf_empty = sf_full + C::kSfEntries;                     // own: scale entry read by the 4 scale warps
  uint64_t* sft_full = sf_empty + C::kSfEntries;                    // leader: scale buffer written in both CTAs (8 warps)
  uint64_t* sft_empty = sft_full + C::kSfTmemBufs;                  // both: MMAs that read the buffer are complete
  uint64_t* acc_full = sft_empty + C::kSfTmemBufs;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int m_blocks = (p.M + kPairM - 1) / kPairM, n_blocks = (p.N + kPairN - 1) / kPairN;
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
    for (int s = 0; s < C::kSfEntries; ++s) {
      ptx::mbar_init(sf_full + s, 1);
      ptx::mbar_init(sf_empty + s, 4);
    }
    for (int s = 0; s < C::kSfTmemBufs; ++s) {
      ptx::mbar_init(sft_full + s, 8);
      ptx::mbar_init(sft_empty + s, 1);
    }
    ptx::mbar_init(acc_full, 1);
    ptx::mbar_init(acc_empty, 16);
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    ptx::prefetch_tmap(&tmap_sfa);
    ptx::prefetch_tmap(&tmap_sfb);
  }
  if (warp == 1) {
    ptx::tmem_alloc<2>(tmem_holder, 512);
    ptx::tmem_relinquish<2>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_sf0 = tmem_base + BN;

  if (warp < 4) {
    ptx::setmaxnreg_dec<64>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------ TMA producer (both CTAs)
      int stage = 0, entry = 0;
      uint32_t phase = 0, sf_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int mb, nb;
        tile_coord(t, mb, nb);
        const int32_t m0 = mb * kPairM + static_cast<int>(cta_rank) * 128;
        const int32_t n0 = nb * kPairN + static_cast<int>(cta_rank) * (kPairN / 2);
        for (int kt = 0; kt < k_tiles; ++kt) {
          {
            if (!ptx::mbar_wait(sf_empty + entry, sf_phase ^ 1u)) {
              raise_timeout(p.status, 41);
              ok = false;
              break;
            }
            uint8_t* ssfa = sf_smem + entry * P::kSfEntryBytes;
            uint8_t* ssfb = ssfa + P::kSfaBytes;
            ptx::mbar_arrive_expect_tx(sf_full + entry, P::kSfEntryBytes);
            ptx::tma_load_3d(ssfa, &tmap_sfa, sf_full + entry, 0, kt * 4, mb * 2 + static_cast<int>(cta_rank));
            ptx::tma_load_3d(ssfb, &tmap_sfb, sf_full + entry, 0, kt * 4, nb * 2);
            if (++entry == C::kSfEntries) entry = 0, sf_phase ^= 1u;
          }
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1u)) {
            raise_timeout(p.status, 42);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * P::kStageBytes;
          uint8_t* sb = sa + P::kABytes;
          const uint32_t leader_full = ptx::mapa_u32(ptx::smem_u32(full_bar + stage), 0);
          if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar + stage, 2u * P::kStageBytes);
          ptx::tma_load_2d_pair(sa, &tmap_a, leader_full, kt * kBKBytes, m0);
          ptx::tma_load_2d_pair(sb, &tmap_b, leader_full, kt * kBKBytes, n0);
          if (++stage == C::kStages) stage = 0, phase ^= 1u;
        }
      }
      for (int s = 0; s < C::kStages; ++s) {  // drain: all loads landed and were consumed
        const int st = (stage + s) % C::kStages;
        const uint32_t ph = (st >= stage) ? phase : (phase ^ 1u);
        if (!ptx::mbar_wait(empty_bar + st, ph ^ 1u)) {
          raise_timeout(p.status, 43);
          break;
        }
      }
      for (int s = 0; s < C::kSfEntries; ++s) {
        const int e = (entry + s) % C::kSfEntries;
        const uint32_t ph = (e >= entry) ? sf_phase : (sf_phase ^ 1u);
        if (!ptx::mbar_wait(sf_empty + e, ph ^ 1u)) {
          raise_timeout(p.status, 44);
          break;
        }
      }
    } else if (warp == 1 && lane == 0 && cta_rank == 0) {
      // ------------------------------------------------------------ MMA issuer (leader only): MMAs and commits, nothing else
      constexpr uint32_t idesc = ptx::idesc_nvf4(kPairM, BN);
      constexpr uint32_t kStageStep = P::kStageBytes >> 4;
      const uint32_t a_lo0 = ptx::desc_lo_sw128(ptx::smem_u32(smem));
      int stage = 0, tbuf = 0;
      uint32_t phase = 0, sft_phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!ptx::mbar_wait(acc_empty, acc_phase ^ 1u)) {
          raise_timeout(p.status, 45);
          break;
        }
        ptx::tc_fence_after();
        for (int kt = 0; kt < k_tiles; ++kt) {
          // this K tile's scales are in tensor-memory buffer `tbuf` (written by the scale warps of both CTAs)
          if (!ptx::mbar_wait(sft_full + tbuf, sft_phase)) {
            raise_timeout(p.status, 46);
            ok = false;
            break;
          }
          if (!ptx::mbar_wait(full_bar + stage, phase)) {
            raise_timeout(p.status, 47);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * kStageStep;
          const uint32_t b_lo = a_lo + (P::kABytes >> 4);
          const uint32_t sfa_t = tmem_sf0 + tbuf * P::kSfCols;
          const uint32_t sfb_t = sfa_t + 16;
#pragma unroll
          for (int kb = 0; kb < 4; ++kb) {
            const uint32_t accum = (kt > 0 || kb > 0) ? 1u : 0u;
            const uint64_t da = ptx::desc_join(a_lo + kb * 2, ptx::kDescHiSw128);
            const uint64_t db = ptx::desc_join(b_lo + kb * 2, ptx::kDescHiSw128);
            ptx::mma_nvf4<2>(tmem_base, da, db, idesc, accum, sfa_t + kb * 4, sfb_t + kb * 8);
          }
          ptx::tc_commit_pair(empty_bar + stage, 3);     // operand stage and scale buffer are free once these MMAs retire
          ptx::tc_commit_pair(sft_empty + tbuf, 3);
          if (++stage == C::kStages) stage = 0, phase ^= 1u;
          if (++tbuf == C::kSfTmemBufs) tbuf = 0, sft_phase ^= 1u;
        }
        if (ok) ptx::tc_commit_pair(acc_full, 3);
        acc_phase ^= 1u;
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------ scale warps (both CTAs): shared memory -> tensor memory
    ptx::setmaxnreg_dec<80>();
    const int q = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    int entry = 0, tbuf = 0;
    uint32_t sf_phase = 0, sft_phase = 0;
    const int my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
    const int groups = my_tiles * k_tiles;            // one scale entry per K tile
    for (int g = 0; g < groups; ++g) {
      if (!ptx::mbar_wait(sf_full + entry, sf_phase)) {
        raise_timeout(p.status, 48);
        break;
      }
      if (!ptx::mbar_wait(sft_empty + tbuf, sft_phase ^ 1u)) {
        raise_timeout(p.status, 49);
        break;
      }
      ptx::tc_fence_after();
      const uint8_t* ssfa = sf_smem + entry * P::kSfEntryBytes + lane * 16;
      const uint8_t* ssfb = ssfa + P::kSfaBytes;
      const uint32_t dst = tmem_sf0 + lane_base + tbuf * P::kSfCols;
      // lane l of every quarter holds, per 512-byte scale tile, the 16 bytes at offset 16 l: the scales
      // of rows l, l + 32, l + 64, l + 96 for the four 16-element blocks of one MMA (4 columns)
      uint32_t ra[16], rb[32];
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        const uint4 va = *reinterpret_cast<const uint4*>(ssfa + kb * 512);
        const uint4 v0 = *reinterpret_cast<const uint4*>(ssfb + kb * 512);            // B rows 0..127 of the tile
        const uint4 v1 = *reinterpret_cast<const uint4*>(ssfb + 2048 + kb * 512);     // B rows 128..255
        ra[kb * 4 + 0] = va.x, ra[kb * 4 + 1] = va.y, ra[kb * 4 + 2] = va.z, ra[kb * 4 + 3] = va.w;
        rb[kb * 8 + 0] = v0.x, rb[kb * 8 + 1] = v0.y, rb[kb * 8 + 2] = v0.z, rb[kb * 8 + 3] = v0.w;
        rb[kb * 8 + 4] = v1.x, rb[kb * 8 + 5] = v1.y, rb[kb * 8 + 6] = v1.z, rb[kb * 8 + 7] = v1.w;
      }
      ptx::tmem_st_32x32_x16(dst, ra);
      ptx::tmem_st_32x32_x16(dst + 16, rb);
      ptx::tmem_st_32x32_x16(dst + 32, rb + 16);
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(sf_empty + entry);                 // this CTA's shared-memory entry may be refilled
        // the leader's MMA thread counts 8 of these per buffer; the stores are complete (wait::st), so the
        // peer's signal needs no release
        if (cta_rank == 0) ptx::mbar_arrive(sft_full + tbuf);
        else ptx::mbar_arrive_cluster_relaxed(sft_full + tbuf, 0);
      }
      if (++entry == C::kSfEntries) entry = 0, sf_phase ^= 1u;
      if (++tbuf == C::kSfTmemBufs) tbuf = 0, sft_phase ^= 1u;
    }
  } else {
    // ------------------------------------------------------------ epilogue (warpgroups 2 and 3, both CTAs)
    ptx::setmaxnreg_inc<184>();
    const int q = warp & 3;                 // tensor-memory lane quarter this warp may read
    const int half = (warp - 8) >> 2;       // which 128 of the 256 accumulator columns
    uint32_t acc_phase = 0;
    const float gscale = __fmul_rn(__ldg(p.a_scales), __ldg(p.b_scales));
    const bool vec32 = (p.N % 16) == 0, vec16 = (p.N % 8) == 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int mb, nb;
      tile_coord(t, mb, nb);
      if (!ptx::mbar_wait(acc_full, acc_phase)) {
        raise_timeout(p.status, 50);
        break;
      }
      acc_phase ^= 1u;
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * 128;
      uint32_t r[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld_32x32(taddr + c * 32, r + c * 32);
      ptx::tmem_ld_wait();
      // the accumulator is in registers (the loads have completed): hand tensor memory back before
      // converting and storing; no release needed, nothing this warp wrote is part of the signal
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (cta_rank == 0) ptx::mbar_arrive(acc_empty);
        else ptx::mbar_arrive_cluster_relaxed(acc_empty, 0);
      }
      const int row = mb * kPairM + static_cast<int>(cta_rank) * 128 + q * 32 + lane;
      const int col0 = nb * BN + half * 128;
      if (row < p.M) {
        __nv_bfloat16* orow = p.out + static_cast<int64_t>(row) * p.N;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const int col = col0 + v * 16;
          if (col >= p.N) break;
          float x[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) x[i] = __uint_as_float(r[v * 16 + i]) * gscale;
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < p.N) x[i] += __bfloat162float(p.bias[col + i]);
          }
          U32x8 w;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            w.v[i] = *reinterpret_cast<uint32_t*>(&h2);
          }
          if (vec32 && col + 16 <= p.N) {
            st_256(orow + col, w);
          } else if (vec16 && col + 16 <= p.N) {
            *reinterpret_cast<uint4*>(orow + col) = make_uint4(w.v[0], w.v[1], w.v[2], w.v[3]);
            *reinterpret_cast<uint4*>(orow + col + 8) = make_uint4(w.v[4], w.v[5], w.v[6], w.v[7]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col + i < p.N) orow[col + i] = __float2bfloat16_rn(x[i]);
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<2>(tmem_base, 512);
  }
}

}  // namespace gemm
}  // namespace b200q
