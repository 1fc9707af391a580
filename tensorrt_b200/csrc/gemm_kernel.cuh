// Persistent, warp-specialised tcgen05 GEMM for quantized operands (sm_100a).
//
//   out[m, n] = epilogue( sum_k A[m, k] * B[n, k] )            A: [M, K], B: [N, K], both K-major
//
// FP8  (NVF4 = false): tcgen05.mma kind::f8f6f4, E4M3 x E4M3 -> fp32 in tensor memory;
//                      epilogue  acc * sa[m] * sb[n] + bias[n] -> bf16.
// NVFP4 (NVF4 = true): tcgen05.mma kind::mxf4nvf4.block_scale (block 16, UE4M3 scales);
//                      the 128x4 swizzled scale tiles are bulk-copied to shared memory and
//                      moved to tensor memory with tcgen05.cp before the MMAs of a K tile;
//                      epilogue  acc * (ga * gb) + bias[n] -> bf16.
//
// One CTA (192 threads, 224 for NVFP4) per SM walks over output tiles of 128 x BN:
//   warp 0      TMA producer: operand (and scale) tiles into a STAGES-deep shared-memory ring
//   warp 1      allocates tensor memory, issues the MMAs (one lane), commits to mbarriers
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp its own 32-lane quarter),
//               scale, add bias, convert, store; overlaps the next tile's main loop when
//               the accumulator is double-buffered in tensor memory
//   warp 6      NVFP4 only (launched with 224 threads): issues the tcgen05.cp scale copies of
//               every stage from its own thread and commits them to a per-stage barrier the
//               MMA thread waits on (measured 3-4 % faster than copies issued by the MMA thread)
// No TMA multicast is used anywhere.  Every mbarrier wait is bounded; a wait that gives up
// raises a flag in global memory, the CTA drains and leaves, and the host reports
// B200Q_ERR_TIMEOUT from b200q_device_status().
#pragma once

#include "common.cuh"
#include "tcgen05.cuh"

namespace b200q {
namespace gemm {

constexpr int kBM = 128;
constexpr int kBKBytes = 128;       // one 128-byte swizzle row of K per stage: 128 FP8 or 256 FP4 elements
constexpr int kMmaKBytes = 32;      // K bytes consumed by one tcgen05.mma (32 FP8 / 64 FP4 elements)
constexpr int kThreads = 192;
constexpr int kSmemLimit = 232448;  // 227 KiB

template <bool NVF4, int BN>
struct Cfg {
  static constexpr int kABytes = kBM * kBKBytes;
  static constexpr int kBBytes = BN * kBKBytes;
  static constexpr int kSfaBytes = NVF4 ? 2048 : 0;                 // 4 atoms of 512 B (128 rows x 16 scales)
  static constexpr int kSfbBytes = NVF4 ? (BN / 128) * 2048 : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kAccStages = (NVF4 && BN == 256) ? 1 : 2;
  static constexpr int kSfCols = NVF4 ? (16 + 4 * (BN / 32)) : 0;  // tensor-memory columns holding one K tile of scales
  static constexpr int kTailBytes = 2048;                           // barriers, tmem pointer
  static constexpr int kEpiBytes = 2 * 2 * BN * 4;                  // 2 buffers x (col scale, bias) x BN floats
  // Output staging for the TMA store: per epilogue warp kEpiBufs panels of 32 rows x 64 bf16
  // (4 KiB, 128-byte swizzled).  Two panels per warp unless that costs a pipeline stage.
  static constexpr int kPanelBytes = 32 * 128;
  static constexpr int kFixed = 1024 + kTailBytes + kEpiBytes;
  static constexpr int kStages2 = (kSmemLimit - kFixed - 4 * 2 * kPanelBytes) / kStageBytes;
  static constexpr int kStages1 = (kSmemLimit - kFixed - 4 * 1 * kPanelBytes) / kStageBytes;
  static constexpr int kEpiBufs = (kStages2 >= 4 || kStages2 == kStages1) ? 2 : 1;
  static constexpr int kStoreBytes = 4 * kEpiBufs * kPanelBytes;
  static constexpr int kStagesRaw = kEpiBufs == 2 ? kStages2 : kStages1;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStoreBytes + kEpiBytes + kTailBytes;
  // Each shared-memory stage owns its own scale-factor columns in tensor memory, so the
  // tcgen05.cp of K tile i+1 never has to wait for the MMAs of K tile i to finish reading.
  static constexpr int kColsNeeded = kAccStages * BN + kStages * kSfCols;
  static constexpr int kTmemCols = kColsNeeded <= 256 ? 256 : 512;
  static_assert(kStages >= 3, "pipeline too shallow");
  static_assert(kColsNeeded <= 512, "tensor memory overflow");
};

// Output tensor maps: m[0] is the local output; in reduce-scatter mode m[r] is rank r's receive
// buffer viewed as [world * rows_per_rank, N].
struct OutMaps {
  CUtensorMap m[8];
};

struct Params {
  const float* a_scales;   // FP8: [M] or [1]; NVFP4: pointer to the global scale of A
  const float* b_scales;   // FP8: [N] or [1]; NVFP4: pointer to the global scale of B
  int a_scale_stride;      // FP8: 1 (per row) or 0 (per tensor)
  int b_scale_stride;
  const uint8_t* sfa;      // NVFP4: swizzled block scales of A / B
  const uint8_t* sfb;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int M, N;
  int k_bytes;             // bytes per operand row (K for FP8, K/2 for NVFP4)
  int sf_col_tiles;        // NVFP4: number of 4-scale column tiles per row tile (ceil(K/64))
  int tma_store;           // 1: output leaves through TMA stores (needs N % 8 == 0), 0: direct stores
  int rs_world;            // > 1: reduce-scatter epilogue over `rs_world` ranks (TMA stores to peer buffers)
  int rs_rank;             //      this rank
  int rs_rows;             //      rows owned by each rank (M / rs_world, a multiple of 128)
  int static_weights;      // small-M kernel under programmatic dependent launch: 1 = B (weights, their scales, bias) was
                           // written before the preceding kernel on the stream started, so it may be read before
                           // waiting for that kernel; 0 = wait first
  int silu_f;              // FP8 CTA-pair kernel, > 0: B holds F gate rows then F up rows (N = 2 F); the epilogue
                           // writes out[M, F] = silu(gate) * up, each linear output rounded to bf16 first
  const float* act_amax;   // quantizing form of the above: static per-tensor abs-max of the activation; `out` then
  float* act_scale_out;    // receives E4M3 codes [M, F] (one byte each) and act_scale_out[0] the scale amax / 448
  int sf_copier;           // NVFP4, 1-CTA kernel: 1 = a dedicated warp (warp 6 of 224 threads) issues the tcgen05.cp scale copies
  int* status;             // device status word (0 = ok)
};

__device__ __forceinline__ void raise_timeout(int* status, int where) { atomicCAS(status, 0, where); }

// 32 columns of one accumulator row: scale, bias, convert to 16 packed bf16 pairs.
__device__ __forceinline__ void epilogue_convert(const uint32_t* r, float rscale, const float* colscale, const float* colbias,
                                                 uint32_t* w) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float x0 = fmaf(__uint_as_float(r[2 * j]) * rscale, colscale[2 * j], colbias[2 * j]);
    const float x1 = fmaf(__uint_as_float(r[2 * j + 1]) * rscale, colscale[2 * j + 1], colbias[2 * j + 1]);
    __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
}

// Direct (non-TMA) store of 32 converted columns of one row, with a scalar tail for ragged N.
__device__ __forceinline__ void epilogue_store_direct(__nv_bfloat16* orow_chunk, const uint32_t* w, int col0, int N, bool vec_ok) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const int col = col0 + v * 8;
    if (vec_ok && col + 8 <= N) {
      *reinterpret_cast<uint4*>(orow_chunk + v * 8) = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (col + j < N) {
          const uint32_t word = w[4 * v + (j >> 1)];
          const uint16_t hbits = (j & 1) ? static_cast<uint16_t>(word >> 16) : static_cast<uint16_t>(word & 0xffffu);
          reinterpret_cast<uint16_t*>(orow_chunk)[v * 8 + j] = hbits;
        }
      }
    }
  }
}

// Epilogue of one 128 x BN accumulator slice by one warp (lane quarter q): two register sets so
// that the tensor-memory load of chunk c+1 is in flight while chunk c is converted and stored.
// `release` is called once, right after the last tensor-memory load has completed.
template <int BN, int EPI_BUFS, int PANEL_BYTES, typename Release>
__device__ __forceinline__ void epilogue_tile(uint32_t taddr, float rscale, const float* colscale, const float* colbias,
                                              uint8_t* warp_panels, int& sbuf, const CUtensorMap* tmap_out, int store_y, bool tma_store,
                                              __nv_bfloat16* orow, int row, int row0, int n0, int M, int N, bool vec_ok, int lane,
                                              Release release) {
  uint32_t ra[32], rb[32];
  ptx::tmem_ld_32x32(taddr, ra);
#pragma unroll 1
  for (int c = 0; c < BN / 32; c += 2) {
    // ---- chunk c (in ra); prefetch c+1 into rb
    ptx::tmem_ld_wait();
    ptx::tmem_ld_32x32(taddr + (c + 1) * 32, rb);
    uint32_t w[16];
    epilogue_convert(ra, rscale, colscale + c * 32, colbias + c * 32, w);
    uint8_t* panel = warp_panels + sbuf * PANEL_BYTES;
    if (tma_store) {
      // two 32-column chunks fill one 64-column panel (32 rows x 128 bytes, 128-byte swizzle:
      // the 16-byte piece j of row r lands at piece j ^ (r & 7)), then one lane stores it
      if (lane == 0) ptx::bulk_wait_group_read<EPI_BUFS - 1>();
      __syncwarp();
#pragma unroll
      for (int v = 0; v < 4; ++v)
        *reinterpret_cast<uint4*>(panel + lane * 128 + ((v ^ (lane & 7)) * 16)) = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
    } else if (row < M) {
      epilogue_store_direct(orow + c * 32, w, n0 + c * 32, N, vec_ok);
    }
    // ---- chunk c+1 (in rb); prefetch c+2 into ra
    ptx::tmem_ld_wait();
    if (c + 2 < BN / 32) {
      ptx::tmem_ld_32x32(taddr + (c + 2) * 32, ra);
    } else {
      // the whole accumulator has been read: hand the tensor-memory buffer back before the
      // remaining conversion and stores
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) release();
    }
    epilogue_convert(rb, rscale, colscale + (c + 1) * 32, colbias + (c + 1) * 32, w);
    if (tma_store) {
#pragma unroll
      for (int v = 0; v < 4; ++v)
        *reinterpret_cast<uint4*>(panel + lane * 128 + (((4 + v) ^ (lane & 7)) * 16)) = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
      ptx::fence_proxy_async();
      __syncwarp();
      const int col0 = n0 + (c >> 1) * 64;
      if (lane == 0 && row0 < M && col0 < N) {
        ptx::tma_store_2d(tmap_out, panel, col0, store_y);
        ptx::bulk_commit_group();
      }
      if (++sbuf == EPI_BUFS) sbuf = 0;
    } else if (row < M) {
      epilogue_store_direct(orow + (c + 1) * 32, w, n0 + (c + 1) * 32, N, vec_ok);
    }
  }
}

// Epilogue of one 128 x 256 accumulator slice whose columns 0..127 are gate outputs and 128..255 the
// matching up outputs: both are scaled, biased and rounded to bf16 exactly as the plain epilogue does,
// then silu(gate) * up leaves as 64-column panels of the [M, F] activation (TMA stores only).
template <int EPI_BUFS, int PANEL_BYTES, typename Release>
__device__ __forceinline__ void epilogue_tile_silu(uint32_t taddr, float rscale, const float* colscale, const float* colbias,
                                                   uint8_t* warp_panels, int& sbuf, const CUtensorMap* tmap_out, int store_y, int row0,
                                                   int col0, int M, int F, int lane, Release release) {
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t rg[32], ru[32];
    ptx::tmem_ld_32x32(taddr + c * 32, rg);
    ptx::tmem_ld_32x32(taddr + 128 + c * 32, ru);
    ptx::tmem_ld_wait();
    if (c == 3) {   // the whole accumulator has been read: hand the tensor-memory buffer back
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) release();
    }
    uint32_t wg[16], wu[16], w[16];
    epilogue_convert(rg, rscale, colscale + c * 32, colbias + c * 32, wg);
    epilogue_convert(ru, rscale, colscale + 128 + c * 32, colbias + 128 + c * 32, wu);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float g0 = __uint_as_float(wg[j] << 16), g1 = __uint_as_float(wg[j] & 0xffff0000u);
      const float u0 = __uint_as_float(wu[j] << 16), u1 = __uint_as_float(wu[j] & 0xffff0000u);
      const __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul_f32(g0, u0), silu_mul_f32(g1, u1));
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    uint8_t* panel = warp_panels + sbuf * PANEL_BYTES;
    const int half = c & 1;
    if (half == 0) {
      if (lane == 0) ptx::bulk_wait_group_read<EPI_BUFS - 1>();
      __syncwarp();
    }
#pragma unroll
    for (int v = 0; v < 4; ++v)
      *reinterpret_cast<uint4*>(panel + lane * 128 + (((half * 4 + v) ^ (lane & 7)) * 16)) = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
    if (half == 1) {
      ptx::fence_proxy_async();
      __syncwarp();
      const int col = col0 + (c >> 1) * 64;
      if (lane == 0 && row0 < M && col < F) {
        ptx::tma_store_2d(tmap_out, panel, col, store_y);
        ptx::bulk_commit_group();
      }
      if (++sbuf == EPI_BUFS) sbuf = 0;
    }
  }
}

// The same with the activation quantized on the way out: silu(gate) * up is rounded to bf16 (the value the
// unfused graph would hand to its quantizer), divided by the static per-tensor scale with the exact-division
// sequence of the quantize kernels, and stored as E4M3 codes, 32 bytes per row and chunk (plain stores).
template <typename Release>
__device__ __forceinline__ void epilogue_tile_silu_quant(uint32_t taddr, float rscale, const float* colscale, const float* colbias,
                                                         uint8_t* crow, bool row_ok, int col0, int F, float scale, float y, float lim,
                                                         bool fast, int lane, Release release) {
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t rg[32], ru[32];
    ptx::tmem_ld_32x32(taddr + c * 32, rg);
    ptx::tmem_ld_32x32(taddr + 128 + c * 32, ru);
    ptx::tmem_ld_wait();
    if (c == 3) {
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) release();
    }
    uint32_t wg[16], wu[16];
    epilogue_convert(rg, rscale, colscale + c * 32, colbias + c * 32, wg);
    epilogue_convert(ru, rscale, colscale + 128 + c * 32, colbias + 128 + c * 32, wu);
    uint32_t codes[8];
#pragma unroll
    for (int j = 0; j < 16; j += 2) {
      float q[4];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float g0 = __uint_as_float(wg[j + e] << 16), g1 = __uint_as_float(wg[j + e] & 0xffff0000u);
        const float u0 = __uint_as_float(wu[j + e] << 16), u1 = __uint_as_float(wu[j + e] & 0xffff0000u);
        const __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul_f32(g0, u0), silu_mul_f32(g1, u1));
        const float a0 = __low2float(h), a1 = __high2float(h);
        q[2 * e] = fast ? div_path<kDivClamped>(a0, scale, y, lim) : div_path<kDivTrue>(a0, scale, y, lim);
        q[2 * e + 1] = fast ? div_path<kDivClamped>(a1, scale, y, lim) : div_path<kDivTrue>(a1, scale, y, lim);
      }
      codes[j >> 1] = f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16);
    }
    if (row_ok && col0 + c * 32 < F) {
      uint4* dst = reinterpret_cast<uint4*>(crow + c * 32);
      dst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
      dst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
    }
  }
}

template <bool NVF4, int BN>
__global__ void __launch_bounds__(kThreads + 32, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ OutMaps tmap_out, const Params p) {
  using C = Cfg<NVF4, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* store_stage = smem + C::kStages * C::kStageBytes;  // 1024-byte aligned panels
  float* epi = reinterpret_cast<float*>(store_stage + C::kStoreBytes);
  uint8_t* tail = store_stage + C::kStoreBytes + C::kEpiBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full = empty_bar + C::kStages;
  uint64_t* acc_empty = acc_full + C::kAccStages;
  uint64_t* sf_full = acc_empty + C::kAccStages;          // scales of a stage are in tensor memory (copier warp only)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(sf_full + C::kStages);
  volatile uint32_t* abort_flag = tmem_holder + 1;
  const bool copier = NVF4 && p.sf_copier != 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (p.M + kBM - 1) / kBM, n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_tiles = (p.k_bytes + kBKBytes - 1) / kBKBytes;
  constexpr int kGroupM = 16;

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
      ptx::mbar_init(sf_full + s, 1);
    }
    for (int s = 0; s < C::kAccStages; ++s) {
      ptx::mbar_init(acc_full + s, 1);
      ptx::mbar_init(acc_empty + s, 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_a);
    ptx::prefetch_tmap(&tmap_b);
    if (p.tma_store) ptx::prefetch_tmap(&tmap_out.m[0]);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(tmem_holder, C::kTmemCols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coord(t, mb, nb);
        // per-tile constants of the scale-factor loads
        const uint8_t* sfa_src = nullptr;
        const uint8_t* sfb_src[2] = {nullptr, nullptr};
        uint32_t sf_copies = 0;  // bulk copies per K tile: SFA + the live row tiles of SFB
        if constexpr (NVF4) {
          sfa_src = p.sfa + static_cast<int64_t>(mb) * p.sf_col_tiles * 512;
          sf_copies = 1;
          for (int j = 0; j < BN / 128; ++j) {
            const int rt = nb * (BN / 128) + j;
            if (rt * 128 < p.N) {
              sfb_src[j] = p.sfb + static_cast<int64_t>(rt) * p.sf_col_tiles * 512;
              ++sf_copies;
            }
          }
        }
        const int32_t m0 = mb * kBM, n0 = nb * BN;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbar_wait(empty_bar + stage, phase ^ 1u)) {
            raise_timeout(p.status, 1);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          uint32_t sf_bytes = 0;
          if constexpr (NVF4) sf_bytes = static_cast<uint32_t>(min(4, p.sf_col_tiles - kt * 4)) * 512u;
          ptx::mbar_arrive_expect_tx(full_bar + stage, C::kABytes + C::kBBytes + sf_copies * sf_bytes);
          ptx::tma_load_2d(sa, &tmap_a, full_bar + stage, kt * kBKBytes, m0);
          ptx::tma_load_2d(sb, &tmap_b, full_bar + stage, kt * kBKBytes, n0);
          if constexpr (NVF4) {
            uint8_t* ssfa = sb + C::kBBytes;
            uint8_t* ssfb = ssfa + C::kSfaBytes;
            ptx::bulk_load(ssfa, sfa_src + kt * 2048, sf_bytes, full_bar + stage);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              if (sfb_src[j] != nullptr) ptx::bulk_load(ssfb + j * 2048, sfb_src[j] + kt * 2048, sf_bytes, full_bar + stage);
          }
          if (++stage == C::kStages) stage = 0, phase ^= 1u;
        }
      }
      // Drain: every load issued above must have landed before this CTA's shared memory is
      // released.  The consumer arrives on `empty` only after `full` completed, so waiting
      // for the ring to become empty again (bounded) covers all loads in flight.
      for (int s = 0; s < C::kStages; ++s) {
        const int st = (stage + s) % C::kStages;
        const uint32_t ph = (st >= stage) ? phase : (phase ^ 1u);
        if (!ptx::mbar_wait(empty_bar + st, ph ^ 1u)) {
          raise_timeout(p.status, 2);
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // This single thread feeds the tensor pipe; its instruction stream per K tile has to
      // stay well below the ~512 cycles the four MMAs of a K tile take.  Descriptors are
      // kept as 32-bit low halves that advance by immediates, and the full-K-tile path is
      // completely unrolled.
      constexpr uint32_t idesc = NVF4 ? ptx::idesc_nvf4(kBM, BN) : ptx::idesc_f8(kBM, BN);
      constexpr uint32_t kStageStep = C::kStageBytes >> 4;
      const uint32_t smem_u = ptx::smem_u32(smem);
      const uint32_t a_lo0 = ptx::desc_lo_sw128(smem_u);
      const uint32_t tmem_sf0 = tmem_base + C::kAccStages * BN;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!ptx::mbar_wait(acc_empty + acc, acc_phase ^ 1u)) {
          raise_timeout(p.status, 3);
          *abort_flag = 1;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kt = 0; kt < k_tiles; ++kt) {
          if (!ptx::mbar_wait(full_bar + stage, phase)) {
            raise_timeout(p.status, 4);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if constexpr (NVF4) {
            if (copier && !ptx::mbar_wait(sf_full + stage, phase)) {
              raise_timeout(p.status, 6);
              *abort_flag = 1;
              ok = false;
              break;
            }
          }
          ptx::tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * kStageStep;          // A tile; B follows at +kABytes
          const uint32_t b_lo = a_lo + (C::kABytes >> 4);
          const uint32_t tmem_sfa = tmem_sf0 + stage * C::kSfCols;
          const uint32_t tmem_sfb = tmem_sfa + 16;
          int kblocks = kBKBytes / kMmaKBytes;
          if constexpr (NVF4) kblocks = min(4, p.sf_col_tiles - kt * 4);
          if (kblocks == 4) {
            if constexpr (NVF4) if (!copier) {
              const uint32_t sfa_lo = (b_lo & 0x3fffu) + (C::kBBytes >> 4);   // plain address field, no flags
              const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
#pragma unroll
              for (int kb = 0; kb < 4; ++kb) {
                ptx::tmem_cp_sf<1>(tmem_sfa + kb * 4, ptx::desc_join(sfa_lo + kb * 32, ptx::kDescHiSf));
#pragma unroll
                for (int j = 0; j < BN / 128; ++j)
                  ptx::tmem_cp_sf<1>(tmem_sfb + kb * (BN / 32) + j * 4, ptx::desc_join(sfb_lo + j * 128 + kb * 32, ptx::kDescHiSf));
              }
            }
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
              const uint32_t accum = (kt > 0 || kb > 0) ? 1u : 0u;
              const uint64_t da = ptx::desc_join(a_lo + kb * 2, ptx::kDescHiSw128);
              const uint64_t db = ptx::desc_join(b_lo + kb * 2, ptx::kDescHiSw128);
              if constexpr (NVF4)
                ptx::mma_nvf4<1>(tmem_d, da, db, idesc, accum, tmem_sfa + kb * 4, tmem_sfb + kb * (BN / 32));
              else
                ptx::mma_f8<1>(tmem_d, da, db, idesc, accum);
            }
          } else {
            // last, partial K tile of an NVFP4 problem whose K is not a multiple of 256
            const uint32_t sfa_lo = (b_lo & 0x3fffu) + (C::kBBytes >> 4);
            const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
            for (int kb = 0; kb < kblocks && !copier; ++kb) {
              ptx::tmem_cp_sf<1>(tmem_sfa + kb * 4, ptx::desc_join(sfa_lo + kb * 32, ptx::kDescHiSf));
              for (int j = 0; j < BN / 128; ++j)
                ptx::tmem_cp_sf<1>(tmem_sfb + kb * (BN / 32) + j * 4, ptx::desc_join(sfb_lo + j * 128 + kb * 32, ptx::kDescHiSf));
            }
            for (int kb = 0; kb < kblocks; ++kb) {
              const uint32_t accum = (kt > 0 || kb > 0) ? 1u : 0u;
              const uint64_t da = ptx::desc_join(a_lo + kb * 2, ptx::kDescHiSw128);
              const uint64_t db = ptx::desc_join(b_lo + kb * 2, ptx::kDescHiSw128);
              ptx::mma_nvf4<1>(tmem_d, da, db, idesc, accum, tmem_sfa + kb * 4, tmem_sfb + kb * (BN / 32));
            }
          }
          ptx::tc_commit<1>(empty_bar + stage);  // stage reusable once these MMAs (and copies) retire
          if (++stage == C::kStages) stage = 0, phase ^= 1u;
        }
        if (ok) ptx::tc_commit<1>(acc_full + acc);  // accumulator complete
        if (++acc == C::kAccStages) acc = 0, acc_phase ^= 1u;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ scale copier (NVFP4, optional 7th warp)
    // Issues the tcgen05.cp of every stage from its own thread, so that the copies of K tile
    // i + 1 are not queued between the MMAs of tiles i and i + 1 in the MMA thread's stream.
    // A stage's tensor-memory scale columns are free when its shared memory was refilled: the
    // producer waited for the MMAs of the previous use before it issued the loads.
    if constexpr (NVF4) {
      if (copier && lane == 0) {
        const uint32_t smem_u = ptx::smem_u32(smem);
        const uint32_t tmem_sf0 = tmem_base + C::kAccStages * BN;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          for (int kt = 0; kt < k_tiles; ++kt) {
            if (!ptx::mbar_wait(full_bar + stage, phase)) {
              raise_timeout(p.status, 7);
              *abort_flag = 1;
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t sfa_lo = ptx::desc_lo_sf(smem_u + stage * C::kStageBytes + C::kABytes + C::kBBytes);
            const uint32_t sfb_lo = sfa_lo + (C::kSfaBytes >> 4);
            const uint32_t tmem_sfa = tmem_sf0 + stage * C::kSfCols, tmem_sfb = tmem_sfa + 16;
            const int kblocks = min(4, p.sf_col_tiles - kt * 4);
            for (int kb = 0; kb < kblocks; ++kb) {
              ptx::tmem_cp_sf<1>(tmem_sfa + kb * 4, ptx::desc_join(sfa_lo + kb * 32, ptx::kDescHiSf));
#pragma unroll
              for (int j = 0; j < BN / 128; ++j)
                ptx::tmem_cp_sf<1>(tmem_sfb + kb * (BN / 32) + j * 4, ptx::desc_join(sfb_lo + j * 128 + kb * 32, ptx::kDescHiSf));
            }
            ptx::tc_commit<1>(sf_full + stage);
            if (++stage == C::kStages) stage = 0, phase ^= 1u;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const int et = threadIdx.x - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    int sbuf = 0;
    bool dead = false;
    float gscale = 1.0f;
    if constexpr (NVF4) gscale = __fmul_rn(__ldg(p.a_scales), __ldg(p.b_scales));
    const bool vec_ok = (p.N % 8) == 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int mb, nb;
      tile_coord(t, mb, nb);
      const int n0 = nb * BN;
      float* colscale = epi + buf * 2 * BN;
      float* colbias = colscale + BN;
      for (int i = et; i < BN; i += 128) {
        const int n = n0 + i;
        float s = 1.0f, b = 0.0f;
        if (n < p.N) {
          if constexpr (!NVF4) s = __ldg(p.b_scales + static_cast<int64_t>(n) * p.b_scale_stride);
          if (p.bias != nullptr) b = __bfloat162float(p.bias[n]);
        }
        colscale[i] = s;
        colbias[i] = b;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      buf ^= 1;

      // A warp whose wait gave up keeps walking the tile list (so the named barrier above
      // stays matched) but touches neither tensor memory nor the output again.
      if (dead) continue;
      if (!ptx::mbar_wait(acc_full + acc, acc_phase)) {
        raise_timeout(p.status, 5);
        dead = true;
        continue;
      }
      ptx::tc_fence_after();
      const int row0 = mb * kBM + q * 32;
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
      epilogue_tile<BN, C::kEpiBufs, C::kPanelBytes>(taddr, rscale, colscale, colbias, store_stage + q * C::kEpiBufs * C::kPanelBytes,
                                                     sbuf, omap, store_y, p.tma_store != 0, orow, row, row0, n0, p.M, p.N, vec_ok, lane,
                                                     [release_bar]() { ptx::mbar_arrive(release_bar); });
      if (++acc == C::kAccStages) acc = 0, acc_phase ^= 1u;
    }
    // shared memory must stay valid until the last store has read it
    if (lane == 0) {
      ptx::bulk_wait_group_read<0>();
      if (p.rs_world > 1) ptx::bulk_wait_group_all();  // stores to peers are complete before the kernel retires
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, C::kTmemCols);
  }
}

}  // namespace gemm
}  // namespace b200q
