// FP8 scaled-dot-product attention for Q, K, V that come out of `tensorrt::quantize_op(.., 8, 4, ..)`.
//
// The reference marks an SDPA whose three inputs are FP8 fake-quantized
// (py/torch_tensorrt/dynamo/lowering/passes/annotate_fp8_sdpa.py:34-76) and builds a TensorRT attention
// layer whose softmax output is quantized to FP8 with the data-independent scale 1/448, with a static
// 1/sqrt(D) factor on the query (py/torch_tensorrt/dynamo/conversion/impl/attention.py:272-283).  Here:
//
//   S = (Q_hat K_hat^T) * scale            Q_hat, K_hat, V_hat: E4M3 codes x per-tensor scale
//   P = softmax(S)  (optionally causal, lower-right aligned)
//   P_hat = e4m3(P * 448) / 448            exactly the normalized probabilities, quantized
//   O = P_hat V_hat
//
// Both contractions run on the tensor cores (tcgen05.mma kind::f8f6f4, accumulators in tensor memory).
// P_hat is the quantization of the NORMALIZED probabilities, so the row maximum and the row sum must be
// known before the first probability is quantized: the kernel makes two passes over the keys.  Pass 1
// computes Q K^T tile by tile and keeps the running maximum and sum per query row in registers; pass 2
// computes Q K^T again, turns every score into its final probability, quantizes it, writes the 128 x 128
// tile of codes to shared memory in the operand layout and multiplies it with the V tile.  The attention
// core is a few per cent of a decoder layer's arithmetic, so the repeated Q K^T is cheaper than a
// rescaling scheme whose quantization points would differ from the definition above.
//
// One CTA per (batch, head, 128 queries): warp 0 = TMA producer, warp 1 = MMA issue + tensor-memory
// allocation, warps 2-9 = softmax (two threads per query row, each half of the columns; lane quarter = warp & 3).  K and Q tiles are
// [rows, D] with D bytes per row (K-major), V is supplied TRANSPOSED per head ([D, keys], produced by
// b200q_fp8_quantize_transpose) so that the second contraction is K-major too.  D <= 128 (a multiple of
// 16); rows are zero-filled to 128 bytes by the TMA loads.  No TMA multicast; every wait is bounded.
#include "common.cuh"
#include "tcgen05.cuh"

#include <cuda.h>

namespace b200q {
namespace gemm {
int* device_status_word();
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled();
}  // namespace gemm

namespace {

constexpr int kAttThreads = 320;          // producer warp, MMA warp, 8 softmax warps
constexpr int kTile = 128;                 // queries per CTA, keys per step, padded head dimension
constexpr int kTileBytes = kTile * 128;    // one operand tile: 128 rows x 128 bytes
// Two CTAs per SM: while one waits for its tensor-core results the other's softmax warps have the issue
// slots.  Per CTA that leaves 6 operand tiles of shared memory (Q, 2 K stages, 1 V stage, 2 P tiles) and
// 256 columns of tensor memory: one output accumulator and one score tile.  The score tile is computed
// and consumed as two halves of 64 keys (two buffers of 64 columns), so that the tensor core fills one
// half while the softmax warps work on the other.
constexpr int kKStages = 2, kVStages = 1, kSBufs = 2;
constexpr int kHalf = kTile / 2;           // keys per score buffer
constexpr int kTmemCols = 256;
constexpr int kAttSmem = 1024 + kTileBytes * (1 + kKStages + kVStages + 2) + 4096;   // tail: barriers, row statistics

struct AttParams {
  const float* q_scale;     // per-tensor scales (device scalars)
  const float* k_scale;
  const float* v_scale;
  void* out;                // [B, Hq, Sq, D]
  int out_dtype;
  int Hq, Hkv, Sq, Sk, D;
  float softmax_scale;
  int causal;
  int* status;
};

__device__ __forceinline__ void att_timeout(int* status, int where) { atomicCAS(status, 0, where); }

// 2^x on the special-function unit (about 2 ulp; -inf -> 0, subnormal results flushed)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kAttThreads, 2)
fp8_sdpa_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_vt, const AttParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sq = smem;
  uint8_t* sk = sq + kTileBytes;
  uint8_t* sv = sk + kKStages * kTileBytes;
  uint8_t* sp = sv + kVStages * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sp + 2 * kTileBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + kKStages;
  uint64_t* v_full = k_empty + kKStages;
  uint64_t* v_empty = v_full + kVStages;
  uint64_t* s_full = v_empty + kVStages;     // score buffers in tensor memory
  uint64_t* s_empty = s_full + kSBufs;
  uint64_t* p_full = s_empty + kSBufs;       // 2 probability tiles in shared memory
  uint64_t* p_empty = p_full + 2;
  uint64_t* o_full = p_empty + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_full + 1);
  float2* row_stat = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(bars) + 1024);   // [2][kTile] (max, sum) of each column half

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * kTile;
  const int bh = blockIdx.y;                                  // b * Hq + h
  const int b = bh / p.Hq, h = bh - b * p.Hq;
  const int bhkv = b * p.Hkv + h / (p.Hq / p.Hkv);
  const int shift = p.Sk - p.Sq;                              // causal: key j visible to query i when j <= i + shift
  int k_end = p.Sk;
  if (p.causal) k_end = max(0, min(p.Sk, q0 + kTile + shift));
  const int n_tiles = (k_end + kTile - 1) / kTile;

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < kKStages; ++s) ptx::mbar_init(k_full + s, 1), ptx::mbar_init(k_empty + s, 1);
    for (int s = 0; s < kVStages; ++s) ptx::mbar_init(v_full + s, 1), ptx::mbar_init(v_empty + s, 1);
    for (int s = 0; s < kSBufs; ++s) {
      ptx::mbar_init(s_full + s, 1);
      ptx::mbar_init(s_empty + s, 8);   // one arrival per softmax warp
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(p_full + s, 8);
      ptx::mbar_init(p_empty + s, 1);
    }
    ptx::mbar_init(o_full, 1);
    ptx::fence_barrier_init();
    ptx::prefetch_tmap(&tmap_q);
    ptx::prefetch_tmap(&tmap_k);
    ptx::prefetch_tmap(&tmap_vt);
  }
  if (warp == 1) {
    ptx::tmem_alloc<1>(tmem_holder, kTmemCols);
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_o = tmem_base + kSBufs * kHalf;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(q_full, kTileBytes);
      ptx::tma_load_3d(sq, &tmap_q, q_full, 0, q0, bh);
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0;
      bool ok = true;
      for (int pass = 0; pass < 2 && ok; ++pass) {
        for (int j = 0; j < n_tiles; ++j) {
          if (!ptx::mbar_wait(k_empty + ks, kph ^ 1u)) {
            att_timeout(p.status, 61);
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(k_full + ks, kTileBytes);
          ptx::tma_load_3d(sk + ks * kTileBytes, &tmap_k, k_full + ks, 0, j * kTile, bhkv);
          if (++ks == kKStages) ks = 0, kph ^= 1u;
          if (pass == 1) {
            if (!ptx::mbar_wait(v_empty + vs, vph ^ 1u)) {
              att_timeout(p.status, 62);
              ok = false;
              break;
            }
            ptx::mbar_arrive_expect_tx(v_full + vs, kTileBytes);
            ptx::tma_load_3d(sv + vs * kTileBytes, &tmap_vt, v_full + vs, j * kTile, 0, bhkv);
            if (++vs == kVStages) vs = 0, vph ^= 1u;
          }
        }
      }
      // drain: every load issued above has landed and was consumed before shared memory is released
      for (int s = 0; s < kKStages && ok; ++s) {
        const int st = (ks + s) % kKStages;
        const uint32_t ph = (st >= ks) ? kph : (kph ^ 1u);
        if (!ptx::mbar_wait(k_empty + st, ph ^ 1u)) att_timeout(p.status, 63), ok = false;
      }
      for (int s = 0; s < kVStages && ok; ++s) {
        const int st = (vs + s) % kVStages;
        const uint32_t ph = (st >= vs) ? vph : (vph ^ 1u);
        if (!ptx::mbar_wait(v_empty + st, ph ^ 1u)) att_timeout(p.status, 64), ok = false;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::idesc_f8(kTile, kTile);
      const uint32_t q_lo = ptx::desc_lo_sw128(ptx::smem_u32(sq));
      const uint32_t k_lo0 = ptx::desc_lo_sw128(ptx::smem_u32(sk));
      const uint32_t v_lo0 = ptx::desc_lo_sw128(ptx::smem_u32(sv));
      const uint32_t p_lo0 = ptx::desc_lo_sw128(ptx::smem_u32(sp));
      int ks = 0, vs = 0, sb = 0, pb = 0;
      uint32_t kph = 0, vph = 0, sph = 0, pph = 0;
      bool ok = ptx::mbar_wait(q_full, 0);
      if (!ok) att_timeout(p.status, 65);
      // S[sb] = Q K^T for the two halves (64 keys each) of the next key tile in ring order
      constexpr uint32_t idesc_half = ptx::idesc_f8(kTile, kHalf);
      auto issue_scores = [&]() -> bool {
        if (!ptx::mbar_wait(k_full + ks, kph)) {
          att_timeout(p.status, 66);
          return false;
        }
        for (int hh = 0; hh < 2; ++hh) {
          if (!ptx::mbar_wait(s_empty + sb, sph ^ 1u)) {
            att_timeout(p.status, 66);
            return false;
          }
          ptx::tc_fence_after();
          // keys 64 hh .. 64 hh + 63 of the stage: 64 rows of 128 bytes further on (whole swizzle atoms)
          const uint32_t k_lo = k_lo0 + ks * (kTileBytes >> 4) + hh * ((kHalf * 128) >> 4);
#pragma unroll
          for (int kb = 0; kb < 4; ++kb)
            ptx::mma_f8<1>(tmem_base + sb * kHalf, ptx::desc_join(q_lo + kb * 2, ptx::kDescHiSw128),
                           ptx::desc_join(k_lo + kb * 2, ptx::kDescHiSw128), idesc_half, kb > 0 ? 1u : 0u);
          ptx::tc_commit<1>(s_full + sb);
          if (++sb == kSBufs) sb = 0, sph ^= 1u;
        }
        ptx::tc_commit<1>(k_empty + ks);
        if (++ks == kKStages) ks = 0, kph ^= 1u;
        return true;
      };
      for (int j = 0; j < n_tiles && ok; ++j) ok = issue_scores();         // pass 1: scores only
      if (ok && n_tiles > 0) ok = issue_scores();                          // pass 2, first tile
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_scores();                          // scores of tile j + 1 under the softmax of tile j
        if (!ok) break;
        if (!ptx::mbar_wait(p_full + pb, pph) || !ptx::mbar_wait(v_full + vs, vph)) {
          att_timeout(p.status, 67);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t p_lo = p_lo0 + pb * (kTileBytes >> 4);
        const uint32_t v_lo = v_lo0 + vs * (kTileBytes >> 4);
#pragma unroll
        for (int kb = 0; kb < 4; ++kb)
          ptx::mma_f8<1>(tmem_o, ptx::desc_join(p_lo + kb * 2, ptx::kDescHiSw128), ptx::desc_join(v_lo + kb * 2, ptx::kDescHiSw128),
                         idesc, (j > 0 || kb > 0) ? 1u : 0u);
        ptx::tc_commit<1>(p_empty + pb);
        ptx::tc_commit<1>(v_empty + vs);
        if (++vs == kVStages) vs = 0, vph ^= 1u;
        if (++pb == 2) pb = 0, pph ^= 1u;
      }
      if (ok) ptx::tc_commit<1>(o_full);
    }
  } else {
    // ------------------------------------------------------------ softmax (warps 2..9): two threads per query row.
    // A warp reaches the 32 tensor-memory lanes of its quarter (warp & 3); the two warps of a quarter split
    // the columns: of every 64-key score buffer (and of the output) warp set `ch` takes the 32-column chunk ch.
    const int q = warp & 3;
    const int ch = (warp - 2) >> 2;
    const int r = q * 32 + lane;                  // row inside the tile
    const int qi = q0 + r;                        // query index inside the head
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    // scores in the base-2 exponent domain: s2 = acc * c2, c2 = q_scale * k_scale * softmax_scale * log2(e) > 0,
    // so the running maximum is kept on the raw accumulators and the scaling rides in the FMA in front of ex2
    const float c2 = __ldg(p.q_scale) * __ldg(p.k_scale) * p.softmax_scale * 1.4426950408889634f;
    const int last_key = p.causal ? min(k_end - 1, qi + shift) : k_end - 1;   // keys beyond it are masked for this row
    // key tiles below this index are visible to every row of the CTA in full: no per-element mask there
    const int full_tiles = (p.causal ? max(0, min(k_end, q0 + shift + 1)) : k_end) / kTile;
    int sb = 0, pb = 0;
    uint32_t sph = 0, pph = 0;
    float m = -INFINITY, l = 0.0f;                // raw-accumulator maximum, sum of 2^(s2 - m * c2)
    bool ok = true;
    // ---- pass 1: running maximum and sum, one half tile (64 keys) per step
    for (int t = 0; t < 2 * n_tiles && ok; ++t) {
      if (!ptx::mbar_wait(s_full + sb, sph)) {
        att_timeout(p.status, 68);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const bool masked = (t >> 1) >= full_tiles;
      {
        const int c = ch;
        uint32_t v[32];
        ptx::tmem_ld_32x32(tmem_base + lane_addr + sb * kHalf + c * 32, v);
        ptx::tmem_ld_wait();
        if (masked) {
          const int key0 = t * kHalf + c * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + i > last_key) v[i] = 0xff800000u;   // -inf
        }
        // four independent chains each for the maximum and the sum: a warp has few neighbours on its scheduler
        // here, so the length of a dependent chain is what it waits for
        float c0 = __uint_as_float(v[0]), c1 = __uint_as_float(v[1]), c2m = __uint_as_float(v[2]), c3 = __uint_as_float(v[3]);
#pragma unroll
        for (int i = 4; i < 32; i += 4) {
          c0 = fmaxf(c0, __uint_as_float(v[i]));
          c1 = fmaxf(c1, __uint_as_float(v[i + 1]));
          c2m = fmaxf(c2m, __uint_as_float(v[i + 2]));
          c3 = fmaxf(c3, __uint_as_float(v[i + 3]));
        }
        const float cm = fmaxf(fmaxf(c0, c1), fmaxf(c2m, c3));
        if (cm > m) {
          l *= ex2_approx((m - cm) * c2);         // m = -inf: l is 0 and stays 0
          m = cm;
        }
        if (m > -INFINITY) {
          const float off = -m * c2;
          float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            l0 += ex2_approx(fmaf(__uint_as_float(v[i]), c2, off));
            l1 += ex2_approx(fmaf(__uint_as_float(v[i + 1]), c2, off));
            l2 += ex2_approx(fmaf(__uint_as_float(v[i + 2]), c2, off));
            l3 += ex2_approx(fmaf(__uint_as_float(v[i + 3]), c2, off));
          }
          l += (l0 + l1) + (l2 + l3);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(s_empty + sb);
      if (++sb == kSBufs) sb = 0, sph ^= 1u;
    }
    // the two threads of a row each hold the statistics of their columns: merge (every softmax thread gets here)
    row_stat[ch * kTile + r] = make_float2(m, l);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    {
      const float2 o = row_stat[(ch ^ 1) * kTile + r];
      const float mm = fmaxf(m, o.x);
      const float mine = m > -INFINITY ? l * ex2_approx((m - mm) * c2) : 0.0f;
      const float theirs = o.x > -INFINITY ? o.y * ex2_approx((o.x - mm) * c2) : 0.0f;
      l = mine + theirs;
      m = mm;
    }
    // ---- pass 2: final probabilities, quantized with scale 1/448, written as the A operand of P V:
    // 448 * 2^(s2 - m2) / l = 2^(acc * c2 + off2) with the normaliser folded into the exponent
    const float off2 = l > 0.0f ? -m * c2 + __log2f(kE4M3Max / l) : -INFINITY;
    for (int t = 0; t < 2 * n_tiles && ok; ++t) {
      const int hh = t & 1;
      if (!ptx::mbar_wait(s_full + sb, sph) || (hh == 0 && !ptx::mbar_wait(p_empty + pb, pph ^ 1u))) {
        att_timeout(p.status, 69);
        ok = false;
        break;
      }
      ptx::tc_fence_after();
      const bool masked = (t >> 1) >= full_tiles;
      uint8_t* prow = sp + pb * kTileBytes + r * 128;
      {
        const int c = ch;
        uint32_t v[32];
        ptx::tmem_ld_32x32(tmem_base + lane_addr + sb * kHalf + c * 32, v);
        ptx::tmem_ld_wait();
        if (masked) {
          const int key0 = t * kHalf + c * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + i > last_key) v[i] = 0xff800000u;   // -inf -> probability 0
        }
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float pr[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) pr[e] = ex2_approx(fmaf(__uint_as_float(v[4 * i + e]), c2, off2));
          w[i] = f32x2_to_e4m3x2(pr[0], pr[1]) | (f32x2_to_e4m3x2(pr[2], pr[3]) << 16);
        }
        // 128-byte swizzle of the operand layout: the 16-byte piece i of row r lives at piece i ^ (r & 7)
        const int piece = 2 * (hh * 2 + c);
        *reinterpret_cast<uint4*>(prow + ((piece ^ (r & 7)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(prow + (((piece + 1) ^ (r & 7)) * 16)) = make_uint4(w[4], w[5], w[6], w[7]);
      }
      if (hh == 1) ptx::fence_proxy_async();      // the tensor core reads this tile through the async proxy
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (hh == 1) ptx::mbar_arrive(p_full + pb);
        ptx::mbar_arrive(s_empty + sb);
      }
      if (++sb == kSBufs) sb = 0, sph ^= 1u;
      if (hh == 1 && ++pb == 2) pb = 0, pph ^= 1u;
    }
    // ---- output: O * (v_scale / 448) -> out dtype
    if (ok && n_tiles > 0 && !ptx::mbar_wait(o_full, 0)) {
      att_timeout(p.status, 70);
      ok = false;
    }
    // tcgen05.ld is a warp-wide instruction: every lane of the warp takes part in the loads, rows past the
    // end of the sequence only skip their stores
    if (ok && q0 + q * 32 < p.Sq) {
      ptx::tc_fence_after();
      const float oscale = n_tiles > 0 ? __ldg(p.v_scale) / kE4M3Max : 0.0f;
      const int64_t row_off = (static_cast<int64_t>(bh) * p.Sq + qi) * p.D;
#pragma unroll 1
      for (int c = 2 * ch; c < 2 * ch + 2; ++c) {
        if (c * 32 >= p.D) break;
        uint32_t v[32];
        if (n_tiles > 0) {
          ptx::tmem_ld_32x32(tmem_o + lane_addr + c * 32, v);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {             // 8 columns per store
          const int col = c * 32 + g * 8;
          if (col >= p.D || qi >= p.Sq) break;
          float x[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = __uint_as_float(v[g * 8 + i]) * oscale;
          if (p.out_dtype == B200Q_BF16) Elem<__nv_bfloat16>::store8(static_cast<__nv_bfloat16*>(p.out) + row_off + col, x);
          else if (p.out_dtype == B200Q_F16) Elem<__half>::store8(static_cast<__half*>(p.out) + row_off + col, x);
          else Elem<float>::store8(static_cast<float*>(p.out) + row_off + col, x);
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

// x [heads, S, D] -> E4M3 codes transposed per head [heads, D, s_stride] (keys contiguous), zero beyond S.
template <typename T>
__global__ void __launch_bounds__(256)
fp8_quantize_transpose_kernel(const T* __restrict__ x, const float* __restrict__ amax, uint8_t* __restrict__ out, int S, int D,
                              int64_t s_stride, float* __restrict__ scale_out) {
  __shared__ uint8_t tile[64][128 + 16];
  const int head = blockIdx.y;
  const int k0 = blockIdx.x * 64;
  const float scale = fp8_scale_from_amax(__ldg(amax));
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && scale_out != nullptr) *scale_out = scale;
  const float y = b200q_rcp_rn(scale);
  const bool fast = b200q_div_fast_ok(scale);
  const float lim = __fmul_rn(scale, 512.0f);   // |x| >= 512 * scale saturates to 448 anyway
  const int groups = D >> 3;
  for (int t = threadIdx.x; t < 64 * groups; t += 256) {
    const int kk = t / groups, g = t - kk * groups;
    uint2 packed = make_uint2(0u, 0u);
    if (k0 + kk < S) {
      float v[8], qv[8];
      Elem<T>::load8(x + (static_cast<int64_t>(head) * S + k0 + kk) * D + g * 8, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) qv[i] = fast ? div_path<kDivClamped>(v[i], scale, y, lim) : div_path<kDivTrue>(v[i], scale, y, lim);
      packed.x = f32x2_to_e4m3x2(qv[0], qv[1]) | (f32x2_to_e4m3x2(qv[2], qv[3]) << 16);
      packed.y = f32x2_to_e4m3x2(qv[4], qv[5]) | (f32x2_to_e4m3x2(qv[6], qv[7]) << 16);
    }
    *reinterpret_cast<uint2*>(&tile[kk][g * 8]) = packed;
  }
  __syncthreads();
  // every (d, 16-key piece) is one 16-byte store
  for (int t = threadIdx.x; t < D * 4; t += 256) {
    const int d = t >> 2, part = t & 3;
    if (k0 + part * 16 >= s_stride) continue;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      w[i] = 0u;
#pragma unroll
      for (int e = 0; e < 4; ++e) w[i] |= static_cast<uint32_t>(tile[part * 16 + i * 4 + e][d]) << (8 * e);
    }
    *reinterpret_cast<uint4*>(out + (static_cast<int64_t>(head) * D + d) * s_stride + k0 + part * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// [inner bytes, rows, heads] byte tensor -> boxes of 128 x 128 x 1, 128-byte swizzle, zero fill out of bounds
int make_head_map(CUtensorMap* map, const void* base, int64_t inner, int64_t rows, int64_t heads, int64_t row_stride) {
  gemm::EncodeTiledFn fn = gemm::encode_tiled();
  if (fn == nullptr) return B200Q_ERR_CUDA;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride), static_cast<cuuint64_t>(row_stride * rows)};
  const cuuint32_t box[3] = {128, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200Q_OK : B200Q_ERR_CUDA;
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_fp8_quantize_transpose(const void* x, int dtype, int64_t heads, int64_t S, int64_t D, const float* amax, uint8_t* out_t,
                                 int64_t s_stride, float* scale_out, b200q_stream_t stream) {
  if (heads < 0 || S < 0 || D <= 0 || D > 128 || D % 16 != 0 || s_stride < S || s_stride % 16 != 0 || heads > 65535) return B200Q_ERR_INVALID;
  if (heads == 0 || S == 0) return B200Q_OK;
  if (x == nullptr || amax == nullptr || out_t == nullptr) return B200Q_ERR_INVALID;
  if (!aligned(x, 16) || !aligned(out_t, 16) || (dtype == B200Q_F32 && !aligned(x, 32))) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const dim3 grid(static_cast<unsigned>((s_stride + 63) / 64), static_cast<unsigned>(heads));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int s = static_cast<int>(S), d = static_cast<int>(D);
  switch (dtype) {
    case B200Q_BF16: fp8_quantize_transpose_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), amax, out_t, s, d, s_stride, scale_out); break;
    case B200Q_F16: fp8_quantize_transpose_kernel<<<grid, 256, 0, st>>>(static_cast<const __half*>(x), amax, out_t, s, d, s_stride, scale_out); break;
    case B200Q_F32: fp8_quantize_transpose_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(x), amax, out_t, s, d, s_stride, scale_out); break;
    default: return B200Q_ERR_INVALID;
  }
  return check_launch();
}

int b200q_fp8_sdpa(const uint8_t* q_codes, const uint8_t* k_codes, const uint8_t* vt_codes, const float* q_scale, const float* k_scale,
                   const float* v_scale, void* out, int out_dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Sk,
                   int64_t vt_stride, int64_t D, float softmax_scale, int causal, b200q_stream_t stream) {
  if (B < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Sq < 0 || Sk < 0 || D <= 0 || D > 128 || D % 16 != 0) return B200Q_ERR_INVALID;
  if (vt_stride < Sk || vt_stride % 16 != 0 || B * Hq > 65535 || Sq > 0x7fffffffLL || Sk > 0x7fffffffLL) return B200Q_ERR_INVALID;
  if (out_dtype != B200Q_BF16 && out_dtype != B200Q_F16 && out_dtype != B200Q_F32) return B200Q_ERR_INVALID;
  if (!(softmax_scale > 0.0f)) return B200Q_ERR_INVALID;
  if (B == 0 || Sq == 0) return B200Q_OK;
  if (q_codes == nullptr || out == nullptr || q_scale == nullptr || k_scale == nullptr || v_scale == nullptr) return B200Q_ERR_INVALID;
  if (Sk > 0 && (k_codes == nullptr || vt_codes == nullptr)) return B200Q_ERR_INVALID;
  if (!aligned(q_codes, 16) || !aligned(k_codes, 16) || !aligned(vt_codes, 16) || !aligned(out, 32)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  AttParams p{};
  p.status = gemm::device_status_word();
  if (p.status == nullptr) return B200Q_ERR_CUDA;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200Q_ERR_CUDA;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(fp8_sdpa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttSmem) != cudaSuccess) return B200Q_ERR_CUDA;
    configured[dev] = true;
  }
  CUtensorMap tq, tk, tv;
  // a zero-length key axis still needs valid maps: the kernel then loads nothing and writes zeros
  const int64_t sk_map = Sk > 0 ? Sk : 1;
  const void* kbase = Sk > 0 ? static_cast<const void*>(k_codes) : static_cast<const void*>(q_codes);
  const void* vbase = Sk > 0 ? static_cast<const void*>(vt_codes) : static_cast<const void*>(q_codes);
  if (int rc = make_head_map(&tq, q_codes, D, Sq, B * Hq, D)) return rc;
  if (int rc = make_head_map(&tk, kbase, D, sk_map, B * Hkv, D)) return rc;
  if (int rc = make_head_map(&tv, vbase, Sk > 0 ? Sk : 16, D, B * Hkv, Sk > 0 ? vt_stride : 16)) return rc;
  p.q_scale = q_scale;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.out = out;
  p.out_dtype = out_dtype;
  p.Hq = static_cast<int>(Hq);
  p.Hkv = static_cast<int>(Hkv);
  p.Sq = static_cast<int>(Sq);
  p.Sk = static_cast<int>(Sk);
  p.D = static_cast<int>(D);
  p.softmax_scale = softmax_scale;
  p.causal = causal ? 1 : 0;
  const dim3 grid(static_cast<unsigned>((Sq + kTile - 1) / kTile), static_cast<unsigned>(B * Hq));
  fp8_sdpa_kernel<<<grid, kAttThreads, kAttSmem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  return check_launch();
}

}  // extern "C"
