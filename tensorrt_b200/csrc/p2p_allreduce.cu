// Second half of the fused row-parallel linear: reduce + all-gather over peer memory.
//
// The GEMM's reduce-scatter epilogue (gemm_kernel.cuh, rs_world > 1) has already pushed every
// rank's partial output tiles over NVLink into the receive buffer of the rank that owns those
// rows, tile by tile while the GEMM was still computing.  This kernel
//   A. tells every peer "my partials are in your buffer" and waits for the same from all peers,
//   B. sums the `world` partials of the rows this rank owns (fp32), adds the bias once,
//      rounds to bf16 and stores the result into the output buffer of EVERY rank (plain
//      16-byte peer stores; no TMA multicast, no multimem),
//   C. tells every peer "your output rows from me are written" and waits for the same, so that
//      when the kernel retires the local output is complete.
// A runs as its own single-warp launch in front of the reduction (see exchange_flags_kernel).
// Flags are 32-bit epoch numbers in each rank's flag words (2 * world + 1 words, zeroed once):
// word s of rank r = "rank s finished phase A", word world + s = "... phase C", last word =
// block ticket.  Every wait is bounded (b200q_cfg::peer_wait_ms, default 2 s); a wait that gives up
// records it in the device status word and the kernel returns without touching the output again.
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"

namespace b200q {
namespace gemm {
int* device_status_word();
}

namespace {

constexpr int kThreads = 256;

struct Peers {
  int rank, world;
  const __nv_bfloat16* recv;      // this rank's receive buffer [world][rows_per][N]
  __nv_bfloat16* out[8];          // every rank's output [M][N]
  uint32_t* flags[8];             // every rank's flag words
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// true when *p has reached `epoch` within `limit_ns`
__device__ __forceinline__ bool wait_epoch(const uint32_t* p, uint32_t epoch, uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t i = 0;; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - epoch) >= 0) return true;
    if ((i & 0x3fu) == 0x3fu) {
      const uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
}

// Phase A on its own: one warp tells every peer "my partials are in your buffer" and waits for the
// same from all peers.  It is a separate single-warp launch so that a rank that is still waiting
// never keeps SM resources away from the GEMMs of another stream that its peers are waiting for.
struct FlagPeers {
  int rank, world;
  uint32_t* flags[8];
};

__global__ void __launch_bounds__(32) exchange_flags_kernel(const FlagPeers fp, uint32_t epoch, uint64_t limit_ns, int* status) {
  if (threadIdx.x < fp.world) {
    __threadfence_system();
    st_release_sys(fp.flags[threadIdx.x] + fp.rank, epoch);
    if (!wait_epoch(fp.flags[fp.rank] + threadIdx.x, epoch, limit_ns)) atomicCAS(status, 0, 21);
  }
}

__global__ void __launch_bounds__(kThreads)
reduce_gather_kernel(const Peers pr, const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ residual,
                     int64_t rows_per, int64_t N, uint32_t epoch, uint64_t limit_ns, int* status) {
  __shared__ int s_last;
  const int W = pr.world;
  uint32_t* my_flags = pr.flags[pr.rank];

  // phase A ran as exchange_flags_kernel; a wait that gave up there (or earlier) skips the work
  const bool ok = *reinterpret_cast<volatile int*>(status) == 0;

  // ---- B: reduce my rows, store to every rank
  if (ok) {
    const int64_t groups = (rows_per * N) >> 3;
    const int64_t slot = rows_per * N;                    // elements per source slot
    const int64_t out_base = static_cast<int64_t>(pr.rank) * rows_per * N;
    for (int64_t g = blockIdx.x * (int64_t)kThreads + threadIdx.x; g < groups; g += (int64_t)gridDim.x * kThreads) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
      for (int s = 0; s < W; ++s) {
        // written by a peer during this launch sequence: read through L2, never a stale L1 line
        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(pr.recv + s * slot + g * 8));
        float v[8];
        Elem<__nv_bfloat16>::unpack(raw, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[j];
      }
      if (bias != nullptr) {
        const int64_t col = (g * 8) % N;
        float b[8];
        Elem<__nv_bfloat16>::load8(bias + col, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += b[j];
      }
      if (residual != nullptr) {
        // residual stream rows owned by this rank: out = bf16(h + bf16(sum + bias)), the same
        // two roundings as a separate add after the reduction
        float hres[8];
        Elem<__nv_bfloat16>::load8(residual + g * 8, hres);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = hres[j] + __bfloat162float(__float2bfloat16_rn(acc[j]));
      }
      uint4 w;
      uint32_t* u = &w.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        u[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      for (int r = 0; r < W; ++r) *reinterpret_cast<uint4*>(pr.out[r] + out_base + g * 8) = w;
    }
  }

  // ---- C: outputs exchanged; the last block to finish signals and waits
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(my_flags + 2 * W, 1u);
    s_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) my_flags[2 * W] = 0u;  // re-arm the ticket
    // Every CTA read the status word on its own; one that came late may have skipped its rows
    // after an earlier CTA had seen 0.  The word is never cleared on the device, so reading it
    // again here tells whether ALL CTAs did their work: only then are the peers told so.
    if (ok && *reinterpret_cast<volatile int*>(status) == 0) {
      if (threadIdx.x < W) {
        __threadfence_system();
        st_release_sys(pr.flags[threadIdx.x] + W + pr.rank, epoch);
        if (!wait_epoch(my_flags + W + threadIdx.x, epoch, limit_ns)) atomicCAS(status, 0, 22);
      }
    }
  }
}

// Token-sharded residual stream: the owner of a block of tokens reduces the partials, adds the
// bias and the residual it keeps, applies RMSNorm, quantizes per token to FP8 E4M3 and stores
// codes + scales into the gathered activation buffers of EVERY rank (8-byte peer stores), so
// only 1 byte per element crosses NVLink on the way out and the bf16 residual never does.
struct GatherPeers {
  int rank, world;
  const __nv_bfloat16* recv;      // this rank's receive buffer [world][rows_per][N]
  uint8_t* codes[8];              // every rank's gathered FP8 codes [M][N]
  float* scales[8];               // every rank's gathered per-token scales [M]
  uint32_t* flags[8];
};

template <int ITEMS>
__global__ void __launch_bounds__(kThreads)
reduce_norm_quant_gather_kernel(const GatherPeers pr, const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ h,
                                const __nv_bfloat16* __restrict__ w, int64_t rows_per, int64_t N, float eps, uint32_t epoch,
                                uint64_t limit_ns, int* status) {
  __shared__ int s_last;
  __shared__ float red[kThreads / 32];
  const int W = pr.world;
  uint32_t* my_flags = pr.flags[pr.rank];

  const bool ok = *reinterpret_cast<volatile int*>(status) == 0;

  // ---- B: one token per block iteration
  if (ok) {
    const int groups = static_cast<int>(N >> 3);
    const int64_t slot = rows_per * N;
    for (int64_t row = blockIdx.x; row < rows_per; row += gridDim.x) {
      float v[ITEMS][8];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = threadIdx.x + i * kThreads;
        if (g < groups) {
          const int64_t off = row * N + static_cast<int64_t>(g) * 8;
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
          for (int s = 0; s < W; ++s) {
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(pr.recv + s * slot + off));
            float p[8];
            Elem<__nv_bfloat16>::unpack(raw, p);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += p[j];
          }
          if (bias != nullptr) {
            float b[8];
            Elem<__nv_bfloat16>::load8(bias + static_cast<int64_t>(g) * 8, b);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += b[j];
          }
          Elem<__nv_bfloat16>::load8(h + off, v[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] + __bfloat162float(__float2bfloat16_rn(acc[j]))));
            ss = fmaf(v[i][j], v[i][j], ss);
          }
          Elem<__nv_bfloat16>::store8(h + off, v[i]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
        }
      }
      const float inv = rsqrtf(block_sum<kThreads>(ss, red) / static_cast<float>(N) + eps);
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = threadIdx.x + i * kThreads;
        if (g < groups) {
          float wv[8];
          Elem<__nv_bfloat16>::load8(w + static_cast<int64_t>(g) * 8, wv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] * inv * wv[j]));
            amax = fmaxf(amax, fabsf(v[i][j]));
          }
        }
      }
      __syncthreads();  // every thread has left block_sum's scratch
      amax = warp_max(amax);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
      __syncthreads();
      amax = (threadIdx.x & 31) < kThreads / 32 ? red[threadIdx.x & 31] : 0.0f;
      amax = warp_max(amax);
      __syncthreads();  // scratch free for the next token
      const float scale = fp8_scale_from_amax(amax);
      const int64_t grow = static_cast<int64_t>(pr.rank) * rows_per + row;
      if (threadIdx.x < W) pr.scales[threadIdx.x][grow] = scale;
      const float y = b200q_rcp_rn(scale);
      const bool fast = b200q_div_fast_ok(scale);
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = threadIdx.x + i * kThreads;
        if (g < groups) {
          float q[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) q[j] = fast ? b200q_div_by_shared(v[i][j], scale, y) : __fdiv_rn(v[i][j], scale);
          const uint32_t lo = f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16);
          const uint32_t hi = f32x2_to_e4m3x2(q[4], q[5]) | (f32x2_to_e4m3x2(q[6], q[7]) << 16);
          const uint2 packed = make_uint2(lo, hi);
          for (int r = 0; r < W; ++r) *reinterpret_cast<uint2*>(pr.codes[r] + grow * N + static_cast<int64_t>(g) * 8) = packed;
        }
      }
    }
  }

  // ---- C: gathered activations exchanged; the last block to finish signals and waits
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(my_flags + 2 * W, 1u);
    s_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) my_flags[2 * W] = 0u;  // re-arm the ticket
    // Every CTA read the status word on its own; one that came late may have skipped its rows
    // after an earlier CTA had seen 0.  The word is never cleared on the device, so reading it
    // again here tells whether ALL CTAs did their work: only then are the peers told so.
    if (ok && *reinterpret_cast<volatile int*>(status) == 0) {
      if (threadIdx.x < W) {
        __threadfence_system();
        st_release_sys(pr.flags[threadIdx.x] + W + pr.rank, epoch);
        if (!wait_epoch(my_flags + W + threadIdx.x, epoch, limit_ns)) atomicCAS(status, 0, 24);
      }
    }
  }
}


// The same kernel for whole micro-batches of a prefill: persistent CTAs, and every row it reads (the
// `world` partials of a token, then the token's residual) arrives through a ring of shared-memory
// stages filled by bulk asynchronous copies that one thread keeps issuing `stages` rows ahead, across
// tokens.  The one-CTA-per-token form above issues its loads partial by partial and stops loading
// while it reduces and stores; with 2 to 8 partials per token that leaves most of the HBM bandwidth
// unused.  Thread-to-element mapping, summation order and rounding points are unchanged: same bits.
constexpr int kGatherStagesMax = 12;
constexpr int kGatherRingBytes = 96 * 1024;

template <int ITEMS>
__global__ void __launch_bounds__(kThreads, 2)
reduce_norm_quant_gather_stream_kernel(const GatherPeers pr, const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ h,
                                       const __nv_bfloat16* __restrict__ w, int rows_per, int N, float eps, uint32_t epoch,
                                       uint64_t limit_ns, int stages, int* status) {
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ uint64_t full[kGatherStagesMax];
  __shared__ int s_last;
  __shared__ float red[kThreads / 32];
  const int W = pr.world;
  uint32_t* my_flags = pr.flags[pr.rank];
  const bool ok = *reinterpret_cast<volatile int*>(status) == 0;

  if (ok) {
    const int groups = N >> 3;
    const uint32_t row_bytes = static_cast<uint32_t>(N) * 2u;
    const int64_t slot = static_cast<int64_t>(rows_per) * N;
    const int step = static_cast<int>(gridDim.x);
    const int my_rows = (rows_per - static_cast<int>(blockIdx.x) + step - 1) / step;   // rows this CTA walks
    const int per_row = W + 1;                                                         // W partials, then the residual
    const int total = my_rows * per_row;
    if (threadIdx.x == 0) {
      for (int s = 0; s < stages; ++s) ptx::mbar_init(&full[s], 1);
      ptx::fence_barrier_init();
    }
    __syncthreads();
    // copy number q of this CTA: source q % per_row of its row number q / per_row
    auto issue = [&](int q) {
      const int64_t row = static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(q / per_row) * step;
      const int src = q % per_row;
      const __nv_bfloat16* from = src < W ? pr.recv + src * slot + row * N : h + row * N;
      const int s = q % stages;
      ptx::mbar_arrive_expect_tx(&full[s], row_bytes);
      ptx::bulk_load(ring + static_cast<size_t>(s) * row_bytes, from, row_bytes, &full[s]);
    };
    if (threadIdx.x == 0)
      for (int q = 0; q < stages && q < total; ++q) issue(q);
    // norm weights and bias of this thread's groups: the same for every token
    uint4 wp[ITEMS], bp[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kThreads;
      wp[i] = g < groups ? ld_nc_128(w + static_cast<int64_t>(g) * 8) : make_uint4(0u, 0u, 0u, 0u);
      bp[i] = (g < groups && bias != nullptr) ? ld_nc_128(bias + static_cast<int64_t>(g) * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
    bool arrived = true;   // after one wait gave up the rest are not waited for: the status word says the result is void
    int q = 0;
    // one stage consumed: wait for it, hand the 16 bytes of every group of this thread to `use`, and once
    // the whole CTA has read it let thread 0 refill it with the copy `stages` places ahead
    auto consume = [&](auto&& use) {
      const int s = q % stages;
      if (arrived && !ptx::mbar_wait(&full[s], static_cast<uint32_t>(q / stages) & 1u)) {
        arrived = false;
        atomicCAS(status, 0, 25);
      }
      const unsigned char* st = ring + static_cast<size_t>(s) * row_bytes;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = threadIdx.x + i * kThreads;
        if (g < groups) use(i, *reinterpret_cast<const uint4*>(st + static_cast<size_t>(g) * 16));
      }
      __syncthreads();
      if (threadIdx.x == 0 && q + stages < total) issue(q + stages);
      ++q;
    };
    for (int64_t row = blockIdx.x; row < rows_per; row += step) {
      float v[ITEMS][8];
#pragma unroll
      for (int i = 0; i < ITEMS; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
      for (int src = 0; src < W; ++src) {
        consume([&](int i, const uint4& raw) {
          float pv[8];
          Elem<__nv_bfloat16>::unpack(raw, pv);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += pv[j];
        });
      }
      float ss = 0.0f;
      consume([&](int i, const uint4& raw) {
        float hv[8];
        Elem<__nv_bfloat16>::unpack(raw, hv);
        if (bias != nullptr) {
          float b[8];
          Elem<__nv_bfloat16>::unpack(bp[i], b);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += b[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[i][j] = __bfloat162float(__float2bfloat16_rn(hv[j] + __bfloat162float(__float2bfloat16_rn(v[i][j]))));
          ss = fmaf(v[i][j], v[i][j], ss);
        }
        Elem<__nv_bfloat16>::store8(h + row * N + static_cast<int64_t>(threadIdx.x + i * kThreads) * 8, v[i]);
      });
      const float inv = rsqrtf(block_sum<kThreads>(ss, red) / static_cast<float>(N) + eps);
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const int g = threadIdx.x + i * kThreads;
        if (g < groups) {
          float wv[8];
          Elem<__nv_bfloat16>::unpack(wp[i], wv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] * inv * wv[j]));
            amax = fmaxf(amax, fabsf(v[i][j]));
          }
        }
      }
      amax = warp_max(amax);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
      __syncthreads();
      amax = (threadIdx.x & 31) < kThreads / 32 ? red[threadIdx.x & 31] : 0.0f;
      amax = warp_max(amax);
      __syncthreads();  // scratch free for the next token
      const float scale = fp8_scale_from_amax(amax);
      const int64_t grow = static_cast<int64_t>(pr.rank) * rows_per + row;
      if (threadIdx.x < W) pr.scales[threadIdx.x][grow] = scale;
      const float y = b200q_rcp_rn(scale);
      auto emit = [&](auto fast_tag) {
        constexpr bool kFast = decltype(fast_tag)::value;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
          const int g = threadIdx.x + i * kThreads;
          if (g < groups) {
            float qv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) qv[j] = kFast ? b200q_div_by_shared(v[i][j], scale, y) : __fdiv_rn(v[i][j], scale);
            const uint32_t lo = f32x2_to_e4m3x2(qv[0], qv[1]) | (f32x2_to_e4m3x2(qv[2], qv[3]) << 16);
            const uint32_t hi = f32x2_to_e4m3x2(qv[4], qv[5]) | (f32x2_to_e4m3x2(qv[6], qv[7]) << 16);
            const uint2 packed = make_uint2(lo, hi);
            for (int r = 0; r < W; ++r) *reinterpret_cast<uint2*>(pr.codes[r] + grow * N + static_cast<int64_t>(g) * 8) = packed;
          }
        }
      };
      if (b200q_div_fast_ok(scale)) emit(std::true_type{});   // one branch per token, not one select per element
      else emit(std::false_type{});
    }
  }

  // ---- gathered activations exchanged; the last block to finish signals and waits (as above)
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(my_flags + 2 * W, 1u);
    s_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) my_flags[2 * W] = 0u;  // re-arm the ticket
    if (ok && *reinterpret_cast<volatile int*>(status) == 0) {
      if (threadIdx.x < W) {
        __threadfence_system();
        st_release_sys(pr.flags[threadIdx.x] + W + pr.rank, epoch);
        if (!wait_epoch(my_flags + W + threadIdx.x, epoch, limit_ns)) atomicCAS(status, 0, 24);
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Decode-sized all-reduce by pulling (a few tokens, M <= 128): the row-parallel GEMM leaves this
// rank's partial [M, N] in its own symmetric buffer, a one-warp kernel tells every peer "my partial
// number c is complete", and the reduction kernel of EVERY rank then reads all `world` partials
// (its own and the peers', plain loads over NVLink), sums them in rank order, adds bias and residual,
// applies RMSNorm and quantizes: the whole replicated activation of the next column-parallel GEMM,
// with no second exchange and no library call.  All ranks compute the same sums in the same order,
// so their results are the same bits.
//
// Flag words of a rank for this protocol: word s (s < world) = number of the last partial rank s has
// completed; word `world` = this rank's own count (read and advanced on the device, so a CUDA graph
// that contains these launches can be replayed).  Two partial buffers are used alternately by
// consecutive all-reduces: a rank overwrites a buffer only after it has waited, in the all-reduce in
// between, for a signal that every peer sends after it finished reading that buffer.
struct PullPeers {
  int rank, world;
  const __nv_bfloat16* partial[8];   // every rank's partial [M, N] of this all-reduce (the buffer of this call)
  uint32_t* flags[8];
};

__global__ void __launch_bounds__(32) pull_signal_kernel(const FlagPeers fp) {
  uint32_t* mine = fp.flags[fp.rank];
  const uint32_t c = *reinterpret_cast<volatile uint32_t*>(mine + fp.world) + 1u;
  __syncwarp();
  if (threadIdx.x < fp.world) {
    __threadfence_system();
    st_release_sys(fp.flags[threadIdx.x] + fp.rank, c);
  }
  __syncwarp();
  if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(mine + fp.world) = c;
}

__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 r;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
  return r;
}

// One CTA per token.  QUANT: h += sum, RMSNorm, per-token FP8 codes and scales (local).  !QUANT: h += sum only.
template <int ITEMS, bool QUANT>
__global__ void __launch_bounds__(kThreads)
pull_reduce_kernel(const PullPeers pr, const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ codes, float* __restrict__ scales, int64_t N, float eps,
                   uint64_t limit_ns, int* status) {
  __shared__ float red[kThreads / 32];
  const int W = pr.world;
  // every peer's partial of this all-reduce is complete (bounded wait on this rank's own flag words)
  if (threadIdx.x < W) {
    const uint32_t* mine = pr.flags[pr.rank];
    const uint32_t c = *reinterpret_cast<const volatile uint32_t*>(mine + W);
    if (!wait_epoch(mine + threadIdx.x, c, limit_ns)) atomicCAS(status, 0, 25);
  }
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(status) != 0) return;

  const int groups = static_cast<int>(N >> 3);
  const int64_t row = blockIdx.x;
  float v[ITEMS][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int g = threadIdx.x + i * kThreads;
    if (g < groups) {
      const int64_t off = row * N + static_cast<int64_t>(g) * 8;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
      for (int s = 0; s < W; ++s) {
        const uint4 raw = ld_relaxed_sys_v4(pr.partial[s] + off);   // peer memory: never from a stale cache line
        float q[8];
        Elem<__nv_bfloat16>::unpack(raw, q);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += q[j];
      }
      if (bias != nullptr) {
        float b[8];
        Elem<__nv_bfloat16>::load8(bias + static_cast<int64_t>(g) * 8, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += b[j];
      }
      float hv[8];
      Elem<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(h + off), hv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[i][j] = __bfloat162float(__float2bfloat16_rn(hv[j] + __bfloat162float(__float2bfloat16_rn(acc[j]))));
        ss = fmaf(v[i][j], v[i][j], ss);
      }
      Elem<__nv_bfloat16>::store8(h + off, v[i]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
    }
  }
  if constexpr (QUANT) {
    const float inv = rsqrtf(block_sum<kThreads>(ss, red) / static_cast<float>(N) + eps);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kThreads;
      if (g < groups) {
        float wv[8];
        Elem<__nv_bfloat16>::load8(w + static_cast<int64_t>(g) * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] * inv * wv[j]));
          amax = fmaxf(amax, fabsf(v[i][j]));
        }
      }
    }
    __syncthreads();  // every thread has left block_sum's scratch
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = (threadIdx.x & 31) < kThreads / 32 ? red[threadIdx.x & 31] : 0.0f;
    amax = warp_max(amax);
    const float scale = fp8_scale_from_amax(amax);
    if (threadIdx.x == 0) scales[row] = scale;
    const float y = b200q_rcp_rn(scale);
    const bool fast = b200q_div_fast_ok(scale);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int g = threadIdx.x + i * kThreads;
      if (g < groups) {
        float q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) q[j] = fast ? b200q_div_by_shared(v[i][j], scale, y) : __fdiv_rn(v[i][j], scale);
        const uint32_t lo = f32x2_to_e4m3x2(q[0], q[1]) | (f32x2_to_e4m3x2(q[2], q[3]) << 16);
        const uint32_t hi = f32x2_to_e4m3x2(q[4], q[5]) | (f32x2_to_e4m3x2(q[6], q[7]) << 16);
        *reinterpret_cast<uint2*>(codes + row * N + static_cast<int64_t>(g) * 8) = make_uint2(lo, hi);
      }
    }
  }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

// b200q_cfg::peer_wait_ms -> nanoseconds (0 / no cfg: the library default)
static uint64_t peer_wait_ns(const b200q_cfg* cfg) {
  if (cfg == nullptr || cfg->peer_wait_ms == 0) return ptx::kWaitLimitNs;
  return static_cast<uint64_t>(cfg->peer_wait_ms) * 1000000ull;
}

static int reduce_gather_impl(const b200q_peers* peers, const void* bias, const void* residual, int64_t M, int64_t N, uint32_t epoch,
                              b200q_stream_t stream, const b200q_cfg* cfg) {
  if (peers == nullptr || M <= 0 || N <= 0 || N % 8 != 0) return B200Q_ERR_INVALID;
  if (cfg != nullptr && cfg->reserved != 0) return B200Q_ERR_INVALID;
  const uint64_t limit_ns = peer_wait_ns(cfg);
  const int W = peers->world;
  if (W < 1 || W > 8 || peers->rank < 0 || peers->rank >= W || M % (static_cast<int64_t>(W) * 128) != 0) return B200Q_ERR_INVALID;
  Peers pr{};
  pr.rank = peers->rank;
  pr.world = W;
  pr.recv = static_cast<const __nv_bfloat16*>(peers->recv[peers->rank]);
  for (int r = 0; r < W; ++r) {
    if (peers->recv[r] == nullptr || peers->out[r] == nullptr || peers->flags[r] == nullptr) return B200Q_ERR_INVALID;
    if (!aligned(peers->recv[r], 16) || !aligned(peers->out[r], 16)) return B200Q_ERR_ALIGN;
    pr.out[r] = static_cast<__nv_bfloat16*>(peers->out[r]);
    pr.flags[r] = peers->flags[r];
  }
  if (residual != nullptr && !aligned(residual, 16)) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  int* status = gemm::device_status_word();
  if (status == nullptr) return B200Q_ERR_CUDA;
  const int64_t rows_per = M / W;
  const int64_t groups = (rows_per * N) >> 3;
  int64_t blocks = (groups + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  FlagPeers fp{};
  fp.rank = pr.rank;
  fp.world = W;
  for (int r = 0; r < W; ++r) fp.flags[r] = pr.flags[r];
  exchange_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(fp, epoch, limit_ns, status);
  reduce_gather_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      pr, static_cast<const __nv_bfloat16*>(bias), static_cast<const __nv_bfloat16*>(residual), rows_per, N, epoch, limit_ns, status);
  return check_launch();
}

int b200q_reduce_gather(const b200q_peers* peers, const void* bias, int64_t M, int64_t N, uint32_t epoch, b200q_stream_t stream,
                        const b200q_cfg* cfg) {
  return reduce_gather_impl(peers, bias, nullptr, M, N, epoch, stream, cfg);
}

int b200q_reduce_add_gather(const b200q_peers* peers, const void* bias, const void* residual_shard, int64_t M, int64_t N,
                            uint32_t epoch, b200q_stream_t stream, const b200q_cfg* cfg) {
  if (residual_shard == nullptr) return B200Q_ERR_INVALID;
  return reduce_gather_impl(peers, bias, residual_shard, M, N, epoch, stream, cfg);
}

int b200q_reduce_add_rms_norm_fp8_quantize_gather(const b200q_gather_peers* peers, const void* bias, void* h_shard,
                                                  const void* norm_weight, float eps, int64_t M, int64_t N, uint32_t epoch,
                                                  b200q_stream_t stream, const b200q_cfg* cfg) {
  if (peers == nullptr || h_shard == nullptr || norm_weight == nullptr || M <= 0 || N <= 0 || N % 16 != 0 || N > 16384)
    return B200Q_ERR_INVALID;
  if (cfg != nullptr && cfg->reserved != 0) return B200Q_ERR_INVALID;
  const uint64_t limit_ns = peer_wait_ns(cfg);
  const int W = peers->world;
  if (W < 1 || W > 8 || peers->rank < 0 || peers->rank >= W || M % (static_cast<int64_t>(W) * 128) != 0) return B200Q_ERR_INVALID;
  GatherPeers pr{};
  pr.rank = peers->rank;
  pr.world = W;
  pr.recv = static_cast<const __nv_bfloat16*>(peers->recv[peers->rank]);
  for (int r = 0; r < W; ++r) {
    if (peers->recv[r] == nullptr || peers->codes[r] == nullptr || peers->scales[r] == nullptr || peers->flags[r] == nullptr)
      return B200Q_ERR_INVALID;
    if (!aligned(peers->recv[r], 16) || !aligned(peers->codes[r], 16) || !aligned(peers->scales[r], 4)) return B200Q_ERR_ALIGN;
    pr.codes[r] = peers->codes[r];
    pr.scales[r] = peers->scales[r];
    pr.flags[r] = peers->flags[r];
  }
  if (!aligned(h_shard, 16) || !aligned(norm_weight, 16) || (bias != nullptr && !aligned(bias, 16))) return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  int* status = gemm::device_status_word();
  if (status == nullptr) return B200Q_ERR_CUDA;
  const int64_t rows_per = M / W;
  int64_t blocks = rows_per;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  const int items = static_cast<int>(((N >> 3) + kThreads - 1) / kThreads);
  const unsigned grid = static_cast<unsigned>(blocks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(bias);
  __nv_bfloat16* hp = static_cast<__nv_bfloat16*>(h_shard);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(norm_weight);
  FlagPeers fp{};
  fp.rank = pr.rank;
  fp.world = W;
  for (int r = 0; r < W; ++r) fp.flags[r] = pr.flags[r];
  exchange_flags_kernel<<<1, 32, 0, st>>>(fp, epoch, limit_ns, status);
  // whole micro-batches: persistent CTAs fed through a shared-memory ring, an equal number of tokens each
  if (items <= 4 && rows_per >= 64 && kGatherRingBytes / (N * 2) >= 3) {
    int stages = static_cast<int>(kGatherRingBytes / (N * 2));
    if (stages > kGatherStagesMax) stages = kGatherStagesMax;
    const int64_t slots = static_cast<int64_t>(sm_count()) * 2;
    const int64_t rows_per_cta = (rows_per + slots - 1) / slots;
    const unsigned sgrid = static_cast<unsigned>((rows_per + rows_per_cta - 1) / rows_per_cta);
    const size_t smem = static_cast<size_t>(stages) * static_cast<size_t>(N) * 2;
    const int r32 = static_cast<int>(rows_per), n32 = static_cast<int>(N);
#define B200Q_RNQG(I)                                                                                                          \
  do {                                                                                                                          \
    cudaFuncSetAttribute(reduce_norm_quant_gather_stream_kernel<I>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGatherRingBytes); \
    reduce_norm_quant_gather_stream_kernel<I><<<sgrid, kThreads, smem, st>>>(pr, bp, hp, wp, r32, n32, eps, epoch, limit_ns, stages, status); \
  } while (0)
    if (items <= 1) B200Q_RNQG(1);
    else if (items <= 2) B200Q_RNQG(2);
    else B200Q_RNQG(4);
#undef B200Q_RNQG
    return check_launch();
  }
  if (items <= 1) reduce_norm_quant_gather_kernel<1><<<grid, kThreads, 0, st>>>(pr, bp, hp, wp, rows_per, N, eps, epoch, limit_ns, status);
  else if (items <= 2) reduce_norm_quant_gather_kernel<2><<<grid, kThreads, 0, st>>>(pr, bp, hp, wp, rows_per, N, eps, epoch, limit_ns, status);
  else if (items <= 4) reduce_norm_quant_gather_kernel<4><<<grid, kThreads, 0, st>>>(pr, bp, hp, wp, rows_per, N, eps, epoch, limit_ns, status);
  else reduce_norm_quant_gather_kernel<8><<<grid, kThreads, 0, st>>>(pr, bp, hp, wp, rows_per, N, eps, epoch, limit_ns, status);
  return check_launch();
}

static int fill_pull(PullPeers& pr, FlagPeers& fp, const b200q_pull_peers* peers) {
  if (peers == nullptr) return B200Q_ERR_INVALID;
  const int W = peers->world;
  if (W < 1 || W > 8 || peers->rank < 0 || peers->rank >= W) return B200Q_ERR_INVALID;
  pr.rank = fp.rank = peers->rank;
  pr.world = fp.world = W;
  for (int r = 0; r < W; ++r) {
    if (peers->partial[r] == nullptr || peers->flags[r] == nullptr) return B200Q_ERR_INVALID;
    if (!aligned(peers->partial[r], 16)) return B200Q_ERR_ALIGN;
    pr.partial[r] = static_cast<const __nv_bfloat16*>(peers->partial[r]);
    pr.flags[r] = fp.flags[r] = peers->flags[r];
  }
  return B200Q_OK;
}

int b200q_pull_signal(const b200q_pull_peers* peers, b200q_stream_t stream) {
  PullPeers pr{};
  FlagPeers fp{};
  if (int rc = fill_pull(pr, fp, peers)) return rc;
  if (int rc = check_arch()) return rc;
  pull_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(fp);
  return check_launch();
}

static int pull_reduce_impl(const b200q_pull_peers* peers, const void* bias, void* h, const void* norm_weight, float eps,
                            uint8_t* codes_out, float* scales_out, int64_t M, int64_t N, bool quant, b200q_stream_t stream,
                            const b200q_cfg* cfg) {
  if (h == nullptr || M <= 0 || M > 1024 || N <= 0 || N % 16 != 0 || N > 16384) return B200Q_ERR_INVALID;
  if (quant && (norm_weight == nullptr || codes_out == nullptr || scales_out == nullptr)) return B200Q_ERR_INVALID;
  if (cfg != nullptr && cfg->reserved != 0) return B200Q_ERR_INVALID;
  PullPeers pr{};
  FlagPeers fp{};
  if (int rc = fill_pull(pr, fp, peers)) return rc;
  if (!aligned(h, 16) || (bias != nullptr && !aligned(bias, 16)) || (quant && (!aligned(norm_weight, 16) || !aligned(codes_out, 8))))
    return B200Q_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  int* status = gemm::device_status_word();
  if (status == nullptr) return B200Q_ERR_CUDA;
  const uint64_t limit_ns = peer_wait_ns(cfg);
  const int items = static_cast<int>(((N >> 3) + kThreads - 1) / kThreads);
  const unsigned grid = static_cast<unsigned>(M);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(bias);
  __nv_bfloat16* hp = static_cast<__nv_bfloat16*>(h);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(norm_weight);
#define B200Q_PULL(I)                                                                                                        \
  do {                                                                                                                         \
    if (quant) pull_reduce_kernel<I, true><<<grid, kThreads, 0, st>>>(pr, bp, hp, wp, codes_out, scales_out, N, eps, limit_ns, status); \
    else pull_reduce_kernel<I, false><<<grid, kThreads, 0, st>>>(pr, bp, hp, wp, codes_out, scales_out, N, eps, limit_ns, status);      \
  } while (0)
  if (items <= 1) B200Q_PULL(1);
  else if (items <= 2) B200Q_PULL(2);
  else if (items <= 4) B200Q_PULL(4);
  else B200Q_PULL(8);
#undef B200Q_PULL
  return check_launch();
}

int b200q_pull_reduce_add_rms_norm_fp8_quantize(const b200q_pull_peers* peers, const void* bias, void* h, const void* norm_weight,
                                                float eps, uint8_t* codes_out, float* scales_out, int64_t M, int64_t N,
                                                b200q_stream_t stream, const b200q_cfg* cfg) {
  return pull_reduce_impl(peers, bias, h, norm_weight, eps, codes_out, scales_out, M, N, true, stream, cfg);
}

int b200q_pull_reduce_add(const b200q_pull_peers* peers, const void* bias, void* h, int64_t M, int64_t N, b200q_stream_t stream,
                          const b200q_cfg* cfg) {
  return pull_reduce_impl(peers, bias, h, nullptr, 0.0f, nullptr, nullptr, M, N, false, stream, cfg);
}

}  // extern "C"
