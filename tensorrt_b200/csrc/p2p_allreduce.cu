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
// Flags are 32-bit epoch numbers in each rank's flag words (2 * world + 1 words, zeroed once):
// word s of rank r = "rank s finished phase A", word world + s = "... phase C", last word =
// block ticket.  Every wait is bounded (2 s); a wait that gives up records it in the device
// status word and the kernel returns without touching the output again.
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

// true when *p has reached `epoch` within the time limit
__device__ __forceinline__ bool wait_epoch(const uint32_t* p, uint32_t epoch) {
  uint64_t t0 = 0;
  for (uint32_t i = 0;; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - epoch) >= 0) return true;
    if ((i & 0xffu) == 0xffu) {
      const uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > ptx::kWaitLimitNs) return false;
    }
  }
}

__global__ void __launch_bounds__(kThreads)
reduce_gather_kernel(const Peers pr, const __nv_bfloat16* __restrict__ bias, int64_t rows_per, int64_t N, uint32_t epoch,
                     int* status) {
  __shared__ int s_ok;
  __shared__ int s_last;
  const int W = pr.world;
  uint32_t* my_flags = pr.flags[pr.rank];

  // ---- A: partials exchanged
  if (blockIdx.x == 0 && threadIdx.x < W) {
    __threadfence_system();
    st_release_sys(pr.flags[threadIdx.x] + pr.rank, epoch);
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < W && !wait_epoch(my_flags + threadIdx.x, epoch)) {
    s_ok = 0;
    atomicCAS(status, 0, 21);
  }
  __syncthreads();
  const bool ok = s_ok != 0;

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
    if (ok) {
      if (threadIdx.x < W) {
        __threadfence_system();
        st_release_sys(pr.flags[threadIdx.x] + W + pr.rank, epoch);
        if (!wait_epoch(my_flags + W + threadIdx.x, epoch)) atomicCAS(status, 0, 22);
      }
    }
  }
}

}  // namespace
}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_reduce_gather(const b200q_peers* peers, const void* bias, int64_t M, int64_t N, uint32_t epoch, b200q_stream_t stream) {
  if (peers == nullptr || M <= 0 || N <= 0 || N % 8 != 0) return B200Q_ERR_INVALID;
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
  if (int rc = check_arch()) return rc;
  int* status = gemm::device_status_word();
  if (status == nullptr) return B200Q_ERR_CUDA;
  const int64_t rows_per = M / W;
  const int64_t groups = (rows_per * N) >> 3;
  int64_t blocks = (groups + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 4;
  if (blocks > cap) blocks = cap;
  reduce_gather_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      pr, static_cast<const __nv_bfloat16*>(bias), rows_per, N, epoch, status);
  return check_launch();
}

}  // extern "C"
