// Native communication context: peer mappings of per-rank device buffers for the fused row-parallel
// entry points (b200q_peers, b200q_gather_peers, b200q_pull_peers), without any Python or torch in the way.
//
// The reference's runtime binds a communicator to its engine in C++ (TRTEngine::bind_nccl_comm,
// core/runtime/TRTEngine.cpp:821-928: resolve the process group, take its ncclComm_t, hand it to the
// execution context).  The kernels of this library do not call a collective library; what they need from
// the "communicator" is, for every buffer, a pointer that is valid in THIS process for every rank's copy.
// One process per GPU on one node: CUDA IPC provides that.  The context owns the buffers; the only thing it
// asks from its host is an all-gather of a few bytes between the ranks (the host already has one: MPI, a
// c10d store or process group, sockets), passed in as a callback.
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

struct b200q_comm {
  int rank = 0, world = 1, device = 0;
  b200q_allgather_fn allgather = nullptr;
  void* user = nullptr;
  struct Allocation {
    void* local = nullptr;
    void* peer[8] = {};
  };
  std::vector<Allocation> allocations;
  std::mutex mu;
};

extern "C" {

int b200q_comm_create(int rank, int world, b200q_allgather_fn allgather, void* user, b200q_comm** out) {
  if (out == nullptr || world < 1 || world > 8 || rank < 0 || rank >= world || (world > 1 && allgather == nullptr)) return B200Q_ERR_INVALID;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B200Q_ERR_CUDA;
  b200q_comm* c = new (std::nothrow) b200q_comm();
  if (c == nullptr) return B200Q_ERR_CUDA;
  c->rank = rank;
  c->world = world;
  c->device = dev;
  c->allgather = allgather;
  c->user = user;
  *out = c;
  return B200Q_OK;
}

int b200q_comm_alloc(b200q_comm* comm, size_t bytes, void* ptrs[8]) {
  if (comm == nullptr || ptrs == nullptr || bytes == 0) return B200Q_ERR_INVALID;
  std::lock_guard<std::mutex> lk(comm->mu);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != comm->device) return B200Q_ERR_INVALID;   // the device the context was created on
  // whole 2 MiB pages: an IPC handle names the driver's underlying block, and small allocations would
  // otherwise share one
  constexpr size_t kPage = size_t(2) << 20;
  bytes = (bytes + kPage - 1) / kPage * kPage;
  b200q_comm::Allocation a;
  if (cudaMalloc(&a.local, bytes) != cudaSuccess) {
    cudaGetLastError();
    return B200Q_ERR_CUDA;
  }
  if (cudaMemset(a.local, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaFree(a.local);
    return B200Q_ERR_CUDA;
  }
  for (int r = 0; r < 8; ++r) ptrs[r] = nullptr;
  a.peer[comm->rank] = a.local;
  if (comm->world > 1) {
    cudaIpcMemHandle_t mine;
    if (cudaIpcGetMemHandle(&mine, a.local) != cudaSuccess) {
      cudaFree(a.local);
      return B200Q_ERR_CUDA;
    }
    std::vector<cudaIpcMemHandle_t> all(static_cast<size_t>(comm->world));
    if (comm->allgather(comm->user, &mine, all.data(), sizeof(mine)) != 0) {
      cudaFree(a.local);
      return B200Q_ERR_CUDA;
    }
    for (int r = 0; r < comm->world; ++r) {
      if (r == comm->rank) continue;
      if (cudaIpcOpenMemHandle(&a.peer[r], all[static_cast<size_t>(r)], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        for (int q = 0; q < r; ++q)
          if (q != comm->rank && a.peer[q] != nullptr) cudaIpcCloseMemHandle(a.peer[q]);
        cudaFree(a.local);
        return B200Q_ERR_CUDA;
      }
    }
  }
  for (int r = 0; r < comm->world; ++r) ptrs[r] = a.peer[r];
  comm->allocations.push_back(a);
  return B200Q_OK;
}

int b200q_comm_destroy(b200q_comm* comm) {
  if (comm == nullptr) return B200Q_OK;
  int rc = B200Q_OK;
  {
    std::lock_guard<std::mutex> lk(comm->mu);
    cudaDeviceSynchronize();
    // every rank has stopped using every mapping before any rank frees its buffer
    if (comm->world > 1) {
      char token = 0;
      std::vector<char> all(static_cast<size_t>(comm->world));
      if (comm->allgather(comm->user, &token, all.data(), 1) != 0) rc = B200Q_ERR_CUDA;
    }
    for (auto& a : comm->allocations)
      for (int r = 0; r < comm->world; ++r)
        if (r != comm->rank && a.peer[r] != nullptr) cudaIpcCloseMemHandle(a.peer[r]);
    if (comm->world > 1) {
      char token = 0;
      std::vector<char> all(static_cast<size_t>(comm->world));
      if (comm->allgather(comm->user, &token, all.data(), 1) != 0) rc = B200Q_ERR_CUDA;
    }
    for (auto& a : comm->allocations) cudaFree(a.local);
    comm->allocations.clear();
  }
  delete comm;
  return rc;
}

}  // extern "C"
