"""The library's own communication context (b200q_comm_*): CUDA-IPC peer mappings exchanged through
a host all-gather.  Two processes share GPU 0 and talk through a gloo group; they only copy through
the peer pointers between host barriers, so no kernel of one process ever waits on the other."""
import os
import sys
import tempfile

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, store_path):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from tensorrt_b200.tp import CommContext, _device_view

    torch.cuda.set_device(0)
    dist.init_process_group("gloo", store=dist.FileStore(store_path, world), rank=rank, world_size=world)
    comm = CommContext()
    nbytes = 1 << 20
    addrs, local = comm.alloc(nbytes)
    addrs2, local2 = comm.alloc(4096)
    assert len(addrs) == world and all(a for a in addrs) and addrs[rank] == local.data_ptr()
    assert int(local.sum()) == 0 and int(local2.sum()) == 0          # handed out zeroed
    local.fill_(rank + 1)
    local2.fill_(10 + rank)
    torch.cuda.synchronize()
    dist.barrier()
    for r in range(world):
        peer = _device_view(addrs[r], nbytes)
        assert bool((peer == r + 1).all()), (rank, r)
        peer2 = _device_view(addrs2[r], 4096)
        assert bool((peer2 == 10 + r).all()), (rank, r)
    torch.cuda.synchronize()
    dist.barrier()
    # a store into the neighbour's buffer is seen by its owner
    nxt = (rank + 1) % world
    _device_view(addrs[nxt], nbytes)[:256].fill_(100 + rank)
    torch.cuda.synchronize()
    dist.barrier()
    assert bool((local[:256] == 100 + (rank - 1) % world).all())
    assert bool((local[256:] == rank + 1).all())
    dist.barrier()
    comm.close()
    comm.close()                                                     # idempotent
    dist.destroy_process_group()


@pytest.mark.gpu
def test_comm_context_two_processes_one_gpu(b200):
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, os.path.join(d, "store")), nprocs=2, join=True)


@pytest.mark.gpu
def test_comm_context_single_rank(b200):
    import ctypes

    from tensorrt_b200 import _lib

    lib = _lib.load()
    h = ctypes.c_void_p()
    assert lib.b200q_comm_create(0, 1, _lib.ALLGATHER_FN(0), None, ctypes.byref(h)) == 0
    ptrs = (ctypes.c_void_p * 8)()
    assert lib.b200q_comm_alloc(h, 1000, ptrs) == 0
    assert ptrs[0] and not ptrs[1]
    assert lib.b200q_comm_alloc(h, 0, ptrs) == -1  # B200Q_ERR_INVALID
    assert lib.b200q_comm_destroy(h) == 0
