"""b200q_amax_static: the abs-max entry point for hosts that cannot allocate.

A TensorRT plugin's enqueue(), code running under CUDA-graph stream capture, or a server
that gave all device memory to its own pool cannot hand this library a freshly allocated
workspace.  For them the library carries its own small scratch array, and this entry point
uses it instead of a caller workspace.  The test calls it through the C ABI, twice in a row
(the scratch keeps the previous call's contents, so the second call proves it re-arms
itself), and requires bit-identical results to b200q_amax, which takes a caller workspace.
Abs-max does not depend on the order of reduction, so the comparison is exact.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _amax_workspace(lib, x):
    ws = torch.zeros(lib.b200q_amax_workspace_bytes(), dtype=torch.uint8, device=x.device)
    out = torch.full((1,), -1.0, dtype=torch.float32, device=x.device)
    rc = lib.b200q_amax(x.data_ptr(), DT[x.dtype], x.numel(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return out


def _amax_static(lib, x, out):
    return lib.b200q_amax_static(x.data_ptr(), DT[x.dtype], x.numel(), out.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_static_amax_matches_workspace_amax_on_two_calls_in_a_row(b200, dtype):
    lib = b200.load_library()
    g = torch.Generator().manual_seed(11)
    a = (torch.randn(3_000_000 + 5, generator=g) * 3).to(dtype).cuda()   # ragged tail, 12 CTAs
    b = (torch.randn(1000, generator=g) * 100).to(dtype).cuda()          # one CTA, larger maximum
    c = (torch.randn(2 ** 20, generator=g) * 0.01).to(dtype).cuda()      # smaller maximum than the call before
    out = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
    for x in (a, b, c, a):                                               # back-to-back calls share the scratch
        expect = _amax_workspace(lib, x)
        assert _amax_static(lib, x, out) == 0
        torch.cuda.synchronize()
        assert out.item() == expect.item() == x.float().abs().max().item()


def test_static_amax_rejects_sizes_beyond_its_scratch(b200):
    lib = b200.load_library()
    limit = lib.b200q_amax_static_max_elements()
    assert limit == 2 ** 28
    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(1, dtype=torch.float32, device="cuda")
    rc = lib.b200q_amax_static(x.data_ptr(), 2, limit + 1, out.data_ptr(), None)   # rejected before any launch
    assert rc == -7
    assert b"scratch" in lib.b200q_status_string(rc)
    assert lib.b200q_amax_static(x.data_ptr(), 9, 64, out.data_ptr(), None) == -1
    # at the limit itself the call is accepted
    big = torch.ones(limit, dtype=torch.float16, device="cuda")
    big[-3] = -7.0
    assert lib.b200q_amax_static(big.data_ptr(), 1, limit, out.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert out.item() == 7.0
