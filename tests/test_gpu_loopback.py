"""The fused row-parallel kernels (GEMM with the reduce-scatter epilogue, peer-memory reduce +
gather, reduce + residual + RMSNorm + FP8 quantize + gather) on ONE GPU, through the C ABI.

`world` virtual ranks live on the same device: each has its own receive / output / gathered
buffers and flag words, and every rank's `b200q_peers` points at all of them, exactly as the
peer mappings of `world` GPUs would.  The launches of all ranks go to ONE stream, phase by phase
(all GEMMs, then all reductions), and before the reductions the host writes the epoch into every
flag word, standing in for "every peer has signalled".  So no kernel ever waits for a kernel that
has not run yet: launches that spin on one another must not share a GPU.  What this covers is the
data path (which tile lands in which slot of which rank, the sum, bias, residual, norm, quantize,
the stores into every rank's buffers) and the signalling side of the flag protocol; the waiting
side is covered by the test at the end, where a wait that nothing satisfies runs out and reports
through the device status word.
"""
import ctypes

import pytest
import torch

import oracle as o

pytestmark = pytest.mark.gpu


class Ranks:
    """Buffers and b200q_peers / b200q_gather_peers of `world` virtual ranks on the current device."""

    def __init__(self, world, M, N):
        from tensorrt_b200 import _lib

        self.world, self.M, self.N, self.rows_per = world, M, N, M // world
        dev = "cuda"
        self.recv = [torch.zeros(world, self.rows_per, N, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        self.out = [torch.full((M, N), -7.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        self.codes = [torch.full((M, N), 0x55, dtype=torch.uint8, device=dev) for _ in range(world)]
        self.scales = [torch.full((M,), -1.0, dtype=torch.float32, device=dev) for _ in range(world)]
        self.flags = [torch.zeros(2 * world + 1, dtype=torch.int32, device=dev) for _ in range(world)]
        self.peers, self.gpeers = [], []
        for r in range(world):
            p, g = _lib.Peers(), _lib.GatherPeers()
            p.rank = g.rank = r
            p.world = g.world = world
            for s in range(world):
                p.recv[s] = g.recv[s] = self.recv[s].data_ptr()
                p.flags[s] = g.flags[s] = self.flags[s].data_ptr()
                p.out[s] = self.out[s].data_ptr()
                g.codes[s], g.scales[s] = self.codes[s].data_ptr(), self.scales[s].data_ptr()
            self.peers.append(p)
            self.gpeers.append(g)
        self.epoch = 0
        self.lib = _lib.load()
        self.stream = torch.cuda.current_stream().cuda_stream

    def peers_signalled(self):
        """Opens a new epoch and writes it into every signal word of every rank (not the ticket)."""
        self.epoch += 1
        for f in self.flags:
            f[: 2 * self.world] = self.epoch
        return self.epoch

    def flag_words(self):
        return [f.cpu().tolist() for f in self.flags]


def _check(rc, what):
    assert rc == 0, f"{what} returned {rc}"


def _problem(world, M, N, K, seed, mode="fp8"):
    """Full x [M, K], w [N, K]; rank r holds the K slice r of both (row-parallel linear)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    ks = K // world
    xs = [x[:, r * ks:(r + 1) * ks].contiguous() for r in range(world)]
    ws = [w[:, r * ks:(r + 1) * ks].contiguous() for r in range(world)]
    if mode == "fp8":
        parts = [o.fp8_linear_ref(a, b).bfloat16() for a, b in zip(xs, ws)]
    else:
        parts = [o.nvfp4_linear_ref(a, b).bfloat16() for a, b in zip(xs, ws)]
    return xs, ws, parts


def _gemm_to_owners(capi, rk, xs, ws, mode, tile):
    """Every rank's partial GEMM with the reduce-scatter epilogue, one after the other."""
    from tensorrt_b200 import _lib

    cfg = _lib.cfg_ref(tile_n=tile)
    keep = []
    for r in range(rk.world):
        xd, wd = xs[r].cuda(), ws[r].cuda()
        ks = xd.shape[1]
        if mode == "fp8":
            xc, xsc = capi.fp8_quantize(xd, None)
            wc, wsc = capi.fp8_quantize(wd, capi.row_amax(wd))
            _check(rk.lib.b200q_fp8_gemm_reduce_scatter(xc.data_ptr(), xsc.data_ptr(), xsc.numel(), wc.data_ptr(), wsc.data_ptr(),
                                                        wsc.numel(), ctypes.byref(rk.peers[r]), rk.M, rk.N, ks, rk.stream, cfg),
                   "b200q_fp8_gemm_reduce_scatter")
            keep += [xc, xsc, wc, wsc]
        else:
            xq = capi.nvfp4_quantize(xd, capi.amax(xd))
            wq = capi.nvfp4_quantize(wd, capi.amax(wd))
            _check(rk.lib.b200q_nvfp4_gemm_reduce_scatter(xq[0].data_ptr(), xq[1].data_ptr(), xq[2].data_ptr(), wq[0].data_ptr(),
                                                          wq[1].data_ptr(), wq[2].data_ptr(), ctypes.byref(rk.peers[r]), rk.M, rk.N,
                                                          ks, rk.stream, cfg), "b200q_nvfp4_gemm_reduce_scatter")
            keep += list(xq) + list(wq)
    return keep


CASES = [(2, 512, 512, 1024, 128), (2, 1024, 768, 2048, 256), (2, 2048, 2560, 1024, 512), (4, 1024, 512, 2048, 0),
         (4, 2048, 2560, 2048, 512), (8, 2048, 256, 4096, 128), (8, 4096, 1280, 4096, 512)]


@pytest.mark.parametrize("world,M,N,K,tile", CASES)
@pytest.mark.parametrize("mode", ["fp8", "nvfp4"])
def test_fused_all_reduce_loopback(b200, mode, world, M, N, K, tile):
    """GEMM (reduce-scatter epilogue) -> b200q_reduce_gather on every virtual rank: every rank's output
    equals the sum of the `world` partial linears (+ bias once), within the GEMM tolerance of the oracle;
    all ranks hold the same bits; a second pass with a new epoch reuses buffers and flags."""
    capi = b200.capi
    xs, ws, parts = _problem(world, M, N, K, seed=world + M + N + K, mode=mode)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(3)) * 0.05).bfloat16()
    ref = o.all_reduce_ref(parts, torch.float32) + bias.float()
    rk = Ranks(world, M, N)
    bias_d = bias.cuda()
    for _ in range(2):
        keep = _gemm_to_owners(capi, rk, xs, ws, mode, tile)
        epoch = rk.peers_signalled()
        for r in range(world):
            _check(rk.lib.b200q_reduce_gather(ctypes.byref(rk.peers[r]), bias_d.data_ptr(), M, N, epoch, rk.stream, None),
                   "b200q_reduce_gather")
        torch.cuda.synchronize()
        del keep
        assert capi.device_status() == 0
        # the receive slot s of rank r holds rank s's partial of the rows r owns
        for r in range(world):
            for s in range(world):
                got = rk.recv[r][s].float().cpu()
                want = parts[s][r * rk.rows_per:(r + 1) * rk.rows_per].float()
                assert o.rel_l2(got, want) <= 1e-2, (r, s)
        for r in range(world):
            assert torch.equal(rk.out[r], rk.out[0])
        assert o.rel_l2(rk.out[0].float().cpu(), ref) <= 1e-2
        # every rank signalled both phases to every peer, and re-armed its ticket
        for words in rk.flag_words():
            assert words[: 2 * world] == [epoch] * (2 * world) and words[2 * world] == 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_known_answer_through_the_fused_reduction(b200, world):
    """The reference's all-reduce check (tests/py/dynamo/distributed/test_native_nccl.py:1666-1692:
    rank r contributes full(r + 1), every rank expects W (W + 1) / 2) through the peer-memory
    reduction: rank s's contribution sits in slot s of every owner's receive buffer."""
    M, N = world * 128, 64
    rk = Ranks(world, M, N)
    for r in range(world):
        for s in range(world):
            rk.recv[r][s] = float(s + 1)
    epoch = rk.peers_signalled()
    for r in range(world):
        _check(rk.lib.b200q_reduce_gather(ctypes.byref(rk.peers[r]), None, M, N, epoch, rk.stream, None), "b200q_reduce_gather")
    torch.cuda.synchronize()
    assert b200.capi.device_status() == 0
    for r in range(world):
        assert torch.allclose(rk.out[r].float().cpu(), torch.full((M, N), world * (world + 1) / 2), atol=1e-3, rtol=1e-3)


# the last three: persistent CTAs that walk 4 and 7 tokens each (ring stages reused across tokens), and
# a row too long for the ring (one CTA per token)
@pytest.mark.parametrize("world,M,N,K", [(2, 512, 512, 1024), (4, 1024, 1024, 2048), (8, 2048, 2048, 4096), (2, 256, 8192, 512),
                                         (2, 2048, 4096, 512), (8, 16384, 1024, 1024), (2, 256, 16384, 512)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_reduce_norm_quantize_gather_loopback(b200, world, M, N, K, with_bias):
    """Token-sharded form: GEMM (reduce-scatter epilogue) -> reduce + bias + residual add + RMSNorm +
    per-token FP8 quantize + gather.  The residual rows each rank keeps are updated exactly as the
    oracle's (fp32 sum of the bf16 partials in rank order, one rounding, bf16 add); the gathered
    codes and scales agree with the oracle's quantized norm up to the bf16 rounding flips an fp32
    sum order allows, are the same bits on every rank, and the last step of a stack
    (b200q_reduce_add_gather) returns residual + sum."""
    capi = b200.capi
    xs, ws, parts = _problem(world, M, N, K, seed=11 + world + N)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(M, N, generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(N, generator=g)).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.05).bfloat16() if with_bias else None
    total = o.all_reduce_ref(parts, torch.float32)
    if bias is not None:
        total = total + bias.float()
    delta = total.bfloat16()
    h_new = (h.float() + delta.float()).bfloat16()
    x_ref = o.rms_norm_ref(h_new, nw)
    c_ref, s_ref = o.fp8_quantize(x_ref, o.row_amax(x_ref))

    rk = Ranks(world, M, N)
    rp = rk.rows_per
    h_sh = [h[r * rp:(r + 1) * rp].contiguous().cuda() for r in range(world)]
    nw_d = nw.cuda()
    b_d = None if bias is None else bias.cuda()
    keep = _gemm_to_owners(capi, rk, xs, ws, "fp8", 0)
    epoch = rk.peers_signalled()
    f = rk.lib.b200q_reduce_add_rms_norm_fp8_quantize_gather
    for r in range(world):
        _check(f(ctypes.byref(rk.gpeers[r]), None if b_d is None else b_d.data_ptr(), h_sh[r].data_ptr(), nw_d.data_ptr(), 1e-5, M, N,
                 epoch, rk.stream, None), "b200q_reduce_add_rms_norm_fp8_quantize_gather")
    torch.cuda.synchronize()
    del keep
    assert capi.device_status() == 0
    got_h = torch.cat([t.cpu() for t in h_sh])
    # partial GEMM outputs differ from the oracle's in the last bf16 bit here and there, so does their sum
    assert o.rel_l2(got_h.float(), h_new.float()) <= 2e-3
    for r in range(1, world):
        assert torch.equal(rk.codes[r], rk.codes[0]) and torch.equal(rk.scales[r], rk.scales[0])
    codes, scales = rk.codes[0].cpu(), rk.scales[0].cpu()
    assert torch.allclose(scales, s_ref.reshape(-1), rtol=2e-2)
    deq = o.fp8_dequantize(codes, scales.view(-1, 1))
    assert o.rel_l2(deq, x_ref.float()) <= 4e-2
    # against the device's own unfused kernels on the same reduced input: same rounding points
    recv_sum = torch.zeros(world, rp, N, device="cuda")
    for s in range(world):                               # rank order, as the kernel sums
        recv_sum += torch.stack([rk.recv[r][s].float() for r in range(world)])
    recv_sum = recv_sum.view(M, N)
    if b_d is not None:
        recv_sum = recv_sum + b_d.float()
    h2, c2, s2 = capi.add_rms_norm_fp8_quantize(h.cuda(), recv_sum.bfloat16(), nw_d, 1e-5)
    assert torch.equal(h2.cpu(), got_h)
    assert torch.allclose(rk.scales[0], s2, rtol=1e-2) and (rk.codes[0] != c2).float().mean().item() < 2e-2

    # last step of a stack: out = residual shard + reduced partials, full result on every rank
    h_sh2 = [h[r * rp:(r + 1) * rp].contiguous().cuda() for r in range(world)]
    epoch = rk.peers_signalled()
    for r in range(world):
        _check(rk.lib.b200q_reduce_add_gather(ctypes.byref(rk.peers[r]), None if b_d is None else b_d.data_ptr(), h_sh2[r].data_ptr(), M, N,
                                              epoch, rk.stream, None), "b200q_reduce_add_gather")
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    for r in range(world):
        assert torch.equal(rk.out[r].cpu(), got_h)


def test_row_parallel_bias_is_added_once(b200):
    """Bias convention of the fused path: the owner of a row adds the bias after the sum, so every
    rank passes the same full bias and the result carries it exactly once, whatever the rank count."""
    for world in (2, 4):
        M, N = world * 128, 128
        rk = Ranks(world, M, N)
        bias = torch.arange(N, dtype=torch.float32).bfloat16().cuda()
        epoch = rk.peers_signalled()                      # receive buffers are all zero: the result is the bias alone
        for r in range(world):
            _check(rk.lib.b200q_reduce_gather(ctypes.byref(rk.peers[r]), bias.data_ptr(), M, N, epoch, rk.stream, None), "b200q_reduce_gather")
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(rk.out[r], bias.expand(M, N))


@pytest.mark.parametrize("world,M,N,K", [(2, 64, 8192, 2048), (4, 64, 4096, 4096), (8, 64, 8192, 8192), (8, 1, 1024, 1024), (2, 128, 16384, 512)])
def test_pull_all_reduce_loopback(b200, world, M, N, K):
    """Decode-sized all-reduce by pulling: every virtual rank's small-M GEMM writes its partial into its
    own buffer and signals; every rank's reduction then reads all partials, adds bias and residual,
    applies RMSNorm and quantizes.  Launch order on the one stream: all GEMMs and signals first, then
    the reductions, so no kernel waits for one that has not run.  Three all-reduces in a row alternate
    between the two partial buffers and advance the on-device call counter; the third ends the stack
    (no norm).  All ranks must produce the same bits; h is exact against the oracle's order of sums."""
    from tensorrt_b200 import _lib

    capi, lib = b200.capi, _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    partial = [[torch.zeros(M, N, dtype=torch.bfloat16, device="cuda") for _ in range(2)] for _ in range(world)]
    flags = [torch.zeros(world + 1, dtype=torch.int32, device="cuda") for _ in range(world)]
    peers = []
    for slot in range(2):
        per_rank = []
        for r in range(world):
            p = _lib.PullPeers()
            p.rank, p.world = r, world
            for s in range(world):
                p.partial[s], p.flags[s] = partial[s][slot].data_ptr(), flags[s].data_ptr()
            per_rank.append(p)
        peers.append(per_rank)
    g = torch.Generator().manual_seed(world * 1000 + N)
    h0 = torch.randn(M, N, generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(N, generator=g)).bfloat16()
    bias = (torch.randn(N, generator=g) * 0.05).bfloat16()
    h_dev = [h0.clone().cuda() for _ in range(world)]
    h_ref = h0.clone()
    nw_d, bias_d = nw.cuda(), bias.cuda()
    for call in range(3):
        slot, last = call & 1, call == 2
        xs, ws, parts = _problem(world, M, N, K, seed=call + world + N)
        keep = []
        for r in range(world):
            xc, xsc = capi.fp8_quantize(xs[r].cuda(), None)
            wc, wsc = capi.fp8_quantize(ws[r].cuda(), capi.row_amax(ws[r].cuda()))
            capi.fp8_gemm(xc, xsc, wc, wsc, None, out=partial[r][slot])
            _check(lib.b200q_pull_signal(ctypes.byref(peers[slot][r]), stream), "b200q_pull_signal")
            keep += [xc, xsc, wc, wsc]
        outs = []
        for r in range(world):
            if last:
                _check(lib.b200q_pull_reduce_add(ctypes.byref(peers[slot][r]), bias_d.data_ptr(), h_dev[r].data_ptr(), M, N, stream, None),
                       "b200q_pull_reduce_add")
            else:
                codes = torch.empty(M, N, dtype=torch.uint8, device="cuda")
                scales = torch.empty(M, dtype=torch.float32, device="cuda")
                _check(lib.b200q_pull_reduce_add_rms_norm_fp8_quantize(
                    ctypes.byref(peers[slot][r]), bias_d.data_ptr(), h_dev[r].data_ptr(), nw_d.data_ptr(), 1e-5, codes.data_ptr(),
                    scales.data_ptr(), M, N, stream, None), "b200q_pull_reduce_add_rms_norm_fp8_quantize")
                outs.append((codes, scales))
        torch.cuda.synchronize()
        del keep
        assert capi.device_status() == 0
        # the device's own partials, summed in rank order as the kernel does
        acc = torch.zeros(M, N, device="cuda")
        for s in range(world):
            acc += partial[s][slot].float()
            assert o.rel_l2(partial[s][slot].float().cpu(), parts[s].float()) <= 1e-2
        delta = (acc + bias_d.float()).bfloat16()
        h_ref = (h_ref.float() + delta.float().cpu()).bfloat16()
        for r in range(world):
            assert torch.equal(h_dev[r].cpu(), h_ref), (call, r)
        for words in (f.cpu().tolist() for f in flags):
            assert words == [call + 1] * (world + 1)                  # every peer's signal and the own call counter
        if not last:
            for r in range(1, world):
                assert torch.equal(outs[r][0], outs[0][0]) and torch.equal(outs[r][1], outs[0][1])
            x_ref = o.rms_norm_ref(h_ref, nw)
            c_ref, s_ref = o.fp8_quantize(x_ref, o.row_amax(x_ref))
            assert torch.allclose(outs[0][1].cpu(), s_ref.reshape(-1), rtol=2e-2)
            assert o.rel_l2(o.fp8_dequantize(outs[0][0].cpu(), outs[0][1].cpu().view(-1, 1)), x_ref.float()) <= 4e-2
            _, c2, s2 = capi.add_rms_norm_fp8_quantize(h_ref.cuda(), None, nw_d, 1e-5)     # the unfused kernel on the same h
            assert torch.allclose(outs[0][1], s2, rtol=1e-2) and (outs[0][0] != c2).float().mean().item() < 2e-2


def test_a_wait_for_a_peer_that_never_arrives_runs_out(b200):
    """Rank 0 of a 2-rank group calls the reduction, rank 1 never does and nothing sets its flag.
    With a 50 ms limit (b200q_cfg::peer_wait_ms) the wait gives up by itself: the kernels return, the
    device status reports B200Q_ERR_TIMEOUT, the output is untouched, resetting the status clears it
    and the same buffers then serve a normal step."""
    from tensorrt_b200 import _lib

    capi = b200.capi
    world, M, N = 2, 256, 64
    rk = Ranks(world, M, N)
    assert capi.device_status() == 0
    rk.recv[0][:] = 1.0
    rk.recv[1][:] = 1.0
    rk.epoch = 1
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    _check(rk.lib.b200q_reduce_gather(ctypes.byref(rk.peers[0]), None, M, N, 1, rk.stream, _lib.cfg_ref(peer_wait_ms=50)),
           "b200q_reduce_gather")
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1)
    assert 40 <= ms <= 1000, ms                         # gave up near the limit asked for, not at the 2 s default
    assert capi.device_status(reset=False) == -6        # B200Q_ERR_TIMEOUT, and it stays set until reset
    assert capi.device_status(reset=False) == -6
    assert float(rk.out[0].float().min()) == -7.0 and float(rk.out[1].float().max()) == -7.0   # skipped: outputs untouched
    # rank 0 did signal rank 1 (and itself) before it waited
    assert rk.flags[1].cpu().tolist()[0] == 1 and rk.flags[0].cpu().tolist()[0] == 1
    # while the status is set, reductions skip their work instead of producing partial results
    epoch = rk.peers_signalled()
    _check(rk.lib.b200q_reduce_gather(ctypes.byref(rk.peers[0]), None, M, N, epoch, rk.stream, None), "b200q_reduce_gather")
    torch.cuda.synchronize()
    assert float(rk.out[0].float().max()) == -7.0
    assert capi.device_status(reset=True) == -6
    assert capi.device_status() == 0
    # after the reset the group works again
    epoch = rk.peers_signalled()
    for r in range(world):
        _check(rk.lib.b200q_reduce_gather(ctypes.byref(rk.peers[r]), None, M, N, epoch, rk.stream, None), "b200q_reduce_gather")
    torch.cuda.synchronize()
    assert capi.device_status() == 0
    for r in range(world):
        assert torch.equal(rk.out[r].float().cpu(), torch.full((M, N), 2.0))
