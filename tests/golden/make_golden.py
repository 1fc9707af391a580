"""Regenerates the fixtures in this directory:  python tests/golden/make_golden.py

The reference tree holds no golden vectors for FP8/NVFP4 codes or scales, and its eager
implementation of the two quantize ops lives in a third-party package that is not part of
it, so these fixtures are produced by the CPU oracle (oracle/quant_oracle.py) on seeded
inputs.  They pin the oracle against accidental change and give the GPU tests vectors that
do not depend on the oracle being importable next to them.  `formats.npz` is independent of
the oracle's encoders: it is built from the number-format definitions and from torch's own
float8_e4m3fn dtype.
"""
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
import oracle as o  # noqa: E402


def formats():
    e4m3 = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    e2m1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)
    # every tie and the values either side of it, for both formats
    ties_e2m1 = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    probe_e2m1 = np.concatenate([ties_e2m1, np.nextafter(ties_e2m1, np.float32(0)), np.nextafter(ties_e2m1, np.float32(9)),
                                 [0.0, 6.0, 7.0, 100.0]]).astype(np.float32)
    probe_e2m1 = np.concatenate([probe_e2m1, -probe_e2m1])
    code_e2m1 = o.e2m1_encode(torch.from_numpy(probe_e2m1)).numpy()
    np.savez(HERE / "formats.npz", e4m3=e4m3, e2m1=e2m1, probe_e2m1=probe_e2m1, code_e2m1=code_e2m1)


def cases():
    out = {}
    g = torch.Generator().manual_seed(1234)
    for name, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        x = torch.randn(48, 160, generator=g)
        x[torch.rand(48, 160, generator=g) < 0.02] *= 40
        x[5] = 0                      # an all-zero row / zero blocks
        x[7, :16] = -0.0              # negative zeros
        x[9, 16:32] *= 1e-6           # a block far below the tensor amax (stored scale rounds to 0)
        x = x.to(dtype)
        amax_t = x.float().abs().max()
        amax_r = o.row_amax(x)
        c_t, s_t = o.fp8_quantize(x, amax_t)
        c_r, s_r = o.fp8_quantize(x, amax_r)
        p, sc, gs = o.nvfp4_quantize(x, amax_t)
        out[f"{name}_x"] = x.float().numpy()  # exactly representable in the narrow dtype
        out[f"{name}_fp8_tensor_codes"] = c_t.numpy()
        out[f"{name}_fp8_tensor_scale"] = s_t.numpy()
        out[f"{name}_fp8_row_codes"] = c_r.numpy()
        out[f"{name}_fp8_row_scale"] = s_r.numpy()
        out[f"{name}_fp8_fake"] = o.fp8_fake_quant(x, amax_r).float().numpy()
        out[f"{name}_nvfp4_codes"] = p.numpy()
        out[f"{name}_nvfp4_scales"] = sc.numpy()
        out[f"{name}_nvfp4_scales_swizzled"] = o.swizzle_scales(sc).numpy()
        out[f"{name}_nvfp4_global"] = gs.numpy()
        out[f"{name}_nvfp4_fake"] = o.nvfp4_fake_quant(x, amax_t).float().numpy()
    # a static amax below the true maximum: saturation path
    x = (torch.randn(16, 64, generator=g) * 3).bfloat16()
    small = torch.tensor(2.0)
    out["sat_x"] = x.float().numpy()
    out["sat_fp8_codes"] = o.fp8_quantize(x, small)[0].numpy()
    p, sc, gs = o.nvfp4_quantize(x, small)
    out["sat_nvfp4_codes"], out["sat_nvfp4_scales"] = p.numpy(), sc.numpy()
    # small linear: config "FP8 per-tensor Q/DQ Linear" shape family, reduced
    xl = torch.randn(16, 256, generator=g).bfloat16()
    wl = (torch.randn(64, 256, generator=g) * 0.02).bfloat16()
    bl = (torch.randn(64, generator=g) * 0.01).bfloat16()
    out["lin_x"], out["lin_w"], out["lin_b"] = xl.float().numpy(), wl.float().numpy(), bl.float().numpy()
    out["lin_fp8"] = o.fp8_linear_ref(xl, wl, bl).numpy()
    out["lin_fp8_tensor"] = o.fp8_linear_ref(xl, wl, bl, xl.float().abs().max(), wl.float().abs().max()).numpy()
    out["lin_nvfp4"] = o.nvfp4_linear_ref(xl, wl, bl).numpy()
    np.savez_compressed(HERE / "cases.npz", **out)


def layers():
    """Attention, all-reduce and decoder-layer restatements on small seeded inputs (outputs are compared within
    a bf16 unit in the last place: the fp32 sums inside may be ordered differently on another CPU)."""
    out = {}
    g = torch.Generator().manual_seed(4321)
    q = torch.randn(1, 4, 40, 32, generator=g).half()
    k = torch.randn(1, 2, 40, 32, generator=g).half()
    v = torch.randn(1, 2, 40, 32, generator=g).half()
    am = torch.tensor(3.5)
    out["sdpa_q"], out["sdpa_k"], out["sdpa_v"] = q.float().numpy(), k.float().numpy(), v.float().numpy()
    out["sdpa_full"] = o.fp8_sdpa_ref(q, k, v, am, am, am).float().numpy()
    out["sdpa_causal"] = o.fp8_sdpa_ref(q, k, v, am, am, am, is_causal=True).float().numpy()
    out["sdpa_causal_short_q"] = o.fp8_sdpa_ref(q[:, :, -8:], k, v, am, am, am, is_causal=True).float().numpy()   # lower-right mask
    parts = [(torch.randn(6, 16, generator=g) * 3).bfloat16() for _ in range(4)]
    out["ar_parts"] = torch.stack(parts).float().numpy()
    out["ar_sum"] = o.all_reduce_ref(parts, torch.bfloat16).float().numpy()
    hidden, n_q, n_kv, hd, ffn = 64, 4, 2, 16, 128
    rnd = lambda r, c: (torch.randn(r, c, generator=g) * 0.05).bfloat16()  # noqa: E731
    layer = {"norm1": (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16(), "norm2": (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16(),
             "wqkv": rnd((n_q + 2 * n_kv) * hd, hidden), "wo": rnd(hidden, n_q * hd), "wgu": rnd(2 * ffn, hidden), "wdown": rnd(hidden, ffn)}
    h = torch.randn(16, hidden, generator=g).bfloat16()
    for key, t in layer.items():
        out[f"layer_{key}"] = t.float().numpy()
    out["layer_h"] = h.float().numpy()
    for mode in ("fp8", "nvfp4"):
        for world in (1, 2):
            out[f"layer_{mode}_w{world}"] = o.decoder_layer_ref(h, layer, n_q, n_kv, hd, mode, world=world).float().numpy()
    out["layer_fp8_sdpa_w2"] = o.decoder_layer_ref(h, layer, n_q, n_kv, hd, "fp8", world=2, attention="fp8_sdpa", seq_len=8).float().numpy()
    np.savez_compressed(HERE / "layers.npz", **out)


if __name__ == "__main__":
    formats()
    cases()
    layers()
    print("wrote", [p.name for p in HERE.glob("*.npz")])
