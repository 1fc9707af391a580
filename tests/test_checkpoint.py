"""ModelOpt Hugging Face checkpoint -> GEMM operand layouts (tensorrt_b200/checkpoint.py).

The checkpoints are synthetic: weights ~ N(0, 0.02) quantized by the CPU oracle and written with
the tensor names, dtypes and shapes the reference reads (tools/llm/quantize_utils.py:181-266)."""
import json
import os

import pytest
import torch

import oracle as o

N, K = 256, 512
NAMES = ["model.layers.0.self_attn.q_proj", "model.layers.0.self_attn.o_proj", "model.layers.0.mlp.down_proj", "lm_head"]


def _write_checkpoint(path, algo, bias=True):
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(5)
    tensors, truth = {}, {}
    for i, name in enumerate(NAMES):
        w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
        amax = w.float().abs().max()
        in_amax = torch.tensor(3.0 + i)
        if algo == "FP8":
            codes, scale = o.fp8_quantize(w, amax)
            tensors[name + ".weight"] = codes.view(torch.float8_e4m3fn)
            tensors[name + ".weight_scale"] = scale.reshape(()).float()
            tensors[name + ".input_scale"] = (in_amax / 448.0).reshape(())
            truth[name] = (codes, scale.reshape(1).float())
        else:
            codes, scales, gscale = o.nvfp4_quantize(w, amax)
            tensors[name + ".weight"] = codes
            tensors[name + ".weight_scale"] = scales.view(torch.float8_e4m3fn)
            tensors[name + ".weight_scale_2"] = gscale.reshape(()).float()
            tensors[name + ".input_scale"] = (in_amax / (448.0 * 6.0)).reshape(())
            truth[name] = (codes, scales, gscale.reshape(1).float())
        if bias:
            tensors[name + ".bias"] = (torch.randn(N, generator=g) * 0.01).bfloat16()
        truth[name] += (w, in_amax)
    tensors["model.norm.weight"] = torch.ones(K).bfloat16()          # an unquantized tensor: ignored
    os.makedirs(path, exist_ok=True)
    half = len(tensors) // 2
    items = list(tensors.items())
    save_file(dict(items[:half]), os.path.join(path, "model-00001-of-00002.safetensors"))
    save_file(dict(items[half:]), os.path.join(path, "model-00002-of-00002.safetensors"))
    with open(os.path.join(path, "hf_quant_config.json"), "w") as f:
        json.dump({"producer": {"name": "modelopt"}, "quantization": {"quant_algo": algo, "kv_cache_quant_algo": None}}, f)
    return truth, tensors


def test_swizzle_matches_the_oracle_layout(b200):
    from tensorrt_b200.checkpoint import swizzle_block_scales

    g = torch.Generator().manual_seed(0)
    for rows, cols in [(128, 4), (256, 32), (130, 9), (5, 1), (384, 66)]:
        s = torch.randint(0, 256, (rows, cols), dtype=torch.uint8, generator=g)
        assert torch.equal(swizzle_block_scales(s), o.swizzle_scales(s).reshape(-1))
        assert torch.equal(swizzle_block_scales(s.view(torch.float8_e4m3fn)), o.swizzle_scales(s).reshape(-1))


@pytest.mark.parametrize("algo", ["FP8", "NVFP4"])
def test_load_keeps_stored_codes(b200, algo, tmp_path):
    from tensorrt_b200 import Fp8Linear, Nvfp4Linear
    from tensorrt_b200.checkpoint import load_quantization_config, load_quantized_linears

    truth, _ = _write_checkpoint(str(tmp_path), algo)
    cfg = load_quantization_config(str(tmp_path))
    assert cfg["quant_algo"] == algo and cfg["model_path"] == str(tmp_path)
    assert load_quantization_config(str(tmp_path / "nowhere")) is None
    lins = load_quantized_linears(str(tmp_path), device="cpu")
    assert sorted(lins) == sorted(NAMES)
    for name, lin in lins.items():
        t = truth[name]
        assert torch.equal(lin.w_codes, t[0])
        assert lin.bias.dtype == torch.bfloat16 and lin.bias.shape == (N,)
        assert torch.allclose(lin.input_amax, t[-1], rtol=1e-6, atol=0)   # scale * 448 (* 6): one rounding away at most
        if algo == "FP8":
            assert isinstance(lin, Fp8Linear) and torch.equal(lin.w_scales, t[1])
        else:
            assert isinstance(lin, Nvfp4Linear)
            assert torch.equal(lin.w_scales, o.swizzle_scales(t[1]).reshape(-1)) and torch.equal(lin.w_global, t[2])
            assert (lin.out_features, lin.in_features) == (N, K)


@pytest.mark.parametrize("algo", ["FP8", "NVFP4"])
def test_tensor_parallel_shards_and_rank_files(b200, algo, tmp_path):
    from tensorrt_b200.checkpoint import LLAMA_TP_PLAN, load_quantized_linears, load_rank_shard, save_rank_shard

    truth, _ = _write_checkpoint(str(tmp_path), algo)
    world = 2
    for rank in range(world):
        lins = load_quantized_linears(str(tmp_path), device="cpu", rank=rank, world=world, plan=LLAMA_TP_PLAN)
        q, od, head = lins[NAMES[0]], lins[NAMES[1]], lins[NAMES[3]]
        kb = 1 if algo == "FP8" else 2                                     # elements per code byte
        rows = slice(rank * N // world, (rank + 1) * N // world)
        cols = slice(rank * K // world // kb, (rank + 1) * K // world // kb)
        assert torch.equal(q.w_codes, truth[NAMES[0]][0][rows])             # colwise: output rows
        assert q.bias.shape == (N // world,)
        assert torch.equal(od.w_codes, truth[NAMES[1]][0][:, cols])         # rowwise: input columns
        assert (od.bias is None) == (rank != 0)                             # bias added once after the sum
        assert torch.equal(head.w_codes, truth[NAMES[3]][0])                # not in the plan: replicated
        if algo == "NVFP4":
            sc = truth[NAMES[1]][1]
            scols = slice(rank * (K // 16) // world, (rank + 1) * (K // 16) // world)
            assert torch.equal(od.w_scales, o.swizzle_scales(sc[:, scols].contiguous()).reshape(-1))
            assert torch.equal(q.w_scales, o.swizzle_scales(truth[NAMES[0]][1][rows].contiguous()).reshape(-1))
        os.makedirs(tmp_path / "shards", exist_ok=True)              # not next to the checkpoint's own files
        shard = str(tmp_path / "shards" / f"rank{rank}.safetensors")
        save_rank_shard(lins, shard)
        back = load_rank_shard(shard, device="cpu")
        assert sorted(back) == sorted(lins)
        for name in lins:
            for (bn, a), (_, b) in zip(lins[name].named_buffers(), back[name].named_buffers()):
                assert torch.equal(a, b), (name, bn)
            assert (back[name].bias is None) == (lins[name].bias is None)
    with pytest.raises(ValueError):
        load_quantized_linears(str(tmp_path), device="cpu", rank=0, world=3, plan=LLAMA_TP_PLAN)
    with pytest.raises(ValueError):
        load_quantized_linears(str(tmp_path), device="cpu", rank=0, world=2, plan={"*.q_proj": "diagonal"})


def test_unsupported_algo_and_missing_config(b200, tmp_path):
    from tensorrt_b200.checkpoint import load_quantized_linears

    with pytest.raises(RuntimeError):
        load_quantized_linears(str(tmp_path), device="cpu")
    with open(tmp_path / "hf_quant_config.json", "w") as f:
        json.dump({"quantization": {"quant_algo": "W4A16_AWQ"}}, f)
    with pytest.raises(RuntimeError, match="Only FP8 or NVFP4"):
        load_quantized_linears(str(tmp_path), device="cpu")


def test_convert_replaces_linears_in_place(b200, tmp_path):
    from tensorrt_b200 import Fp8Linear
    from tensorrt_b200.checkpoint import convert_linear_to_b200_quantized, load_quantization_config

    _write_checkpoint(str(tmp_path), "FP8")

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.o_proj, self.k_proj = (torch.nn.Linear(K, N) for _ in range(3))

    class Layer(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn = Attn()

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.model = torch.nn.Module()
            self.model.layers = torch.nn.ModuleList([Layer()])
            self.lm_head = torch.nn.Linear(K, N)

    m = convert_linear_to_b200_quantized(Model(), load_quantization_config(str(tmp_path)), device="cpu")
    attn = m.model.layers[0].self_attn
    assert isinstance(attn.q_proj, Fp8Linear) and isinstance(attn.o_proj, Fp8Linear) and isinstance(m.lm_head, Fp8Linear)
    assert isinstance(attn.k_proj, torch.nn.Linear)                         # not in the checkpoint: untouched


@pytest.mark.gpu
@pytest.mark.parametrize("algo", ["FP8", "NVFP4"])
def test_loaded_linear_matches_dequantized_reference_on_gpu(b200, algo, tmp_path):
    from tensorrt_b200.checkpoint import load_quantized_linears

    truth, _ = _write_checkpoint(str(tmp_path), algo)
    lins = load_quantized_linears(str(tmp_path), device="cuda")
    g = torch.Generator().manual_seed(9)
    x = torch.randn(96, K, generator=g).bfloat16()
    for name in NAMES[:2]:
        lin, t = lins[name], truth[name]
        # the checkpoint stores the scale, not the amax: amax = scale * 448 (* 6) can be one rounding
        # away from the value the scale was made from, and with bf16 inputs that flips exact ties
        in_amax = lin.input_amax.cpu()
        if algo == "FP8":
            w_hat = o.fp8_dequantize(t[0], t[1])
            x_hat = o.fp8_fake_quant(x, in_amax).float()
        else:
            w_hat = o.nvfp4_dequantize(t[0], t[1], t[2])
            x_hat = o.nvfp4_fake_quant(x, in_amax).float()
        ref = x_hat @ w_hat.float().t() + lin.bias.float().cpu()
        y = lin(x.cuda())
        assert o.rel_l2(y.float().cpu(), ref) <= 1e-2
