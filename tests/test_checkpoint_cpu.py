"""Checkpoint readers (native fp8 and compressed-tensors layouts, fused modules, expert stacks, TP shards) on CPU:
bytes must come through untouched, scales cast once to FP16, and the loaded layout must dequantise to exactly what the
reference's torch path gives (``w.to(fp16) * scale.to(fp16)`` expanded per block / row)."""
import json

import numpy as np
import pytest
import torch

from oracle import dequant as odq, linear as olin
from vllm_fp8_w8a16_sm70_b200 import checkpoint as ck

st = pytest.importorskip("safetensors.torch")


def _quant(N, K, seed, scheme="block"):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.02
    if scheme == "block":
        q, s = olin.quantize_block_fp8(w)
    else:
        q, s = olin.quantize_channel_fp8(w)
    return q, s          # uint8 [N,K], fp32 scales


def _ref_dequant(q_u8, scale_grid_fp16, block_h):
    """The reference's torch dequant (compressed_tensors_v100.py:231-270), restated."""
    N, K = q_u8.shape
    w16 = q_u8.view(torch.float8_e4m3fn).to(torch.float16)
    s = scale_grid_fp16.repeat_interleave(block_h, 0).repeat_interleave(128, 1)[:N, :K]
    return w16 * s


def _dq(w: ck.Fp8Weight):
    return torch.from_numpy(odq.dequant_block_scaled(w.weight.numpy(), w.scale, w.N, w.K, w.block_h, 128).copy())


def test_native_fp8_linear_from_file(tmp_path):
    q, s = _quant(256, 384, 1)
    f = tmp_path / "m.safetensors"
    st.save_file({"l.q.weight": q.view(torch.float8_e4m3fn), "l.q.weight_scale_inv": s.to(torch.bfloat16),
                  "l.q.bias": torch.arange(256, dtype=torch.bfloat16)}, str(f))
    w = ck.load_linear(f, "l.q")
    assert w.block_h == 128 and w.weight.dtype == torch.uint8 and torch.equal(w.weight, q)
    assert w.scale.dtype == torch.float16 and torch.equal(w.scale, s.to(torch.bfloat16).to(torch.float16))
    assert w.bias.dtype == torch.float16 and w.bias[5] == 5
    assert torch.equal(_dq(w), _ref_dequant(q, w.scale, 128))


def test_compressed_tensors_layouts_are_told_apart():
    q, s = _quant(256, 384, 2)
    blk = ck.load_linear({"a.weight": q.view(torch.float8_e4m3fn), "a.weight_scale": s}, "a")
    assert blk.block_h == 128 and tuple(blk.scale.shape) == (2, 3)
    qc, sc = _quant(200, 176, 3, "channel")
    ch = ck.load_linear({"b.weight": qc, "b.weight_scale": sc.reshape(200, 1)}, "b")
    assert ch.block_h == 1 and tuple(ch.scale.shape) == (200, 2)
    assert torch.equal(_dq(ch), qc.view(torch.float8_e4m3fn).to(torch.float16) * sc.to(torch.float16).reshape(200, 1))
    tn = ck.load_linear({"c.weight": qc, "c.weight_scale": torch.tensor(0.01)}, "c")
    assert tn.block_h == 1 and torch.all(tn.scale == torch.tensor(0.01, dtype=torch.float16))
    with pytest.raises(KeyError):
        ck.load_linear({"d.weight": q}, "d")
    with pytest.raises(ValueError):
        ck.load_linear({"e.weight": q, "e.weight_scale": torch.ones(7)}, "e")
    with pytest.raises(ValueError):
        ck.load_linear({"f.weight": q.float(), "f.weight_scale_inv": s}, "f")
    with pytest.raises(ValueError, match="FP16"):
        ck.block_weight(q, torch.full((2, 3), 1e6))


def test_tensor_scales_of_a_fused_module_expand_per_logical_part():
    q, _ = _quant(384, 256, 4)
    w = ck.tensor_weight(q, torch.tensor([0.5, 0.25, 2.0]), [256, 64, 64])
    assert w.block_h == 1 and w.logical_widths == [256, 64, 64]
    assert torch.all(w.scale[:256] == 0.5) and torch.all(w.scale[256:320] == 0.25) and torch.all(w.scale[320:] == 2.0)
    with pytest.raises(ValueError):
        ck.tensor_weight(q, torch.tensor([0.5, 0.25]), [256, 64, 64])


def test_fused_qkv_equals_concatenation_and_rejects_straddling_blocks():
    parts = {}
    for i, (name, n) in enumerate((("q", 512), ("k", 128), ("v", 128))):
        q, s = _quant(n, 256, 10 + i)
        parts[f"attn.{name}_proj.weight"] = q
        parts[f"attn.{name}_proj.weight_scale_inv"] = s
    w = ck.load_fused(parts, ["attn.q_proj", "attn.k_proj", "attn.v_proj"])
    assert (w.N, w.K) == (768, 256) and w.logical_widths == [512, 128, 128] and tuple(w.scale.shape) == (6, 2)
    x = torch.randn(3, 256).to(torch.float16)
    y = olin.oracle_linear_fp32(x, w.weight, w.scale, 128)
    yq = olin.oracle_linear_fp32(x, parts["attn.q_proj.weight"], parts["attn.q_proj.weight_scale_inv"].to(torch.float16), 128)
    yv = olin.oracle_linear_fp32(x, parts["attn.v_proj.weight"], parts["attn.v_proj.weight_scale_inv"].to(torch.float16), 128)
    assert torch.equal(y[:, :512], yq) and torch.equal(y[:, 640:], yv)
    q_odd, s_odd = _quant(192, 256, 20)
    with pytest.raises(ValueError, match="multiple of 128"):
        ck.fuse_column([ck.block_weight(q_odd, s_odd), ck.block_weight(parts["attn.k_proj.weight"], parts["attn.k_proj.weight_scale_inv"])])
    # channel-scaled parts may have any height
    qa, sa = _quant(192, 256, 21, "channel")
    qb, sb = _quant(64, 256, 22, "channel")
    f = ck.fuse_column([ck.channel_weight(qa, sa), ck.channel_weight(qb, sb)])
    assert f.block_h == 1 and f.N == 256 and tuple(f.scale.shape) == (256, 2)


def test_expert_stack_from_sharded_directory(tmp_path):
    E, I, H = 4, 128, 256
    files = {"a.safetensors": {}, "b.safetensors": {}}
    wmap = {}
    want13, want2 = [], []
    for e in range(E):
        g, gs = _quant(I, H, 100 + e)
        u, us = _quant(I, H, 200 + e)
        d, ds = _quant(H, I, 300 + e)
        want13.append(torch.cat([g, u]))
        want2.append(d)
        for nm, (w, s) in (("gate_proj", (g, gs)), ("up_proj", (u, us)), ("down_proj", (d, ds))):
            fn = "a.safetensors" if e % 2 == 0 else "b.safetensors"
            for key, t in ((f"mlp.experts.{e}.{nm}.weight", w.view(torch.float8_e4m3fn)), (f"mlp.experts.{e}.{nm}.weight_scale_inv", s.to(torch.bfloat16))):
                files[fn][key] = t
                wmap[key] = fn
    for fn, tensors in files.items():
        st.save_file(tensors, str(tmp_path / fn))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wmap}))
    ex = ck.load_experts(tmp_path, "mlp.experts")
    assert tuple(ex.w13.shape) == (E, 2 * I, H) and tuple(ex.w2.shape) == (E, H, I) and ex.block_h == 128
    assert tuple(ex.s13.shape) == (E, 2, 2) and tuple(ex.s2.shape) == (E, 2, 1) and ex.s13.dtype == torch.float16
    assert torch.equal(ex.w13, torch.stack(want13)) and torch.equal(ex.w2, torch.stack(want2))
    loc = ex.local(2, 1)
    assert torch.equal(loc.w13, ex.w13[2:]) and loc.w2.shape[0] == 2
    with pytest.raises(ValueError):
        ex.local(3, 0)


def test_tp_shards_reassemble_the_full_layer():
    tp = 2
    parts = [ck.block_weight(*_quant(n, 512, 30 + i)) for i, n in enumerate((512, 256, 256))]
    fused = ck.fuse_column(parts)
    x = torch.randn(4, 512).to(torch.float16)
    y_full = olin.oracle_linear_fp32(x, fused.weight, fused.scale, 128)
    starts = [0, 512, 768]
    for r in range(tp):
        sh = ck.shard(fused, "column", tp, r)
        assert sh.logical_widths == [256, 128, 128] and sh.N == 512
        y = olin.oracle_linear_fp32(x, sh.weight, sh.scale, 128)
        col = 0
        for s0, wd in zip(starts, (256, 128, 128)):
            assert torch.equal(y[:, col:col + wd], y_full[:, s0 + r * wd:s0 + (r + 1) * wd])
            col += wd
    # row-parallel: partial products of the K shards add up to the full product
    down = ck.block_weight(*_quant(256, 512, 40), bias=torch.ones(256))
    acc = torch.zeros(4, 256)
    for r in range(tp):
        sh = ck.shard(down, "row", tp, r)
        assert (sh.bias is not None) == (r == 0)
        acc += olin.oracle_linear_fp32(x[:, r * 256:(r + 1) * 256].contiguous(), sh.weight, sh.scale, 128)
    ref = olin.oracle_linear_fp32(x, down.weight, down.scale, 128)
    assert torch.allclose(acc, ref, atol=1e-3, rtol=1e-3)
    # channel scales allow a K shard that is not a multiple of 128 (1408 / 8 = 176)
    qc, sc = _quant(128, 1408, 41, "channel")
    ch = ck.channel_weight(qc, sc)
    sh = ck.shard(ch, "row", 8, 3)
    assert (sh.N, sh.K) == (128, 176) and tuple(sh.scale.shape) == (128, 2) and sh.block_h == 1
    with pytest.raises(ValueError):
        ck.shard(ck.block_weight(*_quant(128, 1408, 42)), "row", 8, 0)


def test_module_construction_follows_the_reference_positional_order(tmp_path):
    """``FP8W8A16Linear(ext, weight_fp8, weight_scale, block_h, block_w, bias)`` and
    ``from_safetensors(ext, st_path, weight_key, scale_key)`` exactly as the reference's own test constructs it
    (reference: tests/test_phase_b_module.py:178, src/fp8_w8a16_sm70/module.py:31-40, 65-76).  No kernel runs."""
    from vllm_fp8_w8a16_sm70_b200 import FP8W8A16Linear
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(256, 384, generator=g) * 0.02).to(torch.float8_e4m3fn)
    s = torch.rand(2, 3, generator=g).to(torch.bfloat16)
    f = tmp_path / "one.safetensors"
    st.save_file({"l.weight": w, "l.weight_scale_inv": s}, str(f))
    ext = object()
    layer = FP8W8A16Linear.from_safetensors(ext, f, "l.weight", "l.weight_scale_inv", device="cpu")
    assert layer.ext is ext and (layer.N, layer.K, layer.block_h, layer.block_w) == (256, 384, 128, 128)
    assert layer.weight_fp8.dtype == torch.uint8 and layer.weight_fp8.numel() == 256 * 384
    assert torch.equal(layer.weight_fp8.reshape(256, 384), w.view(torch.uint8))
    assert layer.weight_scale.dtype == torch.float16 and torch.equal(layer.weight_scale.reshape(2, 3), s.to(torch.float16))
    again = FP8W8A16Linear(None, w.view(torch.uint8), s.to(torch.float16), 128, 128, torch.zeros(256))
    assert again.bias is not None and again.bias.dtype == torch.float16
    with pytest.raises(AssertionError):
        FP8W8A16Linear(None, w, s.to(torch.float16))            # float8 tensor where raw bytes are expected
    with pytest.raises(RuntimeError):
        layer(torch.zeros(1, 384, dtype=torch.float16))         # CPU input: the engine has no CPU path
