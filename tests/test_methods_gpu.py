"""GPU tests of the vLLM-facing hooks (apply / apply_weights / MoE apply) and the Linear module."""
import types

import pytest
import torch

from oracle import linear as olin, moe as omoe
from tests.helpers import make_dense, make_moe

pytestmark = pytest.mark.gpu


def test_fp8_linear_method_apply_3d_bf16_bias(lib):
    # reference: vllm_serve.py:1372-1447 (reshape, FP16 cast, bias, cast back); tests/test_phase_b_module.py
    from vllm_fp8_w8a16_sm70_b200 import Fp8LinearMethod
    x, w, s, bh = make_dense(12, 384, 512, seed=1)
    bias = torch.randn(384) * 0.1
    lay = types.SimpleNamespace(weight=w.cuda().view(torch.float8_e4m3fn), weight_scale_inv=s.to(torch.bfloat16).cuda(),
                                weight_block_size=[128, 128], input_size_per_partition=512, output_size_per_partition=384)
    m = Fp8LinearMethod((128, 128))
    m.process_weights_after_loading(lay)
    xb = x.reshape(3, 4, 512).to(torch.bfloat16).cuda()
    y = m.apply(lay, xb, bias.cuda())
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (3, 4, 384)
    ref = olin.oracle_linear_fp32(xb.reshape(12, 512).to(torch.float16).cpu(), w, s.to(torch.bfloat16)) + bias
    st = olin.error_stats(y.reshape(12, 384).float().cpu(), ref)
    assert st["rel_rms"] < 1.2e-2, st    # one extra BF16 rounding of the output


@pytest.mark.parametrize("strategy", ["block", "channel", "tensor"])
def test_compressed_tensors_apply_weights(lib, strategy):
    from vllm_fp8_w8a16_sm70_b200 import CompressedTensorsW8A16Fp8
    from oracle import dequant
    g = torch.Generator().manual_seed(3)
    N, K, M = 352, 512, 5
    wf = torch.randn(N, K, generator=g) * 0.05
    x = torch.randn(M, K, generator=g).to(torch.float16)
    lay = types.SimpleNamespace()
    if strategy == "block":
        q, s = olin.quantize_block_fp8(wf)
        lay.weight, lay.weight_scale = q.cuda(), s.cuda()
        grid, bh = s, 128
    elif strategy == "channel":
        q, s = olin.quantize_channel_fp8(wf)
        lay.weight, lay.weight_scale = q.cuda(), s.cuda()
        grid, bh = torch.from_numpy(dequant.channel_scales_as_blocks(s, N, K)), 1
    else:
        widths = [128, 64, 160]
        st = torch.tensor([0.011, 0.023, 0.007])
        per_row = torch.repeat_interleave(st, torch.tensor(widths)).reshape(N, 1)
        q = (wf / per_row).to(torch.float8_e4m3fn).view(torch.uint8)
        lay.weight, lay.weight_scale, lay.logical_widths = q.cuda(), st.cuda(), widths
        grid, bh = torch.from_numpy(dequant.channel_scales_as_blocks(per_row, N, K)), 1
    m = CompressedTensorsW8A16Fp8(strategy, (128, 128) if strategy == "block" else None)
    m.process_weights_after_loading(lay)
    y = m.apply_weights(lay, x.cuda())
    olin.check_linear(y.cpu(), x, olin.oracle_linear_fp32(x, q, grid, bh), K)


def test_module_equals_raw_op(lib):
    # reference: tests/test_phase_b_module.py (module == raw kernel bit-exact; 3-D input)
    from vllm_fp8_w8a16_sm70_b200 import FP8W8A16Linear, ops
    x, w, s, bh = make_dense(6, 256, 384, seed=2)
    ext = object()                               # the reference's loaded extension goes first; accepted and unused
    mod = FP8W8A16Linear(ext, w, s.to(torch.float16)).cuda()
    assert mod.ext is ext
    y = mod(x.reshape(2, 3, 384).cuda())
    raw = ops.w8a16_linear(x.cuda(), w.cuda(), s.to(torch.float16).cuda(), 256, 384)
    assert tuple(y.shape) == (2, 3, 256) and torch.equal(y.reshape(6, 256).view(torch.int16), raw.view(torch.int16))


def test_swiglu_mlp_chain(lib):
    # reference: tests/test_phase_c_mlp.py:82-233 (gate/up/down chain; max_abs <= 5e-2, max_rel <= 10 %)
    from vllm_fp8_w8a16_sm70_b200 import ops
    g = torch.Generator().manual_seed(0)
    H, F_, M = 512, 1024, 9
    x = torch.randn(M, H, generator=g).to(torch.float16)
    wg, sg = olin.quantize_block_fp8(torch.randn(2 * F_, H, generator=g) * 0.02)
    wd, sd = olin.quantize_block_fp8(torch.randn(H, F_, generator=g) * 0.02)
    gu = ops.w8a16_linear(x.cuda(), wg.cuda(), sg.cuda(), 2 * F_, H)
    h = (torch.nn.functional.silu(gu[:, :F_]) * gu[:, F_:]).contiguous()
    y = ops.w8a16_linear(h, wd.cuda(), sd.cuda(), H, F_).cpu().float()
    gu_ref = olin.oracle_linear_fp32(x, wg, sg)
    ref = olin.oracle_linear_fp32(omoe.silu_mul(gu_ref, F_).to(torch.float16), wd, sd)
    assert float((y - ref).abs().max()) <= 5e-2
    big = ref.abs() > 0.01 * ref.abs().max()
    assert float(((y - ref).abs() / ref.abs())[big].max()) <= 0.10


def test_moe_method_apply(lib):
    from vllm_fp8_w8a16_sm70_b200 import Fp8MoEMethod
    d = make_moe(8, 128, 256, 7, 2, seed=4)
    lay = types.SimpleNamespace(w13_weight=d["w13"].cuda().view(torch.float8_e4m3fn), w2_weight=d["w2"].cuda().view(torch.float8_e4m3fn),
                                w13_weight_scale_inv=d["s13"].to(torch.bfloat16).cuda(), w2_weight_scale_inv=d["s2"].float().cuda(),
                                activation="silu", expert_map=None, apply_router_weight_on_input=False,
                                intermediate_size_per_partition=128, local_num_experts=8)
    m = Fp8MoEMethod(weight_block_size=(128, 128))
    m.process_weights_after_loading(lay)
    assert lay.w13_weight_scale_inv.dtype == torch.float16
    xb = d["x"].to(torch.bfloat16).cuda()
    y = m.apply(lay, xb, d["tw"].cuda(), d["ids"].cuda(), None)
    assert y.dtype == torch.bfloat16
    y6 = m.apply(lay, xb, d["tw"].cuda(), d["ids"].cuda(), None, None)    # newer vLLM passes one more argument
    assert torch.equal(y.view(torch.int16), y6.view(torch.int16))
    ref = omoe.moe_reference_fp32(xb.to(torch.float16).cpu(), d["tw"], d["ids"], d["w13"], d["s13"].to(torch.bfloat16), d["w2"], d["s2"], 128)
    st = omoe.moe_error_stats(y.float().cpu(), ref)
    assert st["cos"] > 0.9999 and st["l2rel"] < 2e-2, st
    lay.activation = "gelu"     # reference: _moe_activation serves SiLU and GELU (vllm_serve.py:1627-1636)
    yg = m.apply(lay, xb, d["tw"].cuda(), d["ids"].cuda(), None)
    refg = omoe.moe_reference_fp32(xb.to(torch.float16).cpu(), d["tw"], d["ids"], d["w13"], d["s13"].to(torch.bfloat16), d["w2"], d["s2"], 128,
                                   activation="gelu")
    st = omoe.moe_error_stats(yg.float().cpu(), refg)
    assert st["cos"] > 0.9999 and st["l2rel"] < 2e-2, st
    lay.activation = "relu"
    with pytest.raises(NotImplementedError):
        m.apply(lay, xb, d["tw"].cuda(), d["ids"].cuda(), None)


def test_checkpoint_to_module_and_moe(lib, tmp_path):
    """File -> loader -> engine: a fused QKV read from a safetensors file, and an expert stack fed to the MoE layer."""
    st = pytest.importorskip("safetensors.torch")
    from oracle import linear as olin, moe as omoe
    from vllm_fp8_w8a16_sm70_b200 import checkpoint as ck, ops
    g = torch.Generator().manual_seed(3)
    tensors = {}
    for i, (nm, n) in enumerate((("q_proj", 512), ("k_proj", 128), ("v_proj", 128))):
        q8, s = olin.quantize_block_fp8(torch.randn(n, 384, generator=g) * 0.02)
        tensors[f"a.{nm}.weight"] = q8.view(torch.float8_e4m3fn)
        tensors[f"a.{nm}.weight_scale_inv"] = s.to(torch.bfloat16)
    E, I, H, topk, M = 4, 128, 256, 2, 5
    for e in range(E):
        for nm, (n, k) in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I))):
            q8, s = olin.quantize_block_fp8(torch.randn(n, k, generator=g) * 0.05)
            tensors[f"m.experts.{e}.{nm}.weight"] = q8.view(torch.float8_e4m3fn)
            tensors[f"m.experts.{e}.{nm}.weight_scale_inv"] = s.to(torch.bfloat16)
    f = tmp_path / "ckpt.safetensors"
    st.save_file(tensors, str(f))
    qkv = ck.load_fused(f, ["a.q_proj", "a.k_proj", "a.v_proj"])
    mod = ck.to_linear_module(qkv)
    x = torch.randn(7, 384, generator=g).to(torch.float16)
    y = mod(x.cuda())
    stt = olin.error_stats(y.cpu(), olin.oracle_linear_fp32(x, qkv.weight, qkv.scale, 128))
    assert stt["rel_rms"] < 1e-2 and stt["finite"]
    ex = ck.load_experts(f, "m.experts")
    xm = torch.randn(M, H, generator=g).to(torch.float16)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(M)]).to(torch.int32)
    tw = torch.softmax(torch.randn(M, topk, generator=g), -1)
    d = ex.to("cuda")
    out = ops.moe_forward(xm.cuda(), tw.cuda(), ids.cuda(), d.w13, d.s13, d.w2, d.s2, block_h=d.block_h)
    omoe.check_moe(out.cpu(), omoe.moe_reference_fp32(xm, tw, ids, ex.w13, ex.s13, ex.w2, ex.s2))


def test_selfcheck_and_variant_counters(lib, monkeypatch):
    """FP8W8A16_SELFCHECK=1: loading a healthy layer passes; a corrupted scale grid is caught and the layer is refused.
    The library's variant counters move with the calls that were made."""
    from vllm_fp8_w8a16_sm70_b200 import Fp8LinearMethod, CompressedTensorsW8A16Fp8, _cabi, observability as obs
    monkeypatch.setenv("FP8W8A16_SELFCHECK", "1")
    x, w, s, bh = make_dense(4, 512, 384, seed=11)
    before = _cabi.variant_counts()
    layer = types.SimpleNamespace(weight=w.cuda().view(torch.float8_e4m3fn), weight_scale_inv=s.cuda().to(torch.bfloat16),
                                  weight_block_size=[128, 128], input_size_per_partition=384, output_size_per_partition=512,
                                  prefix="model.layers.3.self_attn.o_proj")
    Fp8LinearMethod((128, 128)).process_weights_after_loading(layer)          # runs the probe, must not raise
    after = _cabi.variant_counts()
    assert sum(after.values()) > sum(before.values())
    assert after["tc_cluster"] + after["tc_streamk"] + after["tc_tiles"] > before["tc_cluster"] + before["tc_streamk"] + before["tc_tiles"]
    l2 = obs.selfcheck_linear(layer.weight, layer.weight_scale_inv, 512, 384, 128)
    assert l2 < 1e-2
    # the same bytes with a scale grid that belongs to another layout: the check must refuse
    bad = layer.weight_scale_inv.clone()
    bad[0, 0] *= 8
    ok_ref = obs.selfcheck_linear(layer.weight, bad, 512, 384, 128)           # consistent tensors still pass ...
    assert ok_ref < 1e-2
    xc, wc, sc, bhc = make_dense(4, 256, 256, seed=12, scheme="channel")
    lay2 = types.SimpleNamespace(weight=wc.cuda(), weight_scale=sc[:, :1].contiguous().cuda(), prefix="model.layers.3.mlp.down_proj")
    CompressedTensorsW8A16Fp8("CHANNEL").process_weights_after_loading(lay2)
    with pytest.raises(RuntimeError, match="self-check failed"):
        # ... but an engine whose result disagrees with the tensors' own dequantisation does not
        _selfcheck_against_wrong_reference(obs, lay2)


def _selfcheck_against_wrong_reference(obs, lay):
    """The engine's answer is made wrong on purpose (scales doubled on its side only)."""
    real = obs.ops.w8a16_linear
    try:
        obs.ops.w8a16_linear = lambda probe, w8, scale, N, K, bh, bw: real(probe, w8, scale * 2, N, K, bh, bw)
        obs.selfcheck_linear(lay.weight, lay.weight_scale, 256, 256, 1)
    finally:
        obs.ops.w8a16_linear = real


def test_compiled_hook_matches_eager(lib):
    """torch.compile (graph capture only, no codegen) of a function that calls the linear hook: one graph, same numbers."""
    from vllm_fp8_w8a16_sm70_b200 import Fp8LinearMethod
    x, w, s, bh = make_dense(6, 384, 256, seed=21)
    layer = types.SimpleNamespace(weight=w.cuda(), weight_scale_inv=s.cuda().to(torch.float16), weight_block_size=[128, 128],
                                  input_size_per_partition=256, output_size_per_partition=384)
    method = Fp8LinearMethod((128, 128))

    def fn(t):
        return method.apply(layer, t) + 1

    eager = fn(x.cuda())
    torch._dynamo.reset()
    try:
        compiled = torch.compile(fn, backend="aot_eager", fullgraph=True)
        got = compiled(x.cuda())
    finally:
        torch._dynamo.reset()
    assert torch.equal(eager, got)
