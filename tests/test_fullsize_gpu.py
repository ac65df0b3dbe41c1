"""GPU parity at the sizes the benchmark configurations name, against the CPU oracle: the MoE decode layer of 128 experts
(top-8, hidden 2048, intermediate 768) at 8 / 64 / 256 tokens, the channel-scale mix (hidden 4096, intermediate 176 per rank,
128 routed experts + 1 shared through the router block) at 1 / 64 / 2048 tokens, a dense prefill batch of 8192 tokens, and
the compressed-tensors MoE hook.  Weights are generated on the device from seeded generators (a CPU generator would take
minutes at these sizes) and copied back for the oracle, which dequantises only the experts that are hit."""
import types

import pytest
import torch

from oracle import linear as olin, moe as omoe

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(lib):
    from vllm_fp8_w8a16_sm70_b200 import ops as _ops
    return _ops


def _block_fp8(rows, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(rows, K, generator=g, device="cuda") * 0.02
    blocks = w.reshape(rows // 128, 128, K // 128, 128)
    s = blocks.abs().amax(dim=(1, 3)) / 448.0
    q = (blocks / s[:, None, :, None]).reshape(rows, K).to(torch.float8_e4m3fn).view(torch.uint8)
    return q.contiguous(), s.to(torch.float16).contiguous()


def _channel_fp8(rows, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(rows, K, generator=g, device="cuda") * 0.02
    s = w.abs().amax(dim=1, keepdim=True) / 448.0
    q = (w / s).to(torch.float8_e4m3fn).view(torch.uint8)
    return q.contiguous(), s.to(torch.float16).expand(rows, -(-K // 128)).contiguous()


@pytest.fixture(scope="module")
def c4_experts():
    """BASELINE config 4: gate_up [128, 1536, 2048], down [128, 2048, 768], block-128 scales."""
    E, I, H = 128, 768, 2048
    w13 = torch.empty(E, 2 * I, H, dtype=torch.uint8, device="cuda")
    w2 = torch.empty(E, H, I, dtype=torch.uint8, device="cuda")
    s13 = torch.empty(E, 2 * I // 128, H // 128, dtype=torch.float16, device="cuda")
    s2 = torch.empty(E, H // 128, I // 128, dtype=torch.float16, device="cuda")
    for e in range(E):
        w13[e], s13[e] = _block_fp8(2 * I, H, 2 * e)
        w2[e], s2[e] = _block_fp8(H, I, 2 * e + 1)
    return dict(w13=w13, s13=s13, w2=w2, s2=s2, cpu=dict(w13=w13.cpu(), s13=s13.cpu(), w2=w2.cpu(), s2=s2.cpu()))


@pytest.mark.parametrize("M", [8, 64, 256])
def test_c4_moe_decode_layer_full_size(ops, c4_experts, M):
    d = c4_experts
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, 2048, generator=g).to(torch.float16)
    logits = torch.randn(M, 128, generator=g)
    tw, ids = ops.moe_topk_softmax(logits.cuda(), 8, True)
    ids_o, tw_o = omoe.route_topk(logits, 8, True)
    assert torch.equal(ids.cpu(), ids_o)
    y = ops.moe_forward(x.cuda(), tw, ids, d["w13"], d["s13"], d["w2"], d["s2"], block_h=128)
    c = d["cpu"]
    omoe.check_moe(y.cpu(), omoe.moe_reference_fp32(x, tw_o, ids_o, c["w13"], c["s13"], c["w2"], c["s2"], 128))


@pytest.fixture(scope="module")
def c5_block():
    """BASELINE config 5 at one rank of TP = 8: hidden 4096, intermediate 1408 / 8 = 176, per-output-channel scales,
    128 routed experts + 1 shared expert (stored as expert 128), router gate [128, 4096]."""
    from vllm_fp8_w8a16_sm70_b200.moe_block import MoEBlock
    E, I, H = 128, 176, 4096
    w13 = torch.empty(E + 1, 2 * I, H, dtype=torch.uint8, device="cuda")
    w2 = torch.empty(E + 1, H, I, dtype=torch.uint8, device="cuda")
    s13 = torch.empty(E + 1, 2 * I, H // 128, dtype=torch.float16, device="cuda")
    s2 = torch.empty(E + 1, H, 2, dtype=torch.float16, device="cuda")
    for e in range(E + 1):
        w13[e], s13[e] = _channel_fp8(2 * I, H, 500 + 2 * e)
        w2[e], s2[e] = _channel_fp8(H, I, 501 + 2 * e)
    gate = (torch.randn(E, H, generator=torch.Generator(device="cuda").manual_seed(9), device="cuda") / H ** 0.5).to(torch.float16)
    blk = MoEBlock(gate, w13[:E], s13[:E], w2[:E], s2[:E], 8, block_h=1, shared=(w13[E], s13[E], w2[E], s2[E]))
    return blk, dict(w13=w13.cpu(), s13=s13.cpu(), w2=w2.cpu(), s2=s2.cpu())


@pytest.mark.parametrize("M", [1, 64, 2048])
def test_c5_channel_scale_moe_block_full_size(ops, c5_block, M):
    """Router + 128 routed (top-8) + shared expert, K = 176 down projection, 2I = 352 partial-N gate/up
    (kernel shapes of tools/ct_fp8_mixed_moe_numtest_vllm021.sh:95-100 at the model's real expert count)."""
    blk, c = c5_block
    x = (torch.randn(M, 4096, generator=torch.Generator().manual_seed(40 + M)) * 0.5).to(torch.float16)
    out = blk(x.cuda())
    tw, ids = blk.route(x.cuda())
    assert bool((ids[:, 8] == 128).all()) and int(ids.min()) >= 0 and int(ids[:, :8].max()) < 128
    ref = omoe.moe_reference_fp32(x, tw.cpu(), ids.cpu(), c["w13"], c["s13"], c["w2"], c["s2"], 1)
    omoe.check_moe(out.cpu(), ref)


def test_dense_prefill_batch_of_8192_tokens(ops):
    """qkv [7168, 5120] at M = 8192 (the largest prefill batch of the benchmark): the whole output against the bit-exact
    dequant kernel + an fp32 matmul on the device (that kernel is pinned bit for bit against the oracle in
    test_dequant_gpu.py), and a 256-feature slab against the CPU oracle itself, fp32 accumulation."""
    N, K, M = 7168, 5120, 8192
    q, s = _block_fp8(N, K, 123)
    x = torch.randn(M, K, generator=torch.Generator(device="cuda").manual_seed(5), device="cuda").to(torch.float16)
    y = ops.w8a16_linear(x, q, s, N, K)
    wdq = ops.fp8_e4m3_to_fp16_block_scaled(q, s, N, K)
    ref = torch.cat([x.float() @ wdq[n0:n0 + 1024].float().T for n0 in range(0, N, 1024)], 1)
    olin.check_linear(y.cpu(), x.cpu(), ref.cpu(), K)
    n0 = 3 * 1024 + 128                                   # a slab that starts inside the matrix, on a scale-block boundary
    slab = olin.oracle_linear_fp32(x.cpu(), q[n0:n0 + 256].cpu(), s[n0 // 128:n0 // 128 + 2].cpu(), 128)
    olin.check_linear(y[:, n0:n0 + 256].cpu(), x.cpu(), slab, K)


@pytest.mark.parametrize("layout", ["channel", "tensor", "block"])
def test_compressed_tensors_moe_hook(ops, layout):
    """CompressedTensorsFp8MoEMethod.process_weights_after_loading + .apply (the hooks the reference assigns onto
    CompressedTensorsW8A8Fp8MoEMethod, compressed_tensors_v100.py:1226-1229) with the scale layouts a checkpoint
    brings - [E, rows, 1], [E] or a block grid - against the oracle on the equivalent row / block grid."""
    from tests.helpers import make_moe
    from vllm_fp8_w8a16_sm70_b200.moe_method import CompressedTensorsFp8MoEMethod
    E, I, H, M, topk = 8, 176 if layout != "block" else 256, 512, 19, 2
    d = make_moe(E, I, H, M, topk, seed=61, scheme="block" if layout == "block" else "channel")
    if layout == "channel":
        s13_ckpt, s2_ckpt = d["s13"][:, :, :1].float(), d["s2"][:, :, :1].float()           # [E, rows, 1]
        s13_ref, s2_ref, bh = d["s13"], d["s2"], 1
    elif layout == "tensor":
        s13_ckpt, s2_ckpt = d["s13"][:, 0, 0].float(), d["s2"][:, 0, 0].float()             # one scale per expert: [E]
        s13_ref = s13_ckpt.to(torch.float16).reshape(E, 1, 1).expand(E, 2 * I, -(-H // 128)).contiguous()
        s2_ref = s2_ckpt.to(torch.float16).reshape(E, 1, 1).expand(E, H, -(-I // 128)).contiguous()
        bh = 1
    else:
        s13_ckpt, s2_ckpt, s13_ref, s2_ref, bh = d["s13"].float(), d["s2"].float(), d["s13"], d["s2"], 128
    layer = types.SimpleNamespace(w13_weight=d["w13"].cuda().view(torch.float8_e4m3fn), w2_weight=d["w2"].cuda().view(torch.float8_e4m3fn),
                                  w13_weight_scale=s13_ckpt.cuda(), w2_weight_scale=s2_ckpt.cuda(), activation="silu")
    m = CompressedTensorsFp8MoEMethod(types.SimpleNamespace(strategy=types.SimpleNamespace(name=layout.upper())))
    m.process_weights_after_loading(layer)
    m.process_weights_after_loading(layer)                 # idempotent, as vLLM may call it twice
    assert layer.w13_weight_scale.dtype == torch.float16 and m.get_fused_moe_quant_config(layer) is None
    xb = d["x"].to(torch.bfloat16)
    y = m.apply(layer, xb.cuda(), d["tw"].cuda(), d["ids"].to(torch.int64).cuda(), None)     # 5-argument form, bf16 in -> bf16 out
    assert y.dtype == torch.bfloat16
    ref = omoe.moe_reference_fp32(xb.to(torch.float16), d["tw"], d["ids"], d["w13"], s13_ref, d["w2"], s2_ref, bh)
    omoe.check_moe(y.float().cpu(), ref)


def test_workspace_growth_does_not_invalidate_a_captured_graph(ops):
    """A graph captured while the stream's workspace was small must stay valid after a later, larger call made the
    workspace grow: the outgrown buffer is retired, never freed, so the replay still writes its partial tiles and
    counters into memory nobody else owns."""
    from tests.helpers import make_dense, make_moe
    x, w, s, bh = make_dense(4, 5120, 5120, seed=11)          # cluster split-K + stream-K shapes use the workspace
    xd, wd, sd = x.cuda(), w.cuda(), s.cuda()
    side = torch.cuda.Stream()
    out = torch.empty(4, 5120, dtype=torch.float16, device="cuda")
    x2, w2, s2, _ = make_dense(4, 51200 // 8, 5120, seed=12)
    x2d, w2d, s2d = x2.cuda(), w2.cuda(), s2.cuda()
    out2 = torch.empty(4, 51200 // 8, dtype=torch.float16, device="cuda")
    with torch.cuda.stream(side):
        for _ in range(2):
            ops.w8a16_linear(xd, wd, sd, 5120, 5120, out=out)
            ops.w8a16_linear(x2d, w2d, s2d, 6400, 5120, out=out2)
        side.synchronize()
        before = ops._WORKSPACES[(torch.cuda.current_device(), side.cuda_stream)]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            ops.w8a16_linear(xd, wd, sd, 5120, 5120, out=out)
            ops.w8a16_linear(x2d, w2d, s2d, 6400, 5120, out=out2)
        # a MoE batch whose scratch need exceeds the dense floor: the workspace of this stream must grow
        d = make_moe(4, 256, 2048, 1, 2, seed=3)
        M = 6144
        xm = torch.randn(M, 2048, generator=torch.Generator(device="cuda").manual_seed(1), device="cuda").to(torch.float16)
        ids = torch.randint(0, 4, (M, 2), generator=torch.Generator(device="cuda").manual_seed(2), device="cuda", dtype=torch.int32)
        tw = torch.full((M, 2), 0.5, device="cuda")
        ew = [d[k].cuda() for k in ("w13", "s13", "w2", "s2")]
        big = (torch.cat([xm, xm]), torch.cat([tw, tw]), torch.cat([ids, ids]))
        ops.moe_forward(xm, tw, ids, *ew)
        after = ops._WORKSPACES[(torch.cuda.current_device(), side.cuda_stream)]
        assert after.data_ptr() != before.data_ptr() and after.numel() > before.numel(), "the MoE call was meant to outgrow the workspace"
        assert any(r.data_ptr() == before.data_ptr() for r in ops._RETIRED)
        filler = [torch.full((before.numel(),), 0xFF, dtype=torch.uint8, device="cuda") for _ in range(3)]   # would land on a freed buffer
        out.zero_()
        out2.zero_()
        g.replay()
        side.synchronize()
        # growing a workspace during capture is refused, loudly
        g2 = torch.cuda.CUDAGraph()
        with pytest.raises(RuntimeError, match="being captured"):
            with torch.cuda.graph(g2, stream=side):
                ops.moe_forward(*big, *ew)
    del filler
    olin.check_linear(out.cpu(), x, olin.oracle_linear_fp32(x, w, s, bh), 5120)
    olin.check_linear(out2.cpu(), x2, olin.oracle_linear_fp32(x2, w2, s2, bh), 5120)


def test_align_raises_its_shared_memory_limit_per_call_size(ops):
    """64 experts, then 512, then 1024: the route-table kernel needs more than the default 48 KiB of dynamic shared
    memory from ~370 experts on, and a limit set for one size must not be taken for good."""
    for E in (64, 512, 1024, 400):
        for dt in (torch.int32, torch.int64):
            ids = torch.randint(-1, E, (3000,), generator=torch.Generator().manual_seed(E), dtype=dt)
            counts_o, offsets_o, order_o = omoe.align_routes(ids, E)
            counts, offsets, _, sorted_route, _ = ops.moe_align(ids.cuda(), E, 16)
            assert torch.equal(counts.cpu(), counts_o) and torch.equal(offsets.cpu(), offsets_o)
            assert torch.equal(sorted_route.cpu()[: int(offsets_o[-1])], order_o)
