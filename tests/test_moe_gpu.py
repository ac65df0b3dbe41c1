"""GPU parity of the MoE path through the C ABI: routing indices and route tables bit-exact, layer output
within the reference numtests' bar (cos > 0.9999, relative L2 < 2e-2 against the fp32 reference)."""
import numpy as np
import pytest
import torch

from oracle import moe as omoe
from tests.helpers import f16_from_bits, make_moe

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(lib):
    from vllm_fp8_w8a16_sm70_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("M,E,k", [(1, 128, 8), (7, 128, 8), (256, 128, 8), (33, 8, 2), (5, 160, 6), (3, 1024, 40), (4, 4, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("renorm", [True, False])
def test_topk_softmax_indices_bit_exact(ops, M, E, k, dtype, renorm):
    g = torch.Generator().manual_seed(M * 7 + E)
    logits = torch.randn(M, E, generator=g).to(dtype)
    if M > 2:
        logits[1, : E // 2] = logits[1, 0]      # ties -> lowest expert index first
    ids_o, w_o = omoe.route_topk(logits, k, renorm)
    w_g, ids_g = ops.moe_topk_softmax(logits.cuda(), k, renorm)
    assert torch.equal(ids_g.cpu(), ids_o)
    assert torch.allclose(w_g.cpu(), w_o, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("R,E,bt", [(8, 128, 16), (2048, 128, 32), (0, 8, 16), (1, 1, 16), (777, 5, 64), (16384, 128, 128), (40000, 16, 128)])
def test_align_matches_oracle(ops, R, E, bt):
    g = torch.Generator().manual_seed(R + E)
    ids = torch.randint(-1, E + 2, (R,), generator=g, dtype=torch.int64) if R else torch.zeros(0, dtype=torch.int64)
    counts_o, offsets_o, order_o = omoe.align_routes(ids, E)
    for t in (ids, ids.to(torch.int32)):
        counts, offsets, tile_offsets, sorted_route, inv_pos = ops.moe_align(t.cuda(), E, bt)
        assert torch.equal(counts.cpu(), counts_o) and torch.equal(offsets.cpu(), offsets_o)
        nv = int(offsets_o[-1])
        assert torch.equal(sorted_route.cpu()[:nv], order_o) and (sorted_route.cpu()[nv:] == -1).all()
        tiles = torch.zeros(E + 1, dtype=torch.int32)
        tiles[1:] = torch.cumsum((counts_o + bt - 1) // bt, 0)
        assert torch.equal(tile_offsets.cpu(), tiles)
        inv = torch.full((R,), -1, dtype=torch.int32)
        inv[order_o.long()] = torch.arange(nv, dtype=torch.int32)
        assert torch.equal(inv_pos.cpu(), inv)


def test_align_with_expert_map(ops):
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 128, (64, 8), generator=g, dtype=torch.int32)
    ids[0, 0] = -1
    from oracle.tp import expert_partition
    for rank in range(4):
        _, _, emap = expert_partition(128, 4, rank)
        local = omoe.remap_expert_ids(ids, emap).reshape(-1)
        counts_o, offsets_o, order_o = omoe.align_routes(local, 32)
        counts, offsets, _, sorted_route, _ = ops.moe_align(ids.cuda(), 32, 16, expert_map=emap.cuda())
        assert torch.equal(counts.cpu(), counts_o) and torch.equal(sorted_route.cpu()[: int(offsets_o[-1])], order_o)


def layer(ops, d, **kw):
    return ops.moe_forward(d["x"].cuda(), d["tw"].cuda(), d["ids"].cuda(), d["w13"].cuda(), d["s13"].cuda(), d["w2"].cuda(),
                           d["s2"].cuda(), block_h=d["bh"], **kw).cpu()


def reference(d, ids=None):
    return omoe.moe_reference_fp32(d["x"], d["tw"], d["ids"] if ids is None else ids, d["w13"], d["s13"], d["w2"], d["s2"], d["bh"])


@pytest.mark.parametrize("E,I,H,M,topk", [(8, 256, 512, 1, 2), (8, 256, 512, 4, 2), (8, 256, 512, 33, 4), (16, 128, 256, 100, 4),
                                           (4, 384, 1024, 300, 2), (128, 768, 2048, 2, 8),
                                           (8, 256, 512, 4, 4), (8, 256, 512, 17, 1)])   # 16 and 17 routed rows: the two sides of the single-CTA gather limit
def test_layer_block_scaled(ops, E, I, H, M, topk):
    d = make_moe(E, I, H, M, topk, seed=M)
    y = layer(ops, d)
    omoe.check_moe(y, reference(d))
    omoe.check_moe(y, omoe.moe_reference_fp16_chain(d["x"], d["tw"], d["ids"], d["w13"], d["s13"], d["w2"], d["s2"], d["bh"]))


@pytest.mark.parametrize("E,I,H,M,topk", [(8, 176, 512, 1, 2), (8, 176, 512, 4, 2), (8, 176, 512, 16, 4), (16, 176, 512, 8, 2),
                                           (8, 176, 512, 100, 4)])
def test_layer_channel_scaled_I176(ops, E, I, H, M, topk):
    # shapes of tools/ct_fp8_mixed_moe_numtest_vllm021.sh:96-102 (2I = 352 partial-N, K = 176 for w2) at a smaller H
    d = make_moe(E, I, H, M, topk, seed=E + M, scheme="channel")
    omoe.check_moe(layer(ops, d), reference(d))


def test_invalid_routes_contribute_exactly_zero(ops):
    # reference: invalid expert id => zero row (tools/ct_fp8_grouped_coalesced_numtest_vllm021.sh:38,55-56)
    d = make_moe(8, 128, 256, 12, 2, seed=3, invalid_frac=0.4)
    d["ids"][5] = -1
    y = layer(ops, d)
    assert (y[5] == 0).all()
    omoe.check_moe(y, reference(d))
    d["ids"][:] = -1
    assert (layer(ops, d) == 0).all()


def test_expert_map_ranks_sum_to_the_full_layer(ops):
    """Expert-parallel semantics of the reference (vllm_serve.py:2237-2243): each rank computes its local
    experts, non-local routes are zero, the caller's reduce adds the ranks."""
    from oracle.tp import expert_partition
    d = make_moe(16, 128, 256, 20, 4, seed=8)
    total = torch.zeros(20, 256)
    for rank in range(4):
        lo, hi, emap = expert_partition(16, 4, rank)
        dd = dict(d, w13=d["w13"][lo:hi].contiguous(), s13=d["s13"][lo:hi].contiguous(), w2=d["w2"][lo:hi].contiguous(),
                  s2=d["s2"][lo:hi].contiguous())
        total += layer(ops, dd, expert_map=emap.cuda()).float()
    omoe.check_moe(total, reference(d))


def test_weight_on_input_and_int64_ids(ops):
    d = make_moe(8, 128, 256, 9, 1, seed=5)
    d["ids"] = d["ids"].to(torch.int64)
    y = layer(ops, d, weight_on_input=True)
    x_scaled = dict(d, x=(d["x"].float() * d["tw"]).to(torch.float16), tw=torch.ones_like(d["tw"]))
    omoe.check_moe(y, reference(x_scaled))


def test_golden_reference_loop_fixture(ops, golden_dir):
    z = np.load(golden_dir / "moe_reference.npz")
    E, I, H, M, topk = z["dims"].tolist()
    s13 = f16_from_bits(z["s13"]).expand(E, 2 * I, -(-H // 128)).contiguous()
    s2 = torch.from_numpy(z["s2"]).to(torch.float16).expand(E, H, -(-I // 128)).contiguous()
    y = ops.moe_forward(f16_from_bits(z["x"]).cuda(), f16_from_bits(z["topk_w"]).float().cuda(), torch.from_numpy(z["topk_ids"]).cuda(),
                        torch.from_numpy(z["w13"]).cuda(), s13.cuda(), torch.from_numpy(z["w2"]).cuda(), s2.cuda(), block_h=1)
    omoe.check_moe(y.cpu(), torch.from_numpy(z["out_f32"]))


def test_pieces_gather_grouped_combine(ops):
    d = make_moe(8, 256, 512, 10, 2, seed=1)
    E, I, H, M, topk = 8, 256, 512, 10, 2
    bt = ops.moe_token_tile(M * topk, E)
    counts, offsets, tile_offsets, sorted_route, inv_pos = ops.moe_align(d["ids"].cuda(), E, bt)
    xs, wsorted = ops.moe_gather(d["x"].cuda(), sorted_route, d["tw"].cuda(), topk)
    sr = sorted_route.cpu().long()
    assert torch.equal(xs.cpu(), d["x"][sr // topk]) and torch.equal(wsorted.cpu(), d["tw"].reshape(-1)[sr])
    h = ops.moe_grouped_gemm(xs, d["w13"].cuda(), d["s13"].cuda(), offsets, tile_offsets, I, H, 128, bt, paired=True)
    y = ops.moe_grouped_gemm(h, d["w2"].cuda(), d["s2"].cuda(), offsets, tile_offsets, H, I, 128, bt, row_weight=wsorted)
    out = ops.moe_combine(y, inv_pos, M, topk)
    assert torch.equal(out.view(torch.int16), layer(ops, d).cuda().view(torch.int16))
    want = torch.zeros(M, H)
    want.index_add_(0, sr // topk, y.cpu().float())
    assert torch.allclose(out.cpu().float(), want, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("M,E,H,topk,dtype", [(1, 128, 2048, 8, torch.float16), (7, 128, 2048, 8, torch.bfloat16), (64, 60, 512, 4, torch.float32),
                                              (3, 8, 64, 8, torch.float16), (33, 256, 1024, 6, torch.bfloat16),
                                              (1003, 128, 1024, 8, torch.float16), (37, 24, 256, 2, torch.bfloat16)])   # past the cluster kernel's batch limit; few experts
def test_router_gemv_topk_fused(ops, M, E, H, topk, dtype):
    """Gate GEMV + selection in one kernel.  The logits must match an fp32 matmul of the same tensors; given the
    kernel's own logits the picks must be EXACTLY the oracle's (indices bit-exact, ties to the lowest index)."""
    g = torch.Generator().manual_seed(M * 1000 + E)
    x = torch.randn(M, H, generator=g).to(torch.float16)
    gw = (torch.randn(E, H, generator=g) / H ** 0.5).to(dtype)
    if M >= 3:
        gw[5] = gw[2]                       # two experts with identical logits: the lower index must win
    w, ids, logits = ops.moe_router_topk(x.cuda(), gw.cuda(), topk, True, return_logits=True)
    ref_logits = x.float() @ gw.float().T
    assert torch.allclose(logits.cpu(), ref_logits, atol=2e-4, rtol=1e-4)
    ids_o, w_o = omoe.route_topk(logits.cpu(), topk, True)
    assert torch.equal(ids.cpu(), ids_o), "routing indices must be bit-exact given the logits"
    assert torch.allclose(w.cpu(), w_o, atol=1e-6, rtol=1e-5)
    # same picks as the two-step path (logits -> moe_topk_softmax)
    w2, ids2 = ops.moe_topk_softmax(logits, topk, True)
    assert torch.equal(ids2, ids) and torch.equal(w2, w)
    # fixed shared-expert route and routed scaling
    ws, idss = ops.moe_router_topk(x.cuda(), gw.cuda(), topk, True, shared_expert_id=E, routed_scale=2.5)
    assert tuple(idss.shape) == (M, topk + 1) and torch.equal(idss[:, :topk], ids) and bool((idss[:, topk] == E).all())
    assert torch.allclose(ws[:, :topk], w * 2.5, rtol=1e-6) and bool((ws[:, topk] == 1.0).all())


@pytest.mark.parametrize("M", [1, 5, 40])
def test_moe_block_with_shared_expert(ops, M):
    """router -> experts -> routed + shared in one pipeline vs the oracle: routed reference + a dense shared MLP."""
    from vllm_fp8_w8a16_sm70_b200.moe_block import MoEBlock
    E, I, H, topk = 16, 256, 512, 4
    d = make_moe(E + 1, I, H, M, topk, seed=77)             # expert E plays the shared expert
    g = torch.Generator().manual_seed(5)
    gate = (torch.randn(E, H, generator=g) / H ** 0.5).to(torch.float16)
    blk = MoEBlock(gate.cuda(), d["w13"][:E].cuda(), d["s13"][:E].cuda(), d["w2"][:E].cuda(), d["s2"][:E].cuda(), topk,
                   shared=(d["w13"][E].cuda(), d["s13"][E].cuda(), d["w2"][E].cuda(), d["s2"][E].cuda()), routed_scaling_factor=1.5)
    x = d["x"]
    out = blk(x.cuda())
    tw, ids = blk.route(x.cuda())
    ids_c, tw_c = ids.cpu(), tw.cpu()
    assert bool((ids_c[:, topk] == E).all())
    ref = omoe.moe_reference_fp32(x, tw_c, ids_c, d["w13"], d["s13"], d["w2"], d["s2"])      # E + 1 experts, fixed route included
    omoe.check_moe(out.cpu(), ref)
    # the shared part alone equals a dense MLP on every token
    routed_only = omoe.moe_reference_fp32(x, tw_c[:, :topk], ids_c[:, :topk], d["w13"], d["s13"], d["w2"], d["s2"])
    shared_only = omoe.moe_reference_fp32(x, torch.ones(M, 1), torch.full((M, 1), E), d["w13"], d["s13"], d["w2"], d["s2"])
    assert torch.allclose(ref, routed_only + shared_only, atol=1e-4, rtol=1e-4)
    with pytest.raises(ValueError):
        MoEBlock(gate.cuda(), d["w13"][:E].cuda(), d["s13"][:E].cuda(), d["w2"][:E].cuda(), d["s2"][:E].cuda(), topk,
                 shared=(d["w13"][E][:256].cuda(), d["s13"][E].cuda(), d["w2"][E].cuda(), d["s2"][E].cuda()))
