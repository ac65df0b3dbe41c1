"""The expert-parallel exchange kernels (dispatch -> experts -> return -> combine over peer memory) on ONE GPU: several
ranks' buffers live in one process and are attached to each other by pointer, and the three steps of a call are launched
rank by rank in phase order - all dispatches, then all expert steps, then all combines - so that no kernel ever waits for
a kernel queued behind it.  The protocol, the index arithmetic and the numerics are the multi-GPU ones; only the transport
(plain stores into a buffer that happens to be local) differs.  Checked against the CPU oracle of the single-GPU layer."""
import pytest
import torch

from oracle import moe as omoe
from tests.helpers import make_moe

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(lib):
    from vllm_fp8_w8a16_sm70_b200 import ops as _ops
    return _ops


def _ranks(ops, P, max_tokens, topk, H, E, timeout_ms=2000):
    eps = [ops.EpComm(r, P, max_tokens, topk, H, E, timeout_ms=timeout_ms) for r in range(P)]
    for r in range(P):
        for q in range(P):
            if q != r:
                eps[r].attach_ptr(q, eps[q].base)
    return eps


def _call(ops, eps, base, batches, m_max, skip_dispatch=()):
    """One collective call driven from one process: phase by phase over the ranks."""
    P, per = len(eps), base["w13"].shape[0] // len(eps)
    dev = [{k: v.cuda() for k, v in b.items() if k in ("x", "tw", "ids")} for b in batches]
    shard = [tuple(base[k][r * per:(r + 1) * per].contiguous().cuda() for k in ("w13", "s13", "w2", "s2")) for r in range(P)]
    outs = []
    for phase in ("dispatch", "experts", "combine"):
        for r in range(P):
            if phase == "dispatch" and r in skip_dispatch:
                continue
            o = ops.ep_moe_forward(eps[r], dev[r]["x"], dev[r]["tw"], dev[r]["ids"], *shard[r], block_h=base["bh"], m_max=m_max, phase=phase)
            if phase == "combine":
                outs.append(o)
    torch.cuda.synchronize()
    return [o.cpu() for o in outs]


@pytest.mark.parametrize("P,scheme,I", [(2, "block", 128), (4, "block", 256), (4, "channel", 176), (8, "block", 128)])
def test_phase_ordered_ranks_match_the_single_gpu_layer(ops, P, scheme, I):
    E, H, topk = 16, 256, 4
    base = make_moe(E, I, H, 1, topk, seed=5, scheme=scheme)
    eps = _ranks(ops, P, 16, topk, H, E)
    try:
        for call, tokens in enumerate(([5, 12, 0, 7, 1, 16, 3, 9][:P], [16] * P, [1] + [0] * (P - 1))):
            batches = [make_moe(E, I, H, max(m, 1), topk, seed=100 * call + r, scheme=scheme, invalid_frac=0.15) for r, m in enumerate(tokens)]
            for b, m in zip(batches, tokens):
                for k in ("x", "tw", "ids"):
                    b[k] = b[k][:m].contiguous()
            if call == 1:
                batches[0]["ids"] = batches[0]["ids"].to(torch.int64)
            outs = _call(ops, eps, base, batches, max(tokens))
            for r, (b, m) in enumerate(zip(batches, tokens)):
                assert tuple(outs[r].shape) == (m, H)
                if m == 0:
                    continue
                ref = omoe.moe_reference_fp32(b["x"], b["tw"], b["ids"], base["w13"], base["s13"], base["w2"], base["s2"], base["bh"])
                omoe.check_moe(outs[r], ref)
                dropped = (b["ids"] < 0).all(dim=1)
                assert bool((outs[r][dropped] == 0).all()), "a token whose routes were all dropped must come out as exact zeros"
                # and the same answer as the single-GPU entry point on the full expert stack
                one = ops.moe_forward(b["x"].cuda(), b["tw"].cuda(), b["ids"].cuda(), base["w13"].cuda(), base["s13"].cuda(), base["w2"].cuda(),
                                      base["s2"].cuda(), block_h=base["bh"]).cpu()
                assert torch.allclose(outs[r].float(), one.float(), atol=2e-3, rtol=2e-2)
        assert ops.device_status() == 0
    finally:
        for e in eps:
            e.close()


def test_batches_on_both_sides_of_the_single_cta_limit(ops):
    """Up to 16 routed rows one CTA builds the route table AND moves the rows (dispatch: stores into the peers' inboxes;
    expert step: the gather of a small inbox); above that the table kernel is followed by one warp per row.  Ranks of one
    call sit on both sides of the limit, and one call keeps every inbox small enough for the fused gather."""
    E, H, topk, I, P = 16, 256, 4, 128, 4
    base = make_moe(E, I, H, 1, topk, seed=9)
    eps = _ranks(ops, P, 40, topk, H, E)
    try:
        for call, tokens in enumerate(([40, 16, 17, 3], [4, 2, 0, 1], [33, 33, 33, 33])):
            batches = [make_moe(E, I, H, max(m, 1), topk, seed=300 + 10 * call + r, invalid_frac=0.1) for r, m in enumerate(tokens)]
            for b, m in zip(batches, tokens):
                for k in ("x", "tw", "ids"):
                    b[k] = b[k][:m].contiguous()
            outs = _call(ops, eps, base, batches, max(tokens))
            for r, (b, m) in enumerate(zip(batches, tokens)):
                assert tuple(outs[r].shape) == (m, H)
                if m:
                    omoe.check_moe(outs[r], omoe.moe_reference_fp32(b["x"], b["tw"], b["ids"], base["w13"], base["s13"], base["w2"],
                                                                    base["s2"], base["bh"]))
        assert ops.device_status() == 0
    finally:
        for e in eps:
            e.close()


def test_benchmark_shape_top8_of_128_experts(ops):
    """The MoE decode layer of the benchmark (128 experts, top-8, hidden 2048, intermediate 768) split over 8 ranks,
    8 tokens per rank."""
    E, I, H, topk, P, M = 128, 768, 2048, 8, 8, 8
    base = make_moe(E, I, H, 1, topk, seed=1)
    eps = _ranks(ops, P, M, topk, H, E)
    try:
        batches = [make_moe(E, I, H, M, topk, seed=50 + r) for r in range(P)]
        for b in batches:          # route with the device router, as the benchmark does
            b["tw"], b["ids"] = (t.cpu() for t in ops.moe_topk_softmax(b["logits"].cuda(), topk, True))
        outs = _call(ops, eps, base, batches, M)
        for r in (0, 3, 7):
            b = batches[r]
            omoe.check_moe(outs[r], omoe.moe_reference_fp32(b["x"], b["tw"], b["ids"], base["w13"], base["s13"], base["w2"], base["s2"]))
        assert ops.device_status() == 0
    finally:
        for e in eps:
            e.close()


def test_a_missing_rank_runs_the_waits_out_and_reset_recovers(ops):
    """Rank 1 never dispatches: the owners' wait for its header and its own... everybody's wait for what cannot come ends
    at the 50 ms limit, the status word says which wait gave up (256: header, 512: return flag), nothing hangs and the
    context stays usable; after a reset of every rank the next call is correct again."""
    E, I, H, topk, P = 8, 128, 256, 2, 2
    base = make_moe(E, I, H, 1, topk, seed=9)
    eps = _ranks(ops, P, 8, topk, H, E, timeout_ms=50)
    try:
        batches = [make_moe(E, I, H, 4, topk, seed=20 + r) for r in range(P)]
        outs = _call(ops, eps, base, batches, 4, skip_dispatch=(1,))
        st = ops.device_status(reset=True)
        assert st & 256, f"status {st:#x}: the wait for the missing header should have run out"
        assert all(torch.isfinite(o).all() for o in outs)
        # rank 0's own rows that went to rank 0's experts are still right where its routes stayed local; nothing is checked
        # beyond finiteness: the call is void.  Recover: every rank resets, then a complete call.
        torch.cuda.synchronize()
        for e in eps:
            e.reset()
        ops.reset_workspaces()
        outs = _call(ops, eps, base, batches, 4)
        for r, b in enumerate(batches):
            omoe.check_moe(outs[r], omoe.moe_reference_fp32(b["x"], b["tw"], b["ids"], base["w13"], base["s13"], base["w2"], base["s2"]))
        assert ops.device_status() == 0
    finally:
        for e in eps:
            e.close()


def test_argument_checks(ops):
    eps = _ranks(ops, 2, 4, 2, 256, 8)
    try:
        d = make_moe(8, 128, 256, 6, 2, seed=1)
        w = [d[k][:4].contiguous().cuda() for k in ("w13", "s13", "w2", "s2")]
        with pytest.raises(RuntimeError, match="m_max"):
            ops.ep_moe_forward(eps[0], d["x"].cuda(), d["tw"].cuda(), d["ids"].cuda(), *w)              # 6 tokens, buffer built for 4
        with pytest.raises(RuntimeError, match="do not match"):
            ops.ep_moe_forward(eps[0], d["x"][:2].cuda(), d["tw"][:2].cuda(), d["ids"][:2].cuda(), d["w13"].cuda(), d["s13"].cuda(),
                               d["w2"].cuda(), d["s2"].cuda())                                        # all 8 experts on one of 2 ranks
        assert eps[0].nbytes > 0 and eps[0].base != 0
    finally:
        for e in eps:
            e.close()
