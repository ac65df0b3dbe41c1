"""Host-side logic of the multi-GPU paths on CPU: world_size-2 gloo ranks, with the GEMM and the local
expert computation supplied by the oracle (the CUDA engine cannot run here; what is under test is the
sharding, the all-reduce placement and the all-to-all dispatch / combine index arithmetic)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import linear as olin, moe as omoe
from tests.helpers import make_dense, make_moe


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vllm_fp8_w8a16_sm70_b200 import parallel as par
    x, w1, s1, bh = make_dense(5, 512, 256, seed=1)
    _, w2, s2, _ = make_dense(5, 256, 512, seed=2)
    bias = torch.arange(256, dtype=torch.float32) * 1e-3
    # column-parallel up-projection then row-parallel down-projection, as a decoder MLP
    wc, sc = par.shard_column_parallel(w1, s1, world, rank)
    wr, sr = par.shard_row_parallel(w2, s2, world, rank)
    col = par.TensorParallelLinear(wc, sc, bh, "column", linear_fn=lambda t: olin.oracle_linear_fp32(t, wc, sc, bh).to(torch.float16))
    row = par.TensorParallelLinear(wr, sr, bh, "row", linear_fn=lambda t: olin.oracle_linear_fp32(t, wr, sr, bh).to(torch.float32))
    h = col.forward(x)
    y = row.forward(h, bias)
    h_full = olin.oracle_linear_fp32(x, w1, s1, bh).to(torch.float16)
    y_full = olin.oracle_linear_fp32(h_full, w2, s2, bh) + bias
    ok = torch.allclose(h, h_full[:, rank * 256:(rank + 1) * 256]) and torch.allclose(y, y_full, atol=1e-3, rtol=1e-3)
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


def _ep_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vllm_fp8_w8a16_sm70_b200 import parallel as par
    E, I, H, topk = 8, 128, 256, 2
    d = make_moe(E, I, H, 6 + rank, topk, seed=10 + rank, invalid_frac=0.2)   # each rank brings its own tokens
    base = make_moe(E, I, H, 1, topk, seed=99)                                # weights shared by all ranks
    per = E // world
    lo, hi = rank * per, (rank + 1) * per
    w13, s13, w2, s2 = base["w13"], base["s13"], base["w2"], base["s2"]

    def expert_fn(rows, local_ids):
        ones = torch.ones(rows.shape[0], 1)
        return omoe.moe_reference_fp32(rows, ones, local_ids.reshape(-1, 1), w13[lo:hi], s13[lo:hi], w2[lo:hi], s2[lo:hi]).to(torch.float16)

    layer = par.ExpertParallelMoE(w13[lo:hi], s13[lo:hi], w2[lo:hi], s2[lo:hi], E, expert_fn=expert_fn)
    y = layer.forward(d["x"], d["tw"], d["ids"])
    ref = omoe.moe_reference_fp32(d["x"], d["tw"], d["ids"], w13, s13, w2, s2)
    st = omoe.moe_error_stats(y, ref)
    q.put((rank, st["cos"] > 0.9999 and st["l2rel"] < 2e-2))
    dist.destroy_process_group()


def _comm_failure_worker(rank, world, port, q):
    """Without a GPU no rank can create its communicator buffer: every rank must raise (none may hang in a
    collective waiting for the others), and a row-parallel layer without a communicator keeps the NCCL/gloo path."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vllm_fp8_w8a16_sm70_b200 import parallel as par
    try:
        par.make_peer_comm(max_out_elems=1024, timeout_ms=50)
        ok = False
    except RuntimeError as exc:
        ok = "could not be set up" in str(exc)
    q.put((rank, ok))
    dist.destroy_process_group()


def _hook_path_worker(rank, world, port, q):
    """The vLLM-facing hook with a communicator attached must (a) pick its path from rank-invariant facts - the bias
    ARGUMENT arrives on rank 0 only - and (b) return the reduced result on the plain path too.  The GEMM is the oracle's
    (the engine cannot run on CPU); a fused call would raise here, which is exactly what shows that both ranks avoided it."""
    import types
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vllm_fp8_w8a16_sm70_b200 import linear_method as lm, parallel as par
    x, w, s, bh = make_dense(5, 256, 512, seed=3)
    wr, sr = par.shard_row_parallel(w, s.to(torch.float16), world, rank)
    xs = x[:, rank * 256:(rank + 1) * 256].contiguous()
    lm._plain_2d = lambda layer, x2d, scale, N, K, block_h, compiling: olin.oracle_linear_fp32(x2d, layer.weight, scale, block_h).to(torch.float16)
    lm.observability.on_apply = lambda layer: None
    bias = (torch.arange(256, dtype=torch.float32) * 1e-2).to(torch.float16)
    comm = types.SimpleNamespace(max_out_elems=1 << 20)            # large enough: only the bias keeps the call off the fused path
    lay = types.SimpleNamespace(weight=wr, weight_scale_inv=sr, weight_block_size=[128, 128], input_size_per_partition=256,
                                output_size_per_partition=256, w8a16_peer_comm=comm, bias=bias)
    m = lm.Fp8LinearMethod((128, 128))
    y = m.apply(lay, xs, bias if rank == 0 else None)              # vLLM: bias on rank 0 only
    ref = olin.oracle_linear_fp32(x, w, s, bh) + bias.float()
    ok = bool(torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2))
    # too large for the communicator: plain GEMM + all-reduce, still reduced
    lay2 = types.SimpleNamespace(**{**vars(lay), "w8a16_peer_comm": types.SimpleNamespace(max_out_elems=16), "bias": None})
    y2 = m.apply(lay2, xs)
    ok = ok and bool(torch.allclose(y2.float(), olin.oracle_linear_fp32(x, w, s, bh), atol=3e-2, rtol=2e-2))
    # a bias handed to a layer that declares none cannot be agreed on: loud failure, on the rank that sees it
    if rank == 0:
        try:
            m.apply(lay2, xs, bias)
            ok = False
        except RuntimeError as exc:
            ok = ok and "could not agree" in str(exc)
    q.put((rank, ok))
    dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_tp_worker, _ep_worker, _comm_failure_worker, _hook_path_worker])
def test_two_gloo_ranks(worker):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == {0: True, 1: True}


def test_ep_plan_index_arithmetic():
    from vllm_fp8_w8a16_sm70_b200.parallel import ep_plan
    ids = torch.tensor([[5, 0], [-1, 3], [7, 6]])
    order, counts, local = ep_plan(ids, 8, 4)
    assert order.tolist() == [1, 3, 0, 4, 5] and counts.tolist() == [1, 1, 1, 2] and local.tolist() == [0, 1, 1, 1, 0]


def test_shard_rules_reject_unaligned():
    from vllm_fp8_w8a16_sm70_b200 import parallel as par
    w, s = torch.zeros(384, 512, dtype=torch.uint8), torch.zeros(3, 4)
    with pytest.raises(ValueError):
        par.shard_column_parallel(w, s, 2, 0)          # 192 rows per rank: not a multiple of 128
    with pytest.raises(ValueError):
        par.shard_row_parallel(w, s, 8, 0)             # 64 columns per rank with block scales
    wr, sr = par.shard_row_parallel(w, s, 4, 1)
    assert tuple(wr.shape) == (384, 128) and tuple(sr.shape) == (3, 1)
