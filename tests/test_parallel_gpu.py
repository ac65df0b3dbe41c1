"""Multi-GPU parity (needs >= 2 GPUs, skipped otherwise): tensor-parallel dense layers with NCCL all-reduce and
expert-parallel MoE (all-gather / reduce-scatter and all-to-all dispatch) against the single-process CPU oracle."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from oracle import linear as olin, moe as omoe
    from tests.helpers import make_dense, make_moe
    from vllm_fp8_w8a16_sm70_b200 import ops, parallel as par
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    res = {}
    try:
        # ---- dense TP: column-parallel up projection, row-parallel down projection + all-reduce ----
        x, w1, s1, bh = make_dense(9, 1024, 512, seed=1)
        _, w2, s2, _ = make_dense(9, 512, 1024, seed=2)
        wc, sc = par.shard_column_parallel(w1, s1, world, rank)
        wr, sr = par.shard_row_parallel(w2, s2, world, rank)
        col = par.TensorParallelLinear(wc.cuda(), sc.cuda(), bh, "column")
        row = par.TensorParallelLinear(wr.cuda(), sr.cuda(), bh, "row")
        h = col.forward(x.cuda())
        y = row.forward(h)
        h_full = olin.oracle_linear_fp32(x, w1, s1, bh).to(torch.float16)
        per = 1024 // world
        st = olin.error_stats(h.cpu(), h_full[:, rank * per:(rank + 1) * per].float())
        res["tp_col"] = st["rel_rms"] < 1e-2
        y_ref = olin.oracle_linear_fp32(h_full, w2, s2, bh)
        st = olin.error_stats(y.cpu(), y_ref)
        res["tp_row_allreduce"] = st["rel_rms"] < 1.5e-2 and st["finite"]
        # ---- row-parallel GEMM with the all-reduce fused into the kernel (peer memory) ----
        comm = par.make_peer_comm(max_out_elems=256 * 5120, timeout_ms=10000)
        fused_ok, same_ok = True, True
        cases = [(9, 1024, 512 if world <= 4 else 1024), (1, 5120, 5120), (8, 5120, 5120), (64, 5120, 25600), (200, 1024, 2048),
                 (8, 1000, 1024)]
        for ci, (Mf, Nf, Kf) in enumerate(cases):
            xf, wf, sf, bhf = make_dense(Mf, Nf, Kf, seed=20 + ci)
            wsh, ssh = par.shard_row_parallel(wf, sf, world, rank)
            k_per = Kf // world
            xs = xf[:, rank * k_per:(rank + 1) * k_per].contiguous().cuda()
            lay = par.TensorParallelLinear(wsh.cuda(), ssh.cuda(), bhf, "row", comm=comm)
            ref = olin.oracle_linear_fp32(xf, wf, sf, bhf)
            dist.barrier()                            # the CPU-side preparation above takes seconds and differs per rank
            for rep in range(3):                      # both buffer parities, repeated launches
                yf = lay.forward(xs)
            stf = olin.error_stats(yf.cpu(), ref)
            fused_ok = fused_ok and stf["rel_rms"] < 1.5e-2 and stf["finite"]
            both = [torch.empty_like(yf) for _ in range(world)]
            dist.all_gather(both, yf)
            same_ok = same_ok and all(torch.equal(both[0], b) for b in both[1:])
        res["fused_allreduce"] = fused_ok
        res["fused_allreduce_identical_on_all_ranks"] = same_ok
        # the residual stream joins the cross-rank sum inside the kernel (cluster and stream-K shapes), in place
        rok = True
        for ci, (Mf, Nf, Kf) in enumerate([(8, 5120, 5120), (40, 5120, 2048)]):
            xf, wf, sf, bhf = make_dense(Mf, Nf, Kf, seed=60 + ci)
            resid = torch.randn(Mf, Nf, generator=torch.Generator().manual_seed(70 + ci)).to(torch.float16)
            wsh, ssh = par.shard_row_parallel(wf, sf, world, rank)
            k_per = Kf // world
            xs = xf[:, rank * k_per:(rank + 1) * k_per].contiguous().cuda()
            lay = par.TensorParallelLinear(wsh.cuda(), ssh.cuda(), bhf, "row", comm=comm)
            ref = olin.oracle_linear_fp32(xf, wf, sf, bhf) + resid.float()
            dist.barrier()
            rbuf = resid.cuda()
            yr = lay.forward(xs, residual=rbuf)
            stf = olin.error_stats(yr.cpu(), ref)
            rok = rok and stf["rel_rms"] < 1.5e-2 and stf["finite"]
            nccl = par.TensorParallelLinear(wsh.cuda(), ssh.cuda(), bhf, "row").forward(xs, residual=rbuf)
            rok = rok and olin.error_stats(nccl.cpu(), ref)["rel_rms"] < 1.5e-2
        res["fused_allreduce_residual"] = rok
        # CUDA-graph replay of a fused call (the launch counter lives on the device)
        xf, wf, sf, bhf = make_dense(4, 5120, 5120, seed=31)
        wsh, ssh = par.shard_row_parallel(wf, sf, world, rank)
        xs = xf[:, rank * (5120 // world):(rank + 1) * (5120 // world)].contiguous().cuda()
        lay = par.TensorParallelLinear(wsh.cuda(), ssh.cuda(), bhf, "row", comm=comm)
        yg = torch.empty((4, 5120), dtype=torch.float16, device="cuda")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ops.w8a16_linear_allreduce(comm, xs, lay.w, lay.s, lay.N, lay.K, bhf, 128, out=yg)   # warm-up on the capture stream
            side.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                ops.w8a16_linear_allreduce(comm, xs, lay.w, lay.s, lay.N, lay.K, bhf, 128, out=yg)
                ops.w8a16_linear_allreduce(comm, xs, lay.w, lay.s, lay.N, lay.K, bhf, 128, out=yg)
            for _ in range(3):
                g.replay()
            side.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        stg = olin.error_stats(yg.cpu(), olin.oracle_linear_fp32(xf, wf, sf, bhf))
        res["fused_allreduce_graph"] = stg["rel_rms"] < 1.5e-2 and stg["finite"]
        dist.barrier()
        comm.close()
        # ---- MoE EP: each rank brings its own tokens ----
        E, I, H, topk, M = 16, 128, 256, 4, 12
        base = make_moe(E, I, H, 1, topk, seed=99)
        d = make_moe(E, I, H, M, topk, seed=10 + rank)
        per = E // world
        lo, hi = rank * per, (rank + 1) * per
        layer = par.ExpertParallelMoE(base["w13"][lo:hi].cuda(), base["s13"][lo:hi].cuda(), base["w2"][lo:hi].cuda(),
                                      base["s2"][lo:hi].cuda(), E, peer_tokens=16, topk=topk, hidden=H)
        ref = omoe.moe_reference_fp32(d["x"], d["tw"], d["ids"], base["w13"], base["s13"], base["w2"], base["s2"])
        assert layer.modes() == ["peer", "allgather", "a2a"]
        for mode in layer.modes():
            out = layer.forward(d["x"].cuda(), d["tw"].cuda(), d["ids"].cuda(), mode=mode)
            st = omoe.moe_error_stats(out.cpu(), ref)
            res[f"ep_{mode}"] = st["cos"] > 0.9999 and st["l2rel"] < 2e-2
        # the peer-memory exchange with a different batch on every rank (m_max agreed on), and under CUDA-graph replay
        m_r = 3 + 2 * rank
        d2 = make_moe(E, I, H, m_r, topk, seed=40 + rank, invalid_frac=0.2)
        ref2 = omoe.moe_reference_fp32(d2["x"], d2["tw"], d2["ids"], base["w13"], base["s13"], base["w2"], base["s2"])
        out2 = layer.forward_peer(d2["x"].cuda(), d2["tw"].cuda(), d2["ids"].cuda(), m_max=3 + 2 * (world - 1))
        st = omoe.moe_error_stats(out2.cpu(), ref2)
        res["ep_peer_ragged"] = st["cos"] > 0.9999 and st["l2rel"] < 2e-2
        xg, twg, idg = d["x"].cuda(), d["tw"].cuda(), d["ids"].cuda()
        og = torch.empty((M, H), dtype=torch.float16, device="cuda")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ops.ep_moe_forward(layer.peer, xg, twg, idg, layer.w13, layer.s13, layer.w2, layer.s2, out=og)      # workspace of this stream exists
            side.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                ops.ep_moe_forward(layer.peer, xg, twg, idg, layer.w13, layer.s13, layer.w2, layer.s2, out=og)
                ops.ep_moe_forward(layer.peer, xg, twg, idg, layer.w13, layer.s13, layer.w2, layer.s2, out=og)
            og.zero_()
            for _ in range(3):
                g.replay()
            side.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        st = omoe.moe_error_stats(og.cpu(), ref)
        res["ep_peer_graph"] = st["cos"] > 0.9999 and st["l2rel"] < 2e-2
        torch.cuda.synchronize()
        dist.barrier()
        layer.close()
        res["status"] = ops.device_status() == 0
    finally:
        q.put((rank, res))
        dist.destroy_process_group()


def _run(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(60)
    for r in range(world):
        assert got[r] and all(got[r].values()), got


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_and_ep_on_two_gpus(lib):
    _run(2)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four or more GPUs")
def test_tp_and_ep_on_all_gpus(lib):
    """The same checks with every GPU of the box as a rank (4 or 8): seven peers' packets per tile in the fused all-reduce."""
    _run(8 if torch.cuda.device_count() >= 8 else 4)
