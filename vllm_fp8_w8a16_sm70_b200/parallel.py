"""Tensor-parallel dense layers and expert-parallel MoE over ``torch.distributed`` (NCCL on GPUs).

In the reference these collectives belong to vLLM: the plugin only sees per-rank shards
(``src/fp8_w8a16_sm70/vllm_serve.py:1386-1387``) and mirrors vLLM's call sites for timing
(row-parallel: split input, apply, all-reduce, bias on rank 0 only — ``vllm_serve.py:2922-2959``;
MoE: experts, then reduce — ``:2785-2853``).  Expert parallelism is only *tolerated* there
(``expert_map`` + a later reduce, ``:2237-2243``); the all-to-all dispatch / combine below is new,
and its oracle is the single-GPU layer.

One process per GPU.  Row-parallel layers can run with the all-reduce fused into the GEMM kernel over peer
memory (``make_peer_comm`` + ``TensorParallelLinear(..., comm=...)``); everything else exchanges through NCCL.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


# ------------------------------------------------------------------------------------------------
# sharding rules (what vLLM's loaders do to the FP8 weight and its block-scale grid)
# ------------------------------------------------------------------------------------------------
def shard_column_parallel(w: torch.Tensor, s: torch.Tensor, tp_size: int, tp_rank: int, block_h: int = 128):
    """Cut along the output dimension: weight rows and scale-grid rows together."""
    N = w.shape[0]
    if N % tp_size:
        raise ValueError(f"N={N} not divisible by tp_size={tp_size}")
    n_per = N // tp_size
    if n_per % block_h:
        raise ValueError(f"per-rank N={n_per} is not a multiple of block_h={block_h}")
    nb_per = n_per // block_h
    return (w[tp_rank * n_per:(tp_rank + 1) * n_per].contiguous(), s[tp_rank * nb_per:(tp_rank + 1) * nb_per].contiguous())


def shard_row_parallel(w: torch.Tensor, s: torch.Tensor, tp_size: int, tp_rank: int, block_w: int = 128):
    """Cut along the input dimension: weight columns and scale-grid columns together."""
    K = w.shape[1]
    if K % tp_size:
        raise ValueError(f"K={K} not divisible by tp_size={tp_size}")
    k_per = K // tp_size
    if k_per % block_w and s.shape[1] > 1:
        # a per-rank K that is not 128-aligned needs per-channel scales (one grid column per started block)
        raise ValueError(f"per-rank K={k_per} is not a multiple of block_w={block_w}")
    kb_per = -(-k_per // block_w)
    return (w[:, tp_rank * k_per:(tp_rank + 1) * k_per].contiguous(), s[:, tp_rank * kb_per:(tp_rank + 1) * kb_per].contiguous())


class TensorParallelLinear:
    """One rank's shard of a column- or row-parallel FP8 linear."""

    def __init__(self, w_shard: torch.Tensor, s_shard: torch.Tensor, block_h: int, mode: str,
                 group: Optional[dist.ProcessGroup] = None, linear_fn: Optional[Callable] = None,
                 comm: Optional["ops.PeerComm"] = None, has_bias: bool = False):
        assert mode in ("column", "row")
        self.w, self.s, self.block_h, self.mode, self.group = w_shard, s_shard, block_h, mode, group
        self.N, self.K = int(w_shard.shape[0]), int(w_shard.shape[1])
        self._custom_linear = linear_fn
        self._linear = linear_fn or (lambda x: ops.w8a16_linear(x, self.w, self.s, self.N, self.K, self.block_h, 128))
        self.comm = comm if mode == "row" else None   # fused GEMM + all-reduce over peer memory
        # whether the LAYER has a bias: the same on every rank, unlike the bias argument of forward (rank 0 only)
        self.has_bias = bool(has_bias)

    def forward(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """column: x [M, K] (replicated) -> [M, N/tp].  row: x [M, K/tp] -> all-reduced [M, N]; the bias is
        added on rank 0 only before the reduce, as vLLM does.  The fused kernel is chosen from rank-invariant facts
        only (token count, communicator size, ``has_bias``): a rank that went another way would leave its peers waiting.
        ``residual`` (row mode, float16 [M, N], replicated): the decoder's residual stream, added to the reduced result
        with one rounding - inside the GEMM kernel on the fused paths."""
        if bias is not None and self.mode == "row" and self.comm is not None and not self.has_bias:
            raise RuntimeError("bias passed to a row-parallel layer built with has_bias=False: the ranks could not agree on the path")
        if self.comm is not None and not self.has_bias and x.shape[0] * self.N <= self.comm_max_elems():
            return ops.w8a16_linear_allreduce(self.comm, x, self.w, self.s, self.N, self.K, self.block_h, 128, residual=residual)
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        if residual is not None and self.mode == "row" and world == 1 and bias is None and self._custom_linear is None:
            return ops.w8a16_linear(x, self.w, self.s, self.N, self.K, self.block_h, 128, residual=residual)
        y = self._linear(x)
        if self.mode == "row":
            if bias is not None and dist.get_rank(self.group) == 0:
                y = y + bias.to(y.dtype)
            if world > 1:
                dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
            if residual is not None:
                y = (y.float() + residual.float()).to(y.dtype)
        elif bias is not None:
            y = y + bias.to(y.dtype)
        return y

    def comm_max_elems(self) -> int:
        return getattr(self.comm, "max_out_elems", 0)


def _make_shared(create: Callable, what: str, group: Optional[dist.ProcessGroup]):
    """Collective set-up of a peer-mapped buffer: every rank of ``group`` creates its buffer on its current CUDA device,
    the IPC handles travel through ``all_gather_object`` and every rank maps every peer.  Failures are agreed on: if any
    rank cannot create or map a buffer, every rank closes what it has and raises, so the callers stay in step.  Ends with
    a barrier so that no rank launches before all mappings exist."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    comm, err = None, None
    try:
        comm = create(rank, world)
        mine = comm.handle()
    except Exception as exc:  # noqa: BLE001 - re-raised on every rank below
        mine, err = None, repr(exc)
    handles = [None] * world
    dist.all_gather_object(handles, (mine, err), group=group)
    if all(h is not None for h, _ in handles):
        try:
            for peer, (h, _) in enumerate(handles):
                if peer != rank:
                    comm.attach(peer, h)
        except Exception as exc:  # noqa: BLE001
            err = repr(exc)
    verdicts = [None] * world
    dist.all_gather_object(verdicts, err, group=group)
    failed = [(r, e) for r, ((h, e0), e) in enumerate(zip(handles, verdicts)) if h is None or e is not None]
    if failed:
        if comm is not None:
            comm.close()
        raise RuntimeError(f"{what} could not be set up: {failed}")
    dist.barrier(group=group)
    return comm


def make_peer_comm(max_out_elems: int, timeout_ms: int = 2000, group: Optional[dist.ProcessGroup] = None) -> "ops.PeerComm":
    """The communicator of the fused row-parallel GEMM + all-reduce (collective; raises on every rank or on none)."""
    return _make_shared(lambda rank, world: ops.PeerComm(rank, world, max_out_elems, timeout_ms), "peer-memory communicator", group)


def make_ep_comm(max_tokens: int, topk: int, hidden: int, num_experts: int, timeout_ms: int = 2000,
                 group: Optional[dist.ProcessGroup] = None) -> "ops.EpComm":
    """The exchange buffer of the expert-parallel MoE layer (collective; raises on every rank or on none)."""
    return _make_shared(lambda rank, world: ops.EpComm(rank, world, max_tokens, topk, hidden, num_experts, timeout_ms),
                        "expert-parallel exchange buffer", group)


def reset_peer_comm(comm, group: Optional[dist.ProcessGroup] = None) -> None:
    """Collective recovery of a peer-memory communicator (``PeerComm`` or ``EpComm``) after the ranks' launch sequences diverged (one rank raised before
    launching, or a kernel gave up waiting for a peer and the device status word reported bit 128): every rank waits
    for its own GPU, all meet at a barrier (no fused kernel is in flight anywhere), each resets its launch number and
    empties its inbox, waits for that, and all meet again before anyone launches."""
    torch.cuda.synchronize(comm.device)
    dist.barrier(group=group)
    comm.reset()
    torch.cuda.synchronize(comm.device)
    ops.reset_workspaces()
    dist.barrier(group=group)


# ------------------------------------------------------------------------------------------------
# expert parallelism: all-to-all dispatch / combine
# ------------------------------------------------------------------------------------------------
def ep_plan(topk_ids: torch.Tensor, num_experts: int, ep_size: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Routes of this rank's tokens grouped by destination rank (experts are partitioned contiguously).

    Returns (order, send_counts, local_ids): ``order`` is a stable permutation of the valid flat route
    indices sorted by destination rank, ``send_counts[p]`` the number of routes going to rank p and
    ``local_ids`` the expert id local to its destination, in ``order``.  Invalid ids (< 0) are dropped."""
    per = num_experts // ep_size
    flat = topk_ids.reshape(-1).to(torch.int64)
    valid = (flat >= 0) & (flat < num_experts)
    dest = torch.where(valid, flat // per, torch.full_like(flat, ep_size))
    order = torch.sort(dest, stable=True).indices
    n_valid = int(valid.sum())
    order = order[:n_valid]
    send_counts = torch.bincount(dest[order], minlength=ep_size)[:ep_size]
    local_ids = (flat[order] % per).to(torch.int32)
    return order, send_counts, local_ids


class ExpertParallelMoE:
    """MoE layer whose experts are split over the ranks of ``group``; each rank brings its own tokens.

    forward: plan -> all-to-all(rows, local expert ids) -> local experts on the received rows (each row is a
    single-expert route, weight 1) -> all-to-all back -> weighted sum per token on the source rank."""

    def __init__(self, w13: torch.Tensor, s13: torch.Tensor, w2: torch.Tensor, s2: torch.Tensor, num_experts: int,
                 block_h: int = 128, group: Optional[dist.ProcessGroup] = None, expert_fn: Optional[Callable] = None,
                 peer_tokens: int = 0, topk: int = 0, hidden: int = 0):
        self.peer = None
        self.w13, self.s13, self.w2, self.s2 = w13, s13, w2, s2
        self.num_experts, self.block_h, self.group = num_experts, block_h, group
        self.ep_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.local_experts = num_experts // self.ep_size
        assert num_experts % self.ep_size == 0 and w13.shape[0] == self.local_experts
        self._experts = expert_fn or self._engine_experts
        import os
        self.coalesce = os.environ.get("FP8W8A16_EP_COALESCE", "1") != "0"
        # peer_tokens > 0: set up the peer-memory exchange (collective) for up to that many tokens per rank and call
        if peer_tokens > 0 and self.ep_size > 1 and expert_fn is None and w13.is_cuda:
            self.peer = make_ep_comm(peer_tokens, topk, hidden or int(w13.shape[2]), num_experts, group=group)

    def modes(self):
        """Exchange modes this layer can run: the two NCCL ones, and "peer" when a peer-memory exchange buffer was set up."""
        return (["peer"] if self.peer is not None else []) + ["allgather", "a2a"]

    def close(self) -> None:
        if self.peer is not None:
            self.peer.close()
            self.peer = None

    def _engine_experts(self, rows: torch.Tensor, local_ids: torch.Tensor) -> torch.Tensor:
        ones = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=rows.device)
        return ops.moe_forward(rows, ones, local_ids.reshape(-1, 1).contiguous(), self.w13, self.s13, self.w2, self.s2,
                               block_h=self.block_h)

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, mode: str = "auto") -> torch.Tensor:
        """``mode``: "a2a" = variable-size all-to-all dispatch / combine (one host synchronisation for the split
        sizes; traffic proportional to the routed rows), "allgather" = fixed-size all-gather of tokens and routes,
        local experts on every token through ``expert_map``, reduce-scatter of the outputs (no host
        synchronisation, CUDA-graph capturable; the right choice for decode batches), "auto" = all-gather up to
        4096 tokens in flight, all-to-all above."""
        if mode == "auto":
            if self.peer is not None and x.shape[0] <= self.peer.max_tokens:
                mode = "peer"
            else:
                mode = "allgather" if x.shape[0] * self.ep_size <= 4096 else "a2a"
        if mode == "peer":
            if self.peer is None:
                raise RuntimeError("this layer was built without a peer-memory exchange buffer (peer_tokens=0)")
            return self.forward_peer(x, topk_weights, topk_ids)
        if mode == "allgather" and self.ep_size > 1 and self._experts == self._engine_experts:
            return self.forward_allgather(x, topk_weights, topk_ids)
        return self.forward_a2a(x, topk_weights, topk_ids)

    def forward_peer(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, m_max: Optional[int] = None) -> torch.Tensor:
        """Dispatch / experts / combine by the library's own kernels over peer memory: only routed rows travel, nothing is
        read back on the host, no NCCL call (CUDA-graph capturable).  ``m_max``: the largest token count of any rank in
        this call, identical on all ranks (default: equal batches)."""
        ids = topk_ids if topk_ids.dtype in (torch.int32, torch.int64) else topk_ids.to(torch.int32)
        tw = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
        return ops.ep_moe_forward(self.peer, x.contiguous(), tw.contiguous(), ids.contiguous(), self.w13, self.s13, self.w2, self.s2,
                                  block_h=self.block_h, m_max=m_max)

    def forward_allgather(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        """Every rank brings M tokens (the same M on all ranks).  all-gather -> [P*M] tokens; this rank's experts
        contribute to every token (routes to other ranks' experts are dropped by the expert_map, exactly the
        reference's tolerated-EP semantics, vllm_serve.py:2237-2243); reduce-scatter(sum) returns each rank the
        finished rows of its own tokens."""
        P = self.ep_size
        M, H = x.shape
        topk = topk_ids.shape[-1]
        ids32 = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        # grouped launch or packed rows: measured, the grouped form wins on 2 GPUs at every batch (60 vs 67 us at 1 token per
        # GPU, 139 vs 152 us at 64) and on 8 GPUs from ~1000 gathered tokens on (267 vs 285 us at 256 per GPU), while for
        # small gathers on 8 GPUs three grouped all-gathers cost more than one (94 vs 80 us at 1 token per GPU)
        grouped_gather = self.coalesce and (P <= 2 or P * M >= 1024)
        if grouped_gather and x.is_cuda and dist.get_backend(self.group) == "nccl":
            # activations, expert ids and route weights gathered by ONE grouped NCCL launch straight into the three tensors
            # the layer takes, without packing and unpacking kernels (FP8W8A16_EP_COALESCE=0 always takes the packed exchange)
            xg = x.new_empty((P * M, H))
            ig = ids32.new_empty((P * M, topk))
            wg = topk_weights.new_empty((P * M, topk))
            with dist._coalescing_manager(group=self.group, device=x.device):
                dist.all_gather_into_tensor(xg, x.contiguous(), group=self.group)
                dist.all_gather_into_tensor(ig, ids32.contiguous(), group=self.group)
                dist.all_gather_into_tensor(wg, topk_weights.contiguous(), group=self.group)
        else:
            # other backends: one collective of packed rows (activations, ids, weights of a token as bytes)
            row_bytes = 2 * H + 8 * topk
            packed = torch.empty((M, row_bytes), dtype=torch.uint8, device=x.device)
            packed[:, :2 * H] = x.contiguous().view(torch.uint8).reshape(M, 2 * H)
            packed[:, 2 * H:2 * H + 4 * topk] = ids32.contiguous().view(torch.uint8).reshape(M, 4 * topk)
            packed[:, 2 * H + 4 * topk:] = topk_weights.contiguous().view(torch.uint8).reshape(M, 4 * topk)
            gathered = torch.empty((P * M, row_bytes), dtype=torch.uint8, device=x.device)
            dist.all_gather_into_tensor(gathered, packed, group=self.group)
            xg = gathered[:, :2 * H].contiguous().view(torch.float16).reshape(P * M, H)
            ig = gathered[:, 2 * H:2 * H + 4 * topk].contiguous().view(torch.int32).reshape(P * M, topk)
            wg = gathered[:, 2 * H + 4 * topk:].contiguous().view(torch.float32).reshape(P * M, topk)
        if getattr(self, "_emap", None) is None or self._emap.device != x.device:
            rank = dist.get_rank(self.group)
            emap = torch.full((self.num_experts,), -1, dtype=torch.int32)
            emap[rank * self.local_experts:(rank + 1) * self.local_experts] = torch.arange(self.local_experts, dtype=torch.int32)
            self._emap = emap.to(x.device)
        y = ops.moe_forward(xg, wg, ig, self.w13, self.s13, self.w2, self.s2, block_h=self.block_h, expert_map=self._emap)
        out = x.new_empty((M, H))
        dist.reduce_scatter_tensor(out, y, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def forward_a2a(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        M, H = x.shape
        topk = topk_ids.shape[-1]
        order, send_counts, local_ids = ep_plan(topk_ids, self.num_experts, self.ep_size)
        send_rows = x.index_select(0, torch.div(order, topk, rounding_mode="floor"))
        if self.ep_size > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
            sc, rc = send_counts.tolist(), recv_counts.tolist()      # one host synchronisation per layer
            recv_rows = x.new_empty((sum(rc), H))
            recv_ids = local_ids.new_empty((sum(rc),))
            dist.all_to_all_single(recv_rows, send_rows.contiguous(), rc, sc, group=self.group)
            dist.all_to_all_single(recv_ids, local_ids.contiguous(), rc, sc, group=self.group)
        else:
            sc = rc = None
            recv_rows, recv_ids = send_rows.contiguous(), local_ids
        y_recv = self._experts(recv_rows, recv_ids) if recv_rows.shape[0] else recv_rows
        if self.ep_size > 1:
            y_back = x.new_empty((send_rows.shape[0], H))
            dist.all_to_all_single(y_back, y_recv.contiguous(), sc, rc, group=self.group)
        else:
            y_back = y_recv
        # weighted combine on the source rank: route weight as FP16 like the reference (vllm_serve.py:1804)
        w16 = topk_weights.reshape(-1)[order].to(torch.float16).float().unsqueeze(-1)
        out = torch.zeros((M, H), dtype=torch.float32, device=x.device)
        out.index_add_(0, torch.div(order, topk, rounding_mode="floor"), (y_back.float() * w16).to(torch.float16).float())
        return out.to(torch.float16)
