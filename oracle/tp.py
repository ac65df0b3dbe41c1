"""Tensor-parallel sharding of FP8 weights and their block-scale grids (test
infrastructure).

Restates the offline emulation of vLLM's TP sharding in
``tests/test_attention_shapes.py:75-101``: column-parallel layers are cut along
the output dimension (weight rows and scale-grid rows together), row-parallel
layers along the input dimension (weight columns and scale-grid columns
together), and fused modules concatenate per-partition shards along dim 0.
"""

from __future__ import annotations

import torch


def shard_col_parallel(W: torch.Tensor, S: torch.Tensor, tp_size: int, tp_rank: int):
    """W [N,K], S [Nb,Kb] -> rank's rows (tests/test_attention_shapes.py:75-84)."""
    N = W.shape[0]
    assert N % tp_size == 0, f"N={N} not divisible by tp_size={tp_size}"
    n_per = N // tp_size
    nb_per = S.shape[0] // tp_size
    return (W[tp_rank * n_per:(tp_rank + 1) * n_per].contiguous(),
            S[tp_rank * nb_per:(tp_rank + 1) * nb_per].contiguous())


def shard_row_parallel(W: torch.Tensor, S: torch.Tensor, tp_size: int, tp_rank: int):
    """W [N,K], S [Nb,Kb] -> rank's columns (tests/test_attention_shapes.py:87-95)."""
    K = W.shape[1]
    assert K % tp_size == 0, f"K={K} not divisible by tp_size={tp_size}"
    k_per = K // tp_size
    kb_per = S.shape[1] // tp_size
    return (W[:, tp_rank * k_per:(tp_rank + 1) * k_per].contiguous(),
            S[:, tp_rank * kb_per:(tp_rank + 1) * kb_per].contiguous())


def fuse_merged(parts_w, parts_s):
    """MergedColumnParallelLinear layout (tests/test_attention_shapes.py:97-101)."""
    return torch.cat(list(parts_w), dim=0).contiguous(), torch.cat(list(parts_s), dim=0).contiguous()


def expert_partition(num_experts: int, ep_size: int, ep_rank: int):
    """Contiguous expert-parallel partition and the global->local ``expert_map``
    (non-local -> -1) consumed at src/fp8_w8a16_sm70/vllm_serve.py:2237-2243."""
    assert num_experts % ep_size == 0
    per = num_experts // ep_size
    lo = ep_rank * per
    emap = torch.full((num_experts,), -1, dtype=torch.int32)
    emap[lo:lo + per] = torch.arange(per, dtype=torch.int32)
    return lo, lo + per, emap
