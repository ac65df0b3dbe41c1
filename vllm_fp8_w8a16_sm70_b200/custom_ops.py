"""``torch.library`` registrations of the engine's two hot ops, with fake (shape-only) implementations.

The reference wraps its pybind calls in ``torch._dynamo.disable`` because Dynamo cannot trace them, which breaks the graph
at every linear (``src/fp8_w8a16_sm70/vllm_serve.py:52-75``).  Registered custom ops are the clean fix: Dynamo / AOT
autograd see ``fp8w8a16_b200::linear`` and ``fp8w8a16_b200::moe_forward`` as opaque nodes with known output shapes, so a
model compiled with ``torch.compile`` keeps one graph, and vLLM's piecewise CUDA-graph capture can include them.  The hooks
(``linear_method`` / ``moe_method``) call the ops directly in eager mode (no dispatcher overhead on the decode path) and go
through these registrations only while a compiler is tracing.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops

NAMESPACE = "fp8w8a16_b200"


@torch.library.custom_op(f"{NAMESPACE}::linear", mutates_args=(), device_types="cuda")
def linear(x: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor, N: int, K: int, block_h: int, block_w: int) -> torch.Tensor:
    return ops.w8a16_linear(x, weight, scales, N, K, block_h, block_w)


@linear.register_fake
def _linear_fake(x, weight, scales, N, K, block_h, block_w):
    torch._check(x.dim() == 2 and x.shape[1] == K, lambda: f"x must be [M, {K}]")
    return x.new_empty((x.shape[0], N), dtype=torch.float16)


@torch.library.custom_op(f"{NAMESPACE}::moe_forward", mutates_args=(), device_types="cuda")
def moe_forward(x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, w13: torch.Tensor, s13: torch.Tensor,
                w2: torch.Tensor, s2: torch.Tensor, block_h: int, weight_on_input: bool, activation: str,
                expert_map: Optional[torch.Tensor] = None) -> torch.Tensor:
    return ops.moe_forward(x, topk_weights, topk_ids, w13, s13, w2, s2, block_h=block_h, weight_on_input=weight_on_input,
                           activation=activation, expert_map=expert_map)


@moe_forward.register_fake
def _moe_forward_fake(x, topk_weights, topk_ids, w13, s13, w2, s2, block_h, weight_on_input, activation, expert_map=None):
    torch._check(x.dim() == 2 and topk_ids.shape[0] == x.shape[0], lambda: "x [M, H] and topk_ids [M, topk] disagree on M")
    return x.new_empty((x.shape[0], w2.shape[1]), dtype=torch.float16)


def compiling() -> bool:
    fn = getattr(torch.compiler, "is_compiling", None)
    return bool(fn()) if fn is not None else False
