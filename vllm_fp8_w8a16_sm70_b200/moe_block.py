"""The MoE block around the reference's hook: router before it, shared expert and the final add after it.

In the reference these steps belong to vLLM's model code (gate Linear -> ``fused_topk`` -> experts hook -> ``routed +
shared`` -> tensor-parallel all-reduce, mirrored for timing at ``src/fp8_w8a16_sm70/vllm_serve.py:2785-2853``); the hook
itself returns the routed-only output.  Here they are fused around the same engine:

* the router gate GEMV and the top-k softmax are one kernel (``ops.moe_router_topk``);
* a shared expert whose shapes match the routed experts' (GLM-4.5-Air: one shared expert of the routed intermediate
  size) is stored as one more row of the expert stack and gets the fixed route ``(E, 1.0)`` from the router kernel, so
  the grouped gate/up and down GEMMs compute it with the routed experts and the combine kernel's sum IS
  ``routed + shared``: no separate dense MLP launches, no extra add.

The block is per rank.  With tensor-parallel experts (every rank holds a slice of every expert, as the reference runs
GLM-4.5-Air) the caller all-reduces the result; with expert parallelism a shared expert must not be folded in (every
rank would add its own copy) and ``shared`` has to stay ``None``.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops


class MoEBlock:
    def __init__(self, gate_weight: torch.Tensor, w13: torch.Tensor, s13: torch.Tensor, w2: torch.Tensor, s2: torch.Tensor,
                 topk: int, block_h: int = 128, renormalize: bool = True, activation: str = "silu",
                 routed_scaling_factor: float = 1.0,
                 shared: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]] = None):
        """``w13 [E, 2I, H]``, ``w2 [E, H, I]`` with their scale grids; ``shared = (w13_s [2I, H], s13_s, w2_s [H, I], s2_s)``
        in the same layout (same I, same scale scheme) or ``None``."""
        E, two_i, H = w13.shape
        if tuple(gate_weight.shape) != (E, H):
            raise ValueError(f"gate_weight must be [{E}, {H}] (got {tuple(gate_weight.shape)})")
        self.num_routed = E
        self.shared_id = -1
        if shared is not None:
            w13_s, s13_s, w2_s, s2_s = shared
            if tuple(w13_s.shape) != (two_i, H) or tuple(w2_s.shape) != tuple(w2.shape[1:]):
                raise ValueError(f"shared expert shapes {tuple(w13_s.shape)} / {tuple(w2_s.shape)} differ from the routed experts' "
                                 f"{(two_i, H)} / {tuple(w2.shape[1:])}: run it as a separate dense MLP")
            if tuple(s13_s.shape) != tuple(s13.shape[1:]) or tuple(s2_s.shape) != tuple(s2.shape[1:]):
                raise ValueError("shared expert scale grids differ from the routed experts' layout")
            w13 = torch.cat([ops._as_u8(w13), ops._as_u8(w13_s).unsqueeze(0)]).contiguous()
            w2 = torch.cat([ops._as_u8(w2), ops._as_u8(w2_s).unsqueeze(0)]).contiguous()
            s13 = torch.cat([s13, s13_s.to(s13.dtype).unsqueeze(0)]).contiguous()
            s2 = torch.cat([s2, s2_s.to(s2.dtype).unsqueeze(0)]).contiguous()
            self.shared_id = E
        self.gate_weight = gate_weight.contiguous()
        self.w13, self.s13, self.w2, self.s2 = w13, s13, w2, s2
        self.topk, self.block_h, self.renormalize, self.activation = topk, block_h, renormalize, activation
        self.routed_scaling_factor = float(routed_scaling_factor)

    def route(self, x: torch.Tensor):
        return ops.moe_router_topk(x, self.gate_weight, self.topk, self.renormalize, shared_expert_id=self.shared_id,
                                   routed_scale=self.routed_scaling_factor)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` float16 ``[M, H]`` -> ``routed (+ shared)`` float16 ``[M, H]``: 6 launches (5 up to 16 routed rows), no host synchronisation."""
        tw, ids = self.route(x)
        return ops.moe_forward(x, tw, ids, self.w13, self.s13, self.w2, self.s2, block_h=self.block_h, activation=self.activation)

    __call__ = forward
