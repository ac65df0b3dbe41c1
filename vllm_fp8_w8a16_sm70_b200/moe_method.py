"""vLLM-facing fused-MoE hooks on the B200 engine.

Mirrors what the reference assigns onto ``Fp8MoEMethod`` / ``Fp8OnlineMoEMethod``
(``src/fp8_w8a16_sm70/vllm_serve.py:1526-1624`` init + process_weights_after_loading,
``:2175-2411`` apply, patched in at ``:2640-2719``) and onto
``CompressedTensorsW8A8Fp8MoEMethod`` (``src/fp8_w8a16_sm70/compressed_tensors_v100.py:978-1234``).

``apply`` returns the ROUTED-ONLY output ``[M, H]``; shared experts and the tensor-parallel reduce
stay with the caller, as in the reference (``vllm_serve.py:2182``).  The reference's per-expert
Python loop, its ``nonzero`` route prep and its ``MAX_ROUTE_SLOTS`` switch disappear: one device-side
pipeline serves every token count without host synchronisation.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .backend import select_backend
from .linear_method import _check_scale_range, _set


def _activation_name(layer) -> str:
    """SiLU / SwiGLU or GELU, as the reference's ``_moe_activation`` (vllm_serve.py:1627-1636); anything else raises."""
    activation = getattr(layer, "activation", "silu")
    name = getattr(activation, "name", str(activation)).upper()
    if "SILU" in name or "SWIGLU" in name:
        return "silu"
    if "GELU" in name:
        return "gelu"
    raise NotImplementedError(f"FP8 W8A16 MoE engine: unsupported activation {activation!r}")


class Fp8MoEMethod:
    """Block-128 FP8 experts: ``w13_weight [E, 2I, H]``, ``w2_weight [E, H, I]`` with
    ``*_weight_scale_inv`` grids ``[E, 2I/128, H/128]`` and ``[E, H/128, I/128]``."""

    def __init__(self, quant_config=None, layer=None, weight_block_size=(128, 128)):
        wbs = getattr(quant_config, "weight_block_size", None) if quant_config is not None else weight_block_size
        self.quant_config = quant_config
        self.weight_block_size = None if wbs is None else tuple(wbs)
        self.block_quant = self.weight_block_size is not None
        self.weight_scale_name = "weight_scale_inv" if self.block_quant else "weight_scale"
        self.block_h = 128

    def maybe_make_prepare_finalize(self, routing_tables=None):
        return None  # vllm_serve.py:2708-2711: no modular-kernel prepare/finalize

    def process_weights_after_loading(self, layer) -> None:
        if getattr(layer, "_already_called_process_weights_after_loading", False):
            return
        if not self.block_quant:
            raise NotImplementedError("FP8 W8A16 MoE engine: native fp8 experts must be block-quantised")
        w13 = layer.w13_weight.data if hasattr(layer.w13_weight, "data") else layer.w13_weight
        w2 = layer.w2_weight.data if hasattr(layer.w2_weight, "data") else layer.w2_weight
        for w in (w13, w2):
            select_backend(strategy="BLOCK", weight_block_size=self.weight_block_size, local_n=int(w.shape[1]),
                           local_k=int(w.shape[2]), need_moe=True)
        for name in ("w13", "w2"):
            s = getattr(layer, f"{name}_{self.weight_scale_name}")
            s = s.data if hasattr(s, "data") else s
            if s.dtype != torch.float16:
                s = s.to(torch.float16)
            _check_scale_range(s, f"{getattr(layer, 'prefix', 'moe')}.{name}")
            _set(layer, f"{name}_{self.weight_scale_name}", s.contiguous())
        _set(layer, "w13_weight", w13.contiguous())
        _set(layer, "w2_weight", w2.contiguous())
        layer.w13_input_scale = None
        layer.w2_input_scale = None
        layer._already_called_process_weights_after_loading = True

    def apply(self, layer, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
              shared_experts_input=None, shared_experts=None) -> torch.Tensor:
        """Accepts both the 5-argument form the reference targets (vllm_serve.py:2683) and the
        6-argument form of newer vLLM; the shared-expert arguments are ignored on purpose."""
        del shared_experts_input, shared_experts
        act = _activation_name(layer)
        x_work = x if x.dtype == torch.float16 else x.to(torch.float16)
        x_work = x_work.contiguous()
        tw = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
        ids = topk_ids if topk_ids.dtype in (torch.int32, torch.int64) else topk_ids.to(torch.int32)
        emap = getattr(layer, "expert_map", None)
        if emap is not None and (emap.dtype != torch.int32 or emap.device != x.device):
            emap = emap.to(device=x.device, dtype=torch.int32)
        s13, s2 = getattr(layer, f"w13_{self.weight_scale_name}"), getattr(layer, f"w2_{self.weight_scale_name}")
        on_input = bool(getattr(layer, "apply_router_weight_on_input", False))
        from . import custom_ops
        if custom_ops.compiling():     # a compiler is tracing: go through the registered op so the graph does not break
            out = custom_ops.moe_forward(x_work, tw.contiguous(), ids.contiguous(), layer.w13_weight.view(torch.uint8), s13,
                                         layer.w2_weight.view(torch.uint8), s2, self.block_h, on_input, act, emap)
        else:
            out = ops.moe_forward(x_work, tw.contiguous(), ids.contiguous(), layer.w13_weight, s13, layer.w2_weight, s2,
                                  block_h=self.block_h, expert_map=emap, weight_on_input=on_input, activation=act)
        return out if out.dtype == x.dtype else out.to(x.dtype)


class CompressedTensorsFp8MoEMethod(Fp8MoEMethod):
    """compressed-tensors FP8 experts (the hooks the reference assigns onto ``CompressedTensorsW8A8Fp8MoEMethod``,
    compressed_tensors_v100.py:1041-1229).  Scale layouts, as the reference's ``_dequant_expert`` accepts them
    (:1060-1071): per output channel ``[E, rows, 1]`` / ``[E, rows]``, per tensor ``[E]`` (and, for a fused w13 whose
    gate and up shards were quantised separately, ``[E, 2]``), or block ``[E, rows/128, K/128]``.  The reference keeps
    w13 FP8 with the channel scale expanded to a ``block_h = 1`` grid and stores w2 as FP16 because its kernels need
    K % 128 == 0 (compressed_tensors_v100.py:1090-1106, :931-950); here both stay FP8: the grouped GEMM takes any K
    that is a multiple of 16 (e.g. I/tp = 176)."""

    def __init__(self, weight_quant=None, input_quant=None, moe=None, layer_name=None, strategy: str = "CHANNEL"):
        super().__init__(quant_config=None, weight_block_size=None)
        strat = getattr(weight_quant, "strategy", None)
        if strat is not None:
            strategy = str(getattr(strat, "name", None) or getattr(strat, "value", None) or strat)
        self.strategy = strategy.upper()
        self.block_quant = "BLOCK" in self.strategy
        self.weight_scale_name = "weight_scale"
        self.block_h = 128 if self.block_quant else 1

    @staticmethod
    def _row_scales(name: str, s: torch.Tensor, E: int, rows: int) -> torch.Tensor:
        """Any of the non-block layouts -> one FP16 scale per (expert, weight row), ``[E, rows, 1]``."""
        n = s.numel()
        if n == E * rows:
            return s.reshape(E, rows, 1)
        if n == E:
            return s.reshape(E, 1, 1).expand(E, rows, 1)
        if n == 2 * E and name == "w13" and rows % 2 == 0:      # one scale per logical shard: gate rows, then up rows
            return s.reshape(E, 2, 1).repeat_interleave(rows // 2, dim=1)
        raise ValueError(f"{name}: cannot map {n} scales ({tuple(s.shape)}) onto [{E},{rows}] weight rows")

    def process_weights_after_loading(self, layer) -> None:
        if getattr(layer, "_already_called_process_weights_after_loading", False):
            return
        for name in ("w13", "w2"):
            w = getattr(layer, f"{name}_weight")
            w = w.data if hasattr(w, "data") else w
            E, rows, K = (int(v) for v in w.shape)
            select_backend(strategy=self.strategy, weight_block_size=(128, 128) if self.block_quant else None, local_n=rows,
                           local_k=K, need_moe=True)
            s = getattr(layer, f"{name}_weight_scale")
            s = (s.data if hasattr(s, "data") else s).to(torch.float16)
            if not self.block_quant:
                s = self._row_scales(name, s, E, rows).expand(E, rows, -(-K // 128))
            elif tuple(s.shape) != (E, -(-rows // 128), -(-K // 128)):
                raise ValueError(f"{name}: block scale grid {tuple(s.shape)} does not match weight [{E},{rows},{K}]")
            _check_scale_range(s, f"{getattr(layer, 'prefix', 'moe')}.{name}")
            _set(layer, f"{name}_weight_scale", s.contiguous())
            _set(layer, f"{name}_weight", w.contiguous())
        layer.w13_input_scale = None
        layer.w2_input_scale = None
        layer._already_called_process_weights_after_loading = True

    def get_fused_moe_quant_config(self, layer):
        return None
