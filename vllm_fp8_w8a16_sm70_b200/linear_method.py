"""vLLM-facing linear hooks on the B200 engine.

Mirrors the methods the reference assigns onto vLLM's classes:

* ``Fp8LinearMethod.process_weights_after_loading`` / ``.apply``
  (``src/fp8_w8a16_sm70/vllm_serve.py:1450-1523`` and ``:1372-1447``, patched in at ``:2592-2638``);
* ``CompressedTensorsW8A16Fp8.process_weights_after_loading`` / ``.apply_weights``
  (``src/fp8_w8a16_sm70/compressed_tensors_v100.py:461-574``).

A ``layer`` is any object with the attributes vLLM gives its linear layers: ``weight``
(float8_e4m3fn or uint8 ``[N, K]``), ``weight_scale_inv`` (native block FP8) or ``weight_scale``
(compressed-tensors), ``weight_block_size``, ``input_size_per_partition``,
``output_size_per_partition`` and, for per-tensor scales of fused modules, ``logical_widths``.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import custom_ops, observability, ops
from .backend import select_backend



def _set(layer, name: str, value: torch.Tensor) -> None:
    """replace_parameter-like: keep nn.Parameter wrapping when the layer is an nn.Module."""
    if isinstance(layer, torch.nn.Module) and isinstance(getattr(layer, name, None), torch.nn.Parameter):
        setattr(layer, name, torch.nn.Parameter(value, requires_grad=False))
    else:
        setattr(layer, name, value)


def _check_scale_range(s16: torch.Tensor, what: str) -> None:
    """A block scale that overflows FP16 when cast (inf) or is NaN would poison every output silently."""
    if s16.numel() and not bool(torch.isfinite(s16).all()):
        raise RuntimeError(f"{what}: scale grid holds non-finite values after the cast to FP16")


def _apply_2d(layer, x: torch.Tensor, bias, N: int, K: int, scale: torch.Tensor, block_h: int) -> torch.Tensor:
    compiling = torch.compiler.is_compiling()
    if not compiling:
        observability.on_apply(layer)
    orig_shape = x.shape
    x2d = x if x.dim() == 2 else x.reshape(-1, K)
    if x2d.dtype != torch.float16:
        x2d = x2d.to(torch.float16)
    if not x2d.is_contiguous():
        x2d = x2d.contiguous()
    if x2d.shape[-1] != K:
        raise RuntimeError(f"x must be [..., {K}] (got {tuple(x.shape)})")
    # A row-parallel layer that carries a peer-memory communicator (``layer.w8a16_peer_comm``, attached by the integrator
    # together with ``reduce_results = False`` and, for a non-default group, ``layer.w8a16_tp_group``) gets its
    # tensor-parallel reduce done HERE, on every path, so the caller always receives the summed result: fused into the
    # GEMM kernel when the call fits the communicator, a plain GEMM + all-reduce otherwise.  Every rank must take the
    # same path (the fused kernel waits for its peers), so the choice uses only facts all ranks share: the token
    # count, the communicator's size and whether the LAYER has a bias.  vLLM passes the bias argument on rank 0 only
    # (vllm_serve.py:2937-2945), so the argument itself must not decide.
    comm = getattr(layer, "w8a16_peer_comm", None)
    if comm is not None:
        layer_bias = getattr(layer, "bias", None) is not None and not getattr(layer, "skip_bias_add", False)
        if bias is not None and not layer_bias:
            raise RuntimeError("a bias was passed to a row-parallel layer whose .bias is None: the ranks could not agree on "
                               "the fused / plain path (set layer.bias on every rank)")
        fused = (not layer_bias) and (not compiling) and x2d.shape[0] * N <= getattr(comm, "max_out_elems", 0)
        if fused:
            out = ops.w8a16_linear_allreduce(comm, x2d, layer.weight, scale, N, K, block_h, 128)
        else:
            out = _plain_2d(layer, x2d, scale, N, K, block_h, compiling)
            if bias is not None:           # rank 0 only: added before the reduce, so it is counted once
                out = out + bias.to(out.dtype)
            import torch.distributed as dist
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=getattr(layer, "w8a16_tp_group", None))
        bias = None
    else:
        out = _plain_2d(layer, x2d, scale, N, K, block_h, compiling)
    if len(orig_shape) != 2:
        out = out.reshape(orig_shape[:-1] + (N,))
    if bias is not None:
        out = out + bias.to(out.dtype)
    if out.dtype != x.dtype:
        out = out.to(x.dtype)
    return out


def _plain_2d(layer, x2d: torch.Tensor, scale: torch.Tensor, N: int, K: int, block_h: int, compiling: bool) -> torch.Tensor:
    """This rank's GEMM alone, float16 ``[M, N]``."""
    if compiling:                   # a compiler is tracing: go through the registered op so the graph does not break
        w8 = layer.weight if layer.weight.dtype == torch.uint8 else layer.weight.view(torch.uint8)
        return custom_ops.linear(x2d, w8, scale, N, K, block_h, 128)
    if not x2d.is_cuda:
        raise RuntimeError(f"x is on {x2d.device}: the engine runs on CUDA tensors only (there is no CPU path)")
    # per-layer plan: pointers, shapes and the C entry point resolved once (rebuilt if the tensors were replaced)
    plan = getattr(layer, "_w8a16_plan", None)
    if plan is None or not plan.matches(layer.weight, scale) or x2d.device != plan.dev:
        plan = ops.LinearPlan(layer.weight, scale, N, K, block_h)
        try:
            layer._w8a16_plan = plan
        except AttributeError:
            pass
    return plan.run(x2d)


class Fp8LinearMethod:
    """Native ``quant_method=fp8`` block-128 checkpoints (``weight`` + ``weight_scale_inv``)."""

    def __init__(self, weight_block_size=(128, 128)):
        self.weight_block_size = None if weight_block_size is None else tuple(weight_block_size)
        self.block_quant = self.weight_block_size is not None

    def process_weights_after_loading(self, layer) -> None:
        """Keep ``[N, K]`` FP8 row-major, cast ``weight_scale_inv`` (BF16 / fp32) to FP16 once, drop
        ``input_scale`` (vllm_serve.py:1450-1523).  Non-block FP8 is out of scope and fails closed
        (vllm_serve.py:2629-2635)."""
        if not self.block_quant:
            raise NotImplementedError("FP8 W8A16 engine: native fp8 checkpoints must be block-quantised")
        weight = layer.weight.data if hasattr(layer.weight, "data") else layer.weight
        scale = layer.weight_scale_inv.data if hasattr(layer.weight_scale_inv, "data") else layer.weight_scale_inv
        N, K = int(weight.shape[0]), int(weight.shape[1])
        wbs = self.weight_block_size or tuple(getattr(layer, "weight_block_size"))
        select_backend(strategy="BLOCK", weight_block_size=wbs, local_n=N, local_k=K)
        if scale.dtype != torch.float16:
            scale = scale.to(torch.float16)
        _check_scale_range(scale, getattr(layer, "prefix", "linear"))
        _set(layer, "weight", weight.contiguous())
        _set(layer, "weight_scale_inv", scale.contiguous())
        layer.weight_block_size = list(wbs)
        layer.input_scale = None
        if observability.selfcheck_enabled():
            observability.selfcheck_linear(layer.weight, layer.weight_scale_inv, N, K, int(wbs[0]), getattr(layer, "prefix", "linear"))

    def apply(self, layer, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``[..., K] -> [..., N]`` in ``x.dtype`` (vllm_serve.py:1372-1447)."""
        N = int(layer.output_size_per_partition)
        K = int(layer.input_size_per_partition)
        block_h, block_w = layer.weight_block_size
        if block_w != 128:
            raise NotImplementedError(f"block_w={block_w} is not supported")
        return _apply_2d(layer, x, bias, N, K, layer.weight_scale_inv, int(block_h))


class CompressedTensorsW8A16Fp8:
    """compressed-tensors W8A16-FP8 layouts: ``weight_scale`` is ``[N/128, K/128]`` (block),
    ``[N, 1]`` (channel) or ``[num_partitions]`` (tensor).  The weight stays FP8-resident in all
    three cases; channel and tensor scales become a ``block_h = 1`` grid ``[N, ceil(K/128)]``
    (compressed_tensors_v100.py:488-492; tensor scales are first expanded per logical shard as
    ``convert_to_channelwise`` does at :247-256)."""

    def __init__(self, strategy: str, weight_block_size=None):
        self.strategy = strategy.upper()
        self.weight_block_size = None if weight_block_size is None else tuple(weight_block_size)

    @classmethod
    def get_min_capability(cls) -> int:
        return 100

    def process_weights_after_loading(self, layer) -> None:
        weight = layer.weight.data if hasattr(layer.weight, "data") else layer.weight
        sf = layer.weight_scale.data if hasattr(layer.weight_scale, "data") else layer.weight_scale
        N, K = int(weight.shape[0]), int(weight.shape[1])
        select_backend(strategy=self.strategy, weight_block_size=self.weight_block_size, local_n=N, local_k=K)
        kb = -(-K // 128)
        if "BLOCK" in self.strategy:
            scale, block_h = sf.to(torch.float16).contiguous(), 128
        elif "TENSOR" in self.strategy:
            widths = list(getattr(layer, "logical_widths", [N]))
            s = sf.to(torch.float16).reshape(-1)
            if s.numel() == 1 and len(widths) > 1:
                s = s.repeat(len(widths))
            if s.numel() != len(widths) or sum(widths) != N:
                raise ValueError(f"tensor-scale layout mismatch: {s.numel()} scales, widths {widths}, N={N}")
            per_row = torch.repeat_interleave(s, torch.tensor(widths, device=s.device))
            scale, block_h = per_row.reshape(N, 1).expand(N, kb).contiguous(), 1
        else:  # CHANNEL
            s = sf.to(torch.float16)
            if s.numel() == N:
                s = s.reshape(N, 1)
            elif s.numel() == 1:
                s = s.reshape(1, 1).expand(N, 1)
            else:
                raise ValueError(f"unexpected weight_scale numel={s.numel()} for strategy={self.strategy} (N={N}); "
                                 "refusing to dequant unsafely")
            scale, block_h = s.expand(N, kb).contiguous(), 1
        _check_scale_range(scale, getattr(layer, "prefix", "linear"))
        _set(layer, "weight", weight.contiguous())
        _set(layer, "weight_scale", scale)
        layer._b200_block_h = block_h
        layer._b200_NK = (N, K)
        layer.input_scale = None
        if observability.selfcheck_enabled():
            observability.selfcheck_linear(layer.weight, layer.weight_scale, N, K, block_h, getattr(layer, "prefix", "linear"))

    def apply_weights(self, layer, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        N, K = layer._b200_NK
        return _apply_2d(layer, x, bias, N, K, layer.weight_scale, layer._b200_block_h)
