"""Load-time self-check and call counters: the cheap production guards the reference keeps around its engine.

* ``selfcheck_linear`` — after a weight has been put into the engine's layout, run the engine on a small random probe
  and compare with the torch dequant-then-matmul of the same tensors on the same device; relative L2 must stay below
  1e-2.  This is the reference's loader guard (``src/fp8_w8a16_sm70/compressed_tensors_v100.py:307-325, 496-517``), with
  one difference: the reference falls back to an FP16 copy of the layer when the check fails, this engine has no
  fallback and raises.  Enabled with ``FP8W8A16_SELFCHECK=1`` (off by default, as a probe GEMM per layer slows loading).
* ``on_apply`` / ``summary`` — per-variant and per-prefix call counters with a periodic one-line summary on rank 0
  (``src/fp8_w8a16_sm70/vllm_serve.py:1403-1429``).  The per-variant numbers come from the library itself
  (``fp8w8a16_variant_counts``), so they also cover calls that did not go through the Python hooks.
  ``FP8W8A16_VARIANT_LOG_EVERY=n`` prints every n calls (0 = never, the default); ``FP8W8A16_PREFIX_PROFILE=1`` adds
  per-layer-prefix call counts.
"""

from __future__ import annotations

import os
import sys
from collections import Counter
from typing import Optional

import torch

from . import _cabi, ops

SELFCHECK_L2REL = 1e-2

_calls = 0
_prefix_calls: Counter = Counter()


def _env_int(name: str, default: int = 0) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


# the hooks call on_apply() on every forward: the environment is read once (reload_env() re-reads it)
_every: Optional[int] = None
_prefix_profile = False


def reload_env() -> None:
    global _every, _prefix_profile
    _every = _env_int("FP8W8A16_VARIANT_LOG_EVERY")
    _prefix_profile = _env_int("FP8W8A16_PREFIX_PROFILE") != 0


def selfcheck_enabled() -> bool:
    return _env_int("FP8W8A16_SELFCHECK") != 0


def selfcheck_linear(weight: torch.Tensor, scale: torch.Tensor, N: int, K: int, block_h: int, what: str = "linear",
                     rows: int = 4) -> float:
    """Engine vs torch dequant-then-matmul on a random probe; returns the relative L2 error, raises above 1e-2."""
    if weight.device.type != "cuda":
        raise RuntimeError(f"{what}: the self-check runs on the GPU the layer lives on (got {weight.device})")
    g = torch.Generator(device=weight.device).manual_seed(1234)
    probe = torch.randn(rows, K, generator=g, device=weight.device, dtype=torch.float32).mul_(0.1).to(torch.float16)
    w8 = weight.view(torch.uint8) if weight.dtype != torch.uint8 else weight
    out = ops.w8a16_linear(probe, w8, scale, N, K, block_h, 128)
    s16 = scale.to(torch.float16).reshape(-(-N // block_h), -(-K // 128))
    ref_rows = []
    step = 4096                      # bound the FP16 copy the check materialises
    wf = w8.reshape(N, K).view(torch.float8_e4m3fn)
    for n0 in range(0, N, step):
        n1 = min(N, n0 + step)
        rows_s = s16[n0 // block_h: -(-n1 // block_h)].repeat_interleave(block_h, 0)[: n1 - n0]
        wdq = wf[n0:n1].to(torch.float16) * rows_s.repeat_interleave(128, 1)[:, :K]
        ref_rows.append(probe.float() @ wdq.float().T)
    ref = torch.cat(ref_rows, 1)
    l2 = float((out.float() - ref).norm() / ref.norm().clamp_min(1e-12))
    if not (l2 < SELFCHECK_L2REL):
        raise RuntimeError(f"{what}: load-time self-check failed (N={N} K={K} block_h={block_h}, relative L2 {l2:.4g} >= "
                           f"{SELFCHECK_L2REL}); refusing to serve this layer")
    return l2


def on_apply(layer=None) -> None:
    """Count one hook call; print the summary every FP8W8A16_VARIANT_LOG_EVERY calls."""
    global _calls
    if _every is None:
        reload_env()
    if _every <= 0:
        return
    every = _every
    _calls += 1
    if _prefix_profile:
        _prefix_calls[getattr(layer, "prefix", "<?>")] += 1
    if _calls % every == 0:
        rank = torch.distributed.get_rank() if torch.distributed.is_available() and torch.distributed.is_initialized() else 0
        if rank == 0:
            print(summary(), file=sys.stderr, flush=True)


def summary() -> str:
    counts = _cabi.variant_counts()
    tot = sum(v for k, v in counts.items() if k != "fused_allreduce") or 1
    parts = [f"{k}={v} ({100.0 * v / tot:.0f}%)" for k, v in counts.items() if v]
    line = f"[fp8w8a16_b200 pid={os.getpid()}] kernel variant counts after {_calls} hook calls: {', '.join(parts) or 'none'}"
    if _prefix_calls:
        line += "\n" + "\n".join(f"[fp8w8a16_b200 pid={os.getpid()}] prefix {p}: calls={c}" for p, c in sorted(_prefix_calls.items()))
    return line


def reset() -> None:
    global _calls
    _calls = 0
    _prefix_calls.clear()
