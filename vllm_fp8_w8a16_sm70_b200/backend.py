"""Backend selector of the reference, collapsed onto the one B200 engine.

The reference chooses per weight between "ours" (CUDA-core / WMMA kernels) and the vendored
TurboMind engine from ``VLLM_V100_FP8_BACKEND`` and an eligibility predicate
(``src/fp8_w8a16_sm70/turbomind_fp8_backend.py:142-209``).  Here there is one engine, so every
weight the kernels cover is eligible and the selector returns the constant ``"b200"``.  The
environment variable is still read and validated (a drop-in launcher keeps working); its value
does not change the result.  What the selector still decides is whether a weight is SUPPORTED,
and it fails loudly when it is not, exactly like the reference's ``turbomind`` mode does for an
ineligible weight (``turbomind_fp8_backend.py:198-202``) — never a silent fallback.
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

BLOCK = 128
ENGINE = "b200"
_VALID_MODES = ("ours", "turbomind", "auto")


def backend_mode() -> str:
    """Resolved VLLM_V100_FP8_BACKEND (ours|turbomind|auto); default auto.  Accepted, ignored."""
    m = os.environ.get("VLLM_V100_FP8_BACKEND", "auto").strip().lower()
    return m if m in _VALID_MODES else "auto"


def engine_supports(*, strategy: str, weight_block_size: Optional[Tuple[int, int]], local_n: int,
                    local_k: int) -> Tuple[bool, str]:
    """(supported, reason) for a per-rank weight [local_n, local_k]."""
    strat = (strategy or "").upper()
    if local_n <= 0 or local_k <= 0:
        return False, f"degenerate dims [{local_n},{local_k}]"
    if local_k % 16 != 0:
        return False, f"K={local_k} is not a multiple of 16 (TMA row pitch)"
    if "BLOCK" in strat:
        if weight_block_size is None or tuple(weight_block_size) != (BLOCK, BLOCK):
            return False, f"weight_block_size={weight_block_size} != (128,128)"
        return True, "block-128"
    if "CHANNEL" in strat:
        return True, "per-channel scale as block_h=1 grid"
    if "TENSOR" in strat:
        return True, "per-tensor scale expanded to per-channel"
    return False, f"unknown strategy {strategy!r}"


def select_backend(*, strategy: str, weight_block_size: Optional[Tuple[int, int]], local_n: int, local_k: int,
                   need_moe: bool = False, mode: Optional[str] = None, has_ops: Optional[bool] = None,
                   quiet: bool = True) -> Tuple[str, str]:
    """Same signature as the reference's ``select_backend``; returns (``"b200"``, reason) or raises
    RuntimeError for a weight the engine does not cover.  ``mode``/``has_ops``/``need_moe`` are
    accepted for call-site compatibility and do not influence the result."""
    mode = mode or backend_mode()
    if mode not in _VALID_MODES:
        raise ValueError(f"invalid backend mode {mode!r}")
    ok, reason = engine_supports(strategy=strategy, weight_block_size=weight_block_size, local_n=local_n, local_k=local_k)
    if not ok:
        raise RuntimeError(f"FP8 W8A16 engine cannot serve this weight: {reason}. Refusing to fall back silently.")
    if not quiet:
        print(f"[fp8-backend] backend={ENGINE} [{reason}] dims=[{local_n},{local_k}] moe={need_moe} "
              f"(VLLM_V100_FP8_BACKEND={mode} accepted, one engine)", flush=True)
    return ENGINE, reason
