"""Dense W8A16 linear oracle (test infrastructure).

Two restatements:

* ``reference_cpu_linear`` — the reference's own CPU-capable path: dequantise
  the whole weight to FP16, then ``F.linear`` on FP16 tensors
  (``src/fp8_w8a16_sm70/compressed_tensors_v100.py:231-270`` + ``:568-572``).
  This is also what the benchmark times as the CPU baseline.
* ``oracle_linear_fp32`` — the reference tests' definition of correct:
  ``A.float() @ W_dq.float().T`` with the FP16 dequantised weight
  (``tests/test_phase5_matmul.py:88-175``, ``tests/test_attention_shapes.py:104-120``),
  accumulated in fp32 (or fp64 on request).

``check_linear`` applies the acceptance bar: max-abs-err <= 2e-3 * ||x||inf *
sqrt(K) and relative RMS error <= 1e-2 against the fp32-accumulate oracle.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from .dequant import dequant_block_scaled

MAX_ABS_COEF = 2e-3     # max-abs-err <= MAX_ABS_COEF * ||x||inf * sqrt(K)
REL_RMS_TOL = 1e-2      # ||y - ref||_2 / ||ref||_2


def dequant_weight_torch(w_u8: torch.Tensor, scales: torch.Tensor, block_h: int, block_w: int) -> torch.Tensor:
    """torch restatement of compressed_tensors_v100.py:244-246 (block) and
    :257-263 (channel, as block_h = 1 with a [N, Kb] grid or [N,1])."""
    N, K = w_u8.shape
    wf = w_u8.view(torch.float8_e4m3fn).to(torch.float16)
    sf = scales.to(torch.float16)
    if sf.dim() == 1:
        sf = sf.reshape(-(-N // block_h), -1)
    if sf.shape[1] == 1 and block_h == 1:
        scale_exp = sf.reshape(N, 1)
    else:
        scale_exp = sf.repeat_interleave(block_h, dim=0).repeat_interleave(block_w, dim=1)[:N, :K]
    return (wf * scale_exp).to(torch.float16).contiguous()


def reference_cpu_linear(x: torch.Tensor, w_u8: torch.Tensor, scales: torch.Tensor,
                         block_h: int = 128, block_w: int = 128, bias=None):
    """The reference's dequant-then-matmul CPU path.  Returns (y_fp16, W_dq_fp16)."""
    w_dq = dequant_weight_torch(w_u8, scales, block_h, block_w)
    y = torch.nn.functional.linear(x.to(torch.float16), w_dq, None if bias is None else bias.to(torch.float16))
    return y, w_dq


def oracle_linear_fp32(x: torch.Tensor, w_u8: torch.Tensor, scales, block_h: int = 128, block_w: int = 128,
                       accumulate: torch.dtype = torch.float32) -> torch.Tensor:
    """fp32- (or fp64-) accumulate oracle on the bit-exact FP16 dequantised weight."""
    N, K = w_u8.shape
    w_dq = torch.from_numpy(dequant_block_scaled(w_u8.cpu().numpy(), scales, N, K, block_h, block_w).copy())
    return x.cpu().to(accumulate) @ w_dq.to(accumulate).T


def error_stats(y: torch.Tensor, ref: torch.Tensor) -> dict:
    y = y.detach().cpu().double()
    ref = ref.detach().cpu().double()
    diff = y - ref
    return {
        "max_abs": float(diff.abs().max()) if diff.numel() else 0.0,
        "rel_rms": float(diff.norm() / ref.norm().clamp_min(1e-30)) if diff.numel() else 0.0,
        "finite": bool(torch.isfinite(y).all()),
    }


def linear_bounds(x: torch.Tensor, K: int) -> dict:
    xinf = float(x.detach().abs().max().cpu()) if x.numel() else 0.0
    return {"max_abs": MAX_ABS_COEF * xinf * math.sqrt(K), "rel_rms": REL_RMS_TOL}


def check_linear(y: torch.Tensor, x: torch.Tensor, ref_fp32: torch.Tensor, K: int) -> dict:
    """Raises AssertionError if y misses the acceptance bar; returns the stats."""
    st = error_stats(y, ref_fp32)
    bd = linear_bounds(x, K)
    assert st["finite"], "non-finite output"
    assert st["max_abs"] <= bd["max_abs"], f"max_abs {st['max_abs']:.4g} > bound {bd['max_abs']:.4g}"
    assert st["rel_rms"] <= bd["rel_rms"], f"rel_rms {st['rel_rms']:.4g} > {bd['rel_rms']}"
    return st


def quantize_block_fp8(w: torch.Tensor, block_h: int = 128, block_w: int = 128):
    """Synthetic-checkpoint recipe of the benchmark configs: per block
    ``s = max|block| / 448`` (fp32) and ``Wq = (W / s).to(float8_e4m3fn)``.
    block_h = 1 gives per-output-channel... per (row, 128-col) blocks; use
    ``quantize_channel_fp8`` for one scale per row.  Returns (uint8 [N,K], fp32 [Nb,Kb])."""
    N, K = w.shape
    Nb, Kb = -(-N // block_h), -(-K // block_w)
    wp = torch.zeros(Nb * block_h, Kb * block_w, dtype=torch.float32)
    wp[:N, :K] = w.float()
    blocks = wp.reshape(Nb, block_h, Kb, block_w)
    s = blocks.abs().amax(dim=(1, 3)) / 448.0
    s = torch.where(s > 0, s, torch.ones_like(s))
    q = (blocks / s[:, None, :, None]).reshape(Nb * block_h, Kb * block_w)[:N, :K]
    q8 = q.to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    return q8, s.contiguous()


def quantize_channel_fp8(w: torch.Tensor):
    """One fp32 scale per output row: ``s = max|row| / 448``.  Returns (uint8 [N,K], fp32 [N,1])."""
    s = w.float().abs().amax(dim=1, keepdim=True) / 448.0
    s = torch.where(s > 0, s, torch.ones_like(s))
    q8 = (w.float() / s).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    return q8, s.contiguous()


def numtest_weights(N: int, K: int, gen: torch.Generator, block_h: int = 128, block_w: int = 128):
    """Seeded recipe of the reference's synthetic numtests
    (tools/qwen27b_fp8_coalesced_numtest.py:24-106): ``W ~ N(0,1)*0.1``,
    scales ``U(0.01,0.03)`` fp16, ``Wq = (W / s).to(float8_e4m3fn)``."""
    Nb, Kb = -(-N // block_h), -(-K // block_w)
    s = (torch.rand(Nb, Kb, generator=gen) * 0.02 + 0.01).to(torch.float16)
    w = torch.randn(N, K, generator=gen) * 0.1
    se = s.float().repeat_interleave(block_h, 0).repeat_interleave(block_w, 1)[:N, :K]
    q8 = (w / se).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    return q8, s


def np_u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().numpy()
