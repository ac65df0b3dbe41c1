"""Dequantised-weight oracle (test infrastructure): FP8 bytes + scales -> FP16.

The reference defines the dequantised weight as ONE FP16 multiply of the
converted byte with the scale rounded to FP16:

* CUDA:  ``out[i,j] = __hmul(cvt(W[i,j]), S[i/bh, j/bw])``
  (``src/fp8_w8a16_sm70/fp8_dequant.cu:113-127``; per-group variant ``:94-106``)
* torch: ``w.to(fp16) * scale.to(fp16).repeat_interleave(bh,0)
  .repeat_interleave(bw,1)[:N,:K]``
  (``src/fp8_w8a16_sm70/compressed_tensors_v100.py:231-270``; the test twin is
  ``tests/test_attention_shapes.py:104-120``).

Scales arriving as fp32 / bf16 are rounded to FP16 first, as the reference does
at load (``src/fp8_w8a16_sm70/vllm_serve.py:1512-1513``).  A NaN byte stays the
FP16 NaN 0x7F80 with its sign, which is what torch's CPU path returns.
"""

from __future__ import annotations

import numpy as np

from .e4m3 import e4m3_to_fp16_bits


def scales_to_fp16(scales) -> np.ndarray:
    """fp32/bf16/fp16 scale grid -> float16 (round to nearest even)."""
    try:
        import torch
        if isinstance(scales, torch.Tensor):
            return scales.detach().cpu().to(torch.float16).numpy()
    except ImportError:  # pragma: no cover
        pass
    return np.asarray(scales).astype(np.float16)


def expand_scales(s16: np.ndarray, N: int, K: int, block_h: int, block_w: int) -> np.ndarray:
    """[ceil(N/bh), ceil(K/bw)] -> [N, K] by block broadcast."""
    s16 = np.asarray(s16, dtype=np.float16).reshape(-(-N // block_h), -(-K // block_w))
    ii = np.arange(N) // block_h
    jj = np.arange(K) // block_w
    return s16[ii][:, jj]


def dequant_block_scaled(w_u8, scales, N: int, K: int, block_h: int = 128, block_w: int = 128) -> np.ndarray:
    """``[N,K]`` uint8 + ``[Nb,Kb]`` scales -> float16 ``[N,K]``, bit-exact contract."""
    w = np.asarray(w_u8, dtype=np.uint8).reshape(N, K)
    s = expand_scales(scales_to_fp16(scales), N, K, block_h, block_w)
    v = e4m3_to_fp16_bits(w).view(np.float16)
    with np.errstate(invalid="ignore", over="ignore"):
        out = (v * s).astype(np.float16)
    nan_in = (w & 0x7F) == 0x7F
    if nan_in.any():
        bits = out.view(np.uint16).copy()
        bits[nan_in] = ((w[nan_in].astype(np.uint16) & 0x80) << 8) | np.uint16(0x7F80)
        out = bits.view(np.float16)
    return out


def dequant_group_scaled(w_u8, scales, group_size: int) -> np.ndarray:
    """Flat per-group variant, fp8_dequant.cu:94-106: ``out[i]=cvt(w[i])*s[i//g]``."""
    w = np.asarray(w_u8, dtype=np.uint8).reshape(-1)
    s = scales_to_fp16(scales).reshape(-1)[np.arange(w.size) // group_size]
    with np.errstate(invalid="ignore", over="ignore"):
        return (e4m3_to_fp16_bits(w).view(np.float16) * s).astype(np.float16)


def channel_scales_as_blocks(scales, N: int, K: int) -> np.ndarray:
    """Channel scale ``[N,1]`` -> ``[N, ceil(K/128)]`` "fake block" grid with
    block_h = 1 (compressed_tensors_v100.py:488-492)."""
    s = scales_to_fp16(scales).reshape(N, 1)
    return np.ascontiguousarray(np.broadcast_to(s, (N, -(-K // 128))))


def tensor_scales_as_channel(scales, logical_widths) -> np.ndarray:
    """Per-partition tensor scales of a fused module -> one scale per output
    row, the way ``convert_to_channelwise`` is used at
    compressed_tensors_v100.py:247-256 (each logical shard's scalar is repeated
    over that shard's rows)."""
    s = scales_to_fp16(scales).reshape(-1)
    widths = list(logical_widths)
    if s.size == 1 and len(widths) > 1:
        s = np.repeat(s, len(widths))
    assert s.size == len(widths), (s.size, widths)
    return np.concatenate([np.full((w,), s[i], dtype=np.float16) for i, w in enumerate(widths)]).reshape(-1, 1)
