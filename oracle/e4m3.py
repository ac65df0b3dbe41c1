"""E4M3-FN byte -> FP16 bit pattern, restated in numpy (test infrastructure).

Follows ``src/fp8_w8a16_sm70/fp8_dequant.cu:44-50`` (``fp8_e4m3_to_fp16_bits``):
the seven magnitude bits are shifted into FP16 position (``mag << 7``), the
result is re-biased with one FP16 multiply by 2**8, the single NaN encoding
(magnitude 0x7F) becomes 0x7F80 and the sign bit is OR-ed back in.  The
reference pins this against torch's CPU ``uint8.view(float8_e4m3fn)
.to(float16)`` for all 256 bytes (``tests/test_fp8.py:160-179``).
"""

from __future__ import annotations

import numpy as np

# tests/test_fp8.py:119-134 — the reference's hand-picked known answers,
# written here as (byte, value); NaN entries carry None.
EDGE_CASES = (
    (0x00, 0.0), (0x80, -0.0), (0x38, 1.0), (0xB8, -1.0), (0x3C, 1.5),
    (0x40, 2.0), (0x30, 0.5), (0x7E, 448.0), (0xFE, -448.0),
    (0x01, 2.0 ** -9), (0x07, 7 * 2.0 ** -9), (0x87, -7 * 2.0 ** -9),
    (0x7F, None), (0xFF, None),
)


def e4m3_to_fp16_bits(b: np.ndarray) -> np.ndarray:
    """uint8 array -> uint16 array of FP16 bit patterns (fp8_dequant.cu:44-50)."""
    b = np.asarray(b, dtype=np.uint8)
    sign = (b.astype(np.uint16) & np.uint16(0x80)) << np.uint16(8)
    mag = b.astype(np.uint16) & np.uint16(0x7F)
    shifted = (mag << np.uint16(7)).astype(np.uint16)
    h = (shifted.view(np.float16) * np.float16(256.0)).astype(np.float16)
    val = np.where(mag == 0x7F, np.uint16(0x7F80), h.view(np.uint16))
    return (sign | val).astype(np.uint16)


def e4m3_to_fp16(b: np.ndarray) -> np.ndarray:
    """uint8 array -> float16 array."""
    return e4m3_to_fp16_bits(b).view(np.float16)


def table_bits() -> np.ndarray:
    """All 256 bytes, as FP16 bit patterns."""
    return e4m3_to_fp16_bits(np.arange(256, dtype=np.uint8))


def e4m3_to_float_by_definition(b: int) -> float:
    """One byte decoded from the E4M3-FN format definition
    (fp8_dequant.cu:6-13: sign 1, exponent 4 bias 7, mantissa 3; no inf;
    0x7F/0xFF NaN).  Independent of the bit trick above; pure Python."""
    s = -1.0 if (b & 0x80) else 1.0
    e = (b >> 3) & 0xF
    m = b & 0x7
    if e == 0xF and m == 0x7:
        return float("nan")
    if e == 0:
        return s * m * 2.0 ** -9
    return s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
