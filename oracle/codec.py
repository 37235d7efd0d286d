"""Carrier-type codecs of the oracle (test infrastructure, see ``oracle/__init__.py``).

bf16 travels as ``uint16`` and e4m3 as ``uint8``, as in the reference's
``src/quark/runtime/npconv.py``:

* ``bf16_to_f32``      follows ``npconv.py:26-31``  (widen by a 16-bit shift)
* ``f32_to_bf16``      follows ``npconv.py:34-42``  (narrow by TRUNCATION, not rounding)
* ``e4m3_to_f32``      follows ``npconv.py:50-62``  (OCP E4M3FN, 0x7F / 0xFF are NaN)
* ``f32_to_e4m3``      follows ``npconv.py:109-148`` (round-to-nearest-even, saturate to 448)

``f32_to_e4m3`` is vectorised; the reference encoder is a per-element Python loop.  The
reference has one quirk: a subnormal whose mantissa rounds up to 8 is masked with ``& 0x7``
(``npconv.py:126-130``), so inputs in ``[0.0146484375, 2**-6)`` encode as 0 rather than
as 0x08 (the smallest normal), which is what round-to-nearest and the hardware
``cvt.rn.satfinite.e4m3x2.f32`` give.  ``reference_quirk=True`` reproduces the reference
byte for byte; the default (False) is the IEEE/hardware behaviour the CUDA kernels follow.
"""

from __future__ import annotations

import numpy as np

E4M3_MAX = 448.0
QUIRK_LO = 0.0146484375  # 7.5 * 2**-9: the lowest value that rounds up to mantissa 8
QUIRK_HI = 2.0**-6


def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


_BF16_MODE = "trunc"


class bf16_rounding:
    """``with bf16_rounding("rne"):`` makes every f32 -> bf16 narrowing of the oracle round to nearest
    even, the rule of the hardware ``cvt.rn.bf16.f32`` that the reference's GPU kernels and ours use.
    The default ("trunc") is what the reference's numpy oracles do.  Truncation shrinks every result by
    half an ulp on average, a bias that accumulates along a chain of ops; comparing a chained GPU run
    against both variants separates that bias from kernel error."""

    def __init__(self, mode: str):
        if mode not in ("trunc", "rne"):
            raise ValueError(mode)
        self.mode = mode

    def __enter__(self):
        global _BF16_MODE
        self.prev, _BF16_MODE = _BF16_MODE, self.mode
        return self

    def __exit__(self, *exc):
        global _BF16_MODE
        _BF16_MODE = self.prev
        return False


def f32_to_bf16(arr: np.ndarray) -> np.ndarray:
    """Truncating narrow, as the reference oracle does (unless ``bf16_rounding("rne")`` is active)."""
    if _BF16_MODE == "rne":
        return f32_to_bf16_rne(arr)
    f32 = np.ascontiguousarray(arr, dtype=np.float32)
    return (f32.view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def f32_to_bf16_rne(arr: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even narrow (what ``cvt.rn.bf16.f32`` does); used for tolerance reasoning only."""
    f32 = np.ascontiguousarray(arr, dtype=np.float32)
    u = f32.view(np.uint32).astype(np.uint64)
    nan = np.isnan(f32)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FC0
    return r


def _decode_e4m3_byte(b: int) -> float:
    sign = (b >> 7) & 1
    exp = (b >> 3) & 0xF
    mant = b & 7
    if exp == 0xF and mant == 7:
        return float("nan")
    val = (mant / 8.0) * 2.0**-6 if exp == 0 else (1.0 + mant / 8.0) * 2.0 ** (exp - 7)
    return -val if sign else val


_E4M3_LUT = np.array([_decode_e4m3_byte(b) for b in range(256)], dtype=np.float32)


def e4m3_to_f32(u8: np.ndarray) -> np.ndarray:
    return _E4M3_LUT[np.asarray(u8, dtype=np.uint8)]


def f32_to_e4m3(arr: np.ndarray, *, reference_quirk: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(arr, dtype=np.float32)
    shape = x.shape
    x = x.ravel()
    sign = (x.view(np.uint32) >> np.uint32(31)).astype(np.uint8) << np.uint8(7)
    ax = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)

    nan = np.isnan(x)
    sat = (ax >= E4M3_MAX) & ~nan
    fin = ~nan & ~sat & (ax > 0)

    a = ax[fin]
    _, e = np.frexp(a)  # a = m * 2**e with m in [0.5, 1)
    e = e.astype(np.int64) - 1  # floor(log2(a))
    sub = e < -6
    code = np.zeros(a.shape, dtype=np.int64)

    # subnormal: value = mant * 2**-9
    m_sub = np.rint(a[sub] * 512.0).astype(np.int64)
    if reference_quirk:
        m_sub = m_sub & 7
    code[sub] = m_sub  # mant 8 lands on 0x08, the smallest normal, as it should

    en = e[~sub]
    m_n = np.rint((a[~sub] / np.exp2(en.astype(np.float64)) - 1.0) * 8.0).astype(np.int64)
    carry = m_n == 8
    m_n[carry] = 0
    en = en + carry
    code[~sub] = ((en + 7) << 3) | m_n

    out[fin] = code.astype(np.uint8)
    out[sat] = 0x7E
    out |= sign
    out[nan] = 0x7F
    return out.reshape(shape)


def to_f32(x: np.ndarray, dtype: str) -> np.ndarray:
    """Widen a carrier array to f32 (``npconv.py:166-220`` ``to_f32_numpy``)."""
    if dtype == "bf16":
        return bf16_to_f32(x)
    if dtype == "e4m3":
        return e4m3_to_f32(x)
    return np.asarray(x).astype(np.float32)


def from_f32(x: np.ndarray, dtype: str, *, reference_quirk: bool = False) -> np.ndarray:
    """Narrow f32 to a carrier array (``npconv.py:228-275`` ``astype_numpy``)."""
    if dtype == "bf16":
        return f32_to_bf16(x)
    if dtype == "e4m3":
        return f32_to_e4m3(x, reference_quirk=reference_quirk)
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    if dtype == "s32":
        return np.rint(x).astype(np.int32)
    raise TypeError(f"unsupported carrier dtype {dtype!r}")


def quirk_band_count(x_f32: np.ndarray) -> int:
    """How many elements fall where the reference encoder and round-to-nearest disagree."""
    ax = np.abs(np.asarray(x_f32, dtype=np.float32))
    return int(np.count_nonzero((ax >= QUIRK_LO) & (ax < QUIRK_HI)))
