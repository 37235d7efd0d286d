"""Helpers shared by the parity tests: seeded inputs in carrier types and the error metrics.

Tolerances (stated once, used everywhere):
* bytes and indices (cache slots, segment tables, e4m3 encodings of given values): exact;
* bf16 results: max |got - want| / max |want| <= 2e-2 per tensor, and cosine >= 0.999;
* fp8 results: cosine >= 0.999 per tensor against the oracle fed the same quantised operands.
"""

from __future__ import annotations

import numpy as np

from oracle import codec

BF16_MAX_REL = 2e-2
COS_MIN = 0.999


def rng(seed=0):
    return np.random.default_rng(seed)


def bf16_randn(r, shape, scale=1.0):
    return codec.f32_to_bf16((scale * r.standard_normal(shape)).astype(np.float32))


def e4m3_randn(r, shape, scale=1.0):
    return codec.f32_to_e4m3((scale * r.standard_normal(shape)).astype(np.float32))


def f32(x, dtype):
    return codec.to_f32(np.asarray(x), dtype)


def max_rel(got_f32, want_f32) -> float:
    den = float(np.max(np.abs(want_f32)))
    return float(np.max(np.abs(got_f32 - want_f32))) / (den if den > 0 else 1.0)


def cosine(got_f32, want_f32) -> float:
    a = got_f32.astype(np.float64).ravel()
    b = want_f32.astype(np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na == 0 and nb == 0:
        return 1.0
    return float(a @ b / (na * nb)) if na > 0 and nb > 0 else 0.0


def assert_close_bf16(got_u16, want_u16, what="", max_rel_tol=BF16_MAX_REL, cos_min=COS_MIN):
    g, w = f32(got_u16, "bf16"), f32(want_u16, "bf16")
    assert np.all(np.isfinite(g)), f"{what}: non-finite values in the result"
    mr, cs = max_rel(g, w), cosine(g, w)
    assert mr <= max_rel_tol and cs >= cos_min, f"{what}: max_rel={mr:.3e} cosine={cs:.6f}"
    return mr, cs


def bf16_ulp_diff(a_u16, b_u16):
    """Distance in bf16 units in the last place between two carrier arrays (sign-magnitude aware)."""

    def key(u):
        u = u.astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)

    return np.abs(key(np.asarray(a_u16)) - key(np.asarray(b_u16)))


def parity_report(rec: dict) -> None:
    """Print one achieved-parity record as a JSON line; with ``QB_PARITY_REPORT`` naming a file, append it there too."""
    import json
    import os

    print(json.dumps(rec))
    path = os.environ.get("QB_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(rec) + "\n")
