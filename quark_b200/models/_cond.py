"""Host-side conditioning tables, computed once per model in numpy f32.

Same arithmetic as the reference, which also does this on the host
(``src/quark/models/_waypoint_15_io.py:385-478``): the noise embedding per scheduler sigma,
then per block six projected rows ``(s0, b0, g0, s1, b1, g1)`` and the output-norm pair; rows are
narrowed to bf16 by truncation like every host-to-device upload of the reference.
"""

from __future__ import annotations

import math

import numpy as np


def _silu(x):
    return x * (1.0 / (1.0 + np.exp(-x)))


def _bf16(a) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(u16) -> np.ndarray:
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def noise_embedding(sigmas, fourier_dim: int, w1_f32, w2_f32) -> np.ndarray:
    """``[n_sigma, d]`` f32: Fourier features of ``1000 * sigma`` -> fc1 -> SiLU -> fc2."""
    half = fourier_dim // 2
    freqs = np.array([10000.0 ** (-i / max(half - 1, 1)) for i in range(half)], dtype=np.float32)
    fourier = np.zeros((len(sigmas), 2 * half), dtype=np.float32)
    for i, s in enumerate(sigmas):
        phase = np.array([float(s) * 1000.0 * f for f in freqs], dtype=np.float32)
        fourier[i, :half] = math.sqrt(2.0) * np.sin(phase)
        fourier[i, half:] = math.sqrt(2.0) * np.cos(phase)
    h = fourier @ w1_f32.T
    return _silu(h) @ w2_f32.T


def block_rows(emb_f32, attn_bias_f32, mlp_bias_f32, proj_ws_f32):
    """Six bf16 ``[1, d]`` rows for one sigma: projections 0-2 of the attention head, 3-5 of the MLP head."""
    h_attn = _silu(emb_f32 + attn_bias_f32)
    h_mlp = _silu(emb_f32 + mlp_bias_f32)
    return tuple(_bf16(((h_attn if j < 3 else h_mlp) @ proj_ws_f32[j].T).reshape(1, -1).astype(np.float32)) for j in range(6))


def out_norm_rows(emb_f32, on_w_f32):
    """``(scale_row, bias_row)`` bf16 of the output norm: ``silu(emb) @ W.T`` split in two halves."""
    d = emb_f32.shape[0]
    ab = _silu(emb_f32) @ on_w_f32.T
    return _bf16(ab[:d].reshape(1, d).astype(np.float32)), _bf16(ab[d:].reshape(1, d).astype(np.float32))
