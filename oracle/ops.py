"""Per-kernel CPU references (test infrastructure, see ``oracle/__init__.py``).

Each function restates one of the reference's numpy oracles; the citation names the file and
lines (paths relative to the reference project) it follows.  All arithmetic is f32 unless
noted, tensors travel in the carrier types of ``oracle/codec.py``.
"""

from __future__ import annotations

import math

import numpy as np

from .codec import from_f32, to_f32

# ---------------------------------------------------------------------------
# ortho-RoPE tables
# ---------------------------------------------------------------------------


def _pixel_freqs(n: int, max_freq: float) -> np.ndarray:
    # src/quark/kernels/kv_cache_update/reference.py:50-51 (f64 on purpose: linspace * pi)
    return np.linspace(1.0, max_freq / 2, n) * math.pi


def _lang_freqs(dim: int, theta: float = 10000.0) -> np.ndarray:
    # src/quark/kernels/kv_cache_update/reference.py:52-55 (f32 exponents -> f32 frequencies)
    exponents = np.arange(0, dim, 2, dtype=np.float32) / dim
    freqs = 1.0 / (theta**exponents)
    return freqs[: dim // 2]


def rope_spatial_angles(H: int, W: int, Dh: int = 64) -> np.ndarray:
    """f32 angles ``[H*W, Dh//4]`` of the x and y parts of the table, for any frame.

    Follows ``_make_ortho_rope_freqs`` (src/quark/kernels/kv_cache_update/reference.py:61-106):
    positions are an f64 linspace narrowed to f32, multiplied by f64 pixel frequencies, each
    frequency repeated twice, the result narrowed to f32 when the table is concatenated.
    """
    if H <= 0 or W <= 0 or Dh <= 0:
        raise ValueError(f"H, W and Dh must be > 0; got H={H}, W={W}, Dh={Dh}")
    max_freq = min(H, W) * 0.8
    fx = np.linspace(-1 + 1 / W, 1 - 1 / W, W).astype(np.float32)[..., None] * _pixel_freqs(Dh // 16, max_freq)
    fy = np.linspace(-1 + 1 / H, 1 - 1 / H, H).astype(np.float32)[..., None] * _pixel_freqs(Dh // 16, max_freq)
    fx = np.repeat(fx, 2, axis=-1)[None, :, :]  # [1, W, Dh/8]
    fy = np.repeat(fy, 2, axis=-1)[:, None, :]  # [H, 1, Dh/8]
    fx = np.broadcast_to(fx, (H, W, fx.shape[-1])).reshape(H * W, -1)
    fy = np.broadcast_to(fy, (H, W, fy.shape[-1])).reshape(H * W, -1)
    return np.concatenate([fx, fy], axis=-1).astype(np.float32)


def rope_temporal_angles(frame_t: int, Dh: int = 64) -> np.ndarray:
    """f32 angles ``[Dh//4]`` of the temporal part for one frame (reference.py:93-97)."""
    raw = np.asarray([frame_t]).astype(np.float32)[..., None] * _lang_freqs(Dh // 4)
    return np.repeat(raw, 2, axis=-1).reshape(-1).astype(np.float32)


def rope_tables(H: int, W: int, frame_t: int, Dh: int = 64):
    """``(cos, sin)`` of shape ``[H*W, Dh//2]`` for frame ``frame_t`` only.

    The reference builds the table for frames ``0..frame_t`` and slices the last frame
    (reference.py:189-191); the rows of one frame do not depend on the others.
    """
    sp = rope_spatial_angles(H, W, Dh)
    tm = np.broadcast_to(rope_temporal_angles(frame_t, Dh)[None, :], (H * W, Dh // 4))
    ang = np.concatenate([sp, tm], axis=-1).astype(np.float32)
    return np.cos(ang), np.sin(ang)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Pairs ``(x[2i], x[2i+1])``, output de-interleaved ``cat([y0, y1])`` (reference.py:31-41)."""
    x32 = x.astype(np.float32, copy=False)
    x0 = x32[..., 0::2]
    x1 = x32[..., 1::2]
    y0 = x0 * cos - x1 * sin
    y1 = x1 * cos + x0 * sin
    return np.concatenate([y0, y1], axis=-1)


# ---------------------------------------------------------------------------
# KV-cache append
# ---------------------------------------------------------------------------


def compute_segments(frame_t: int, num_buckets: int, tpf: int, pinned_dilation: int, max_segments: int = 3):
    """Segment table after the append at ``frame_t`` (reference.py:109-140).

    Returns ``(segments s32[max_segments*2], n_segments int)``.
    """
    L = num_buckets * tpf
    bucket = (frame_t + pinned_dilation - 1) // pinned_dilation
    is_write = (frame_t % pinned_dilation) == 0
    post_wrap = bucket >= num_buckets
    slot = bucket % num_buckets
    if post_wrap and is_write:
        rows = [[0, slot * tpf], [(slot + 1) * tpf, (num_buckets - slot - 1) * tpf], [L, tpf]]
        n = 3
    else:
        rows = [[0, min(bucket, num_buckets) * tpf], [L, tpf]]
        n = 2
    rows.extend([[0, 0]] * (max_segments - len(rows)))
    return np.array(rows, dtype=np.int32).reshape(-1), n


def kv_cache_update(
    qkv,
    frame_t: int,
    frozen: int,
    *,
    n_kv_heads: int,
    n_q_heads: int,
    H_spatial: int,
    W_spatial: int,
    num_buckets: int,
    pinned_dilation: int,
    kv_dtype: str = "bf16",
    Dh: int = 64,
    K_cache=None,
    Vt_cache=None,
    max_segments: int = 3,
    reference_quirk: bool = False,
    quilt_factor: int = 1,
    quilt_offset: int = 0,
    k_scale=None,
    v_scale=None,
):
    """Packed-QKV cache append (src/quark/kernels/kv_cache_update/reference.py:148-251), B = 1.

    ``k_scale`` / ``v_scale`` (f32 ``[n_kv_heads]``, an extension: the reference is scale free) restate the scaled
    caches: ``narrow(RoPE(K) * (1 / k_scale[h]))`` and ``narrow(V * (1 / v_scale[h]))``, reciprocal and product in f32.

    ``qkv`` is ``[tpf, (Hq + 2 Hk) * Dh]`` bf16.  When ``K_cache`` / ``Vt_cache`` are given
    they are updated in place (the read-modify-write the GPU kernel does); when they are
    None fresh zero caches are returned, which is what the reference function models.
    Returns ``(K_cache [Hk*capacity, Dh], Vt_cache [Hk*Dh, capacity], segments, n_segments)``.
    With ``quilt_factor > 1`` the cache keeps tokens ``quilt_offset::quilt_factor`` of the frame (rotated at their
    own positions first), and capacity, slots and segments are those of ``tpf / quilt_factor`` tokens per frame
    (``reference.py:201-235``).
    """
    tpf_all = H_spatial * W_spatial
    tpf = tpf_all // quilt_factor  # tokens of a frame that the cache keeps
    Hk = n_kv_heads
    L = num_buckets * tpf
    cap = L + tpf
    x = to_f32(qkv, "bf16")
    k0 = n_q_heads * Dh
    v0 = (n_q_heads + n_kv_heads) * Dh
    K4 = x[:, k0 : k0 + Hk * Dh].reshape(tpf_all, Hk, Dh).transpose(1, 0, 2)  # [Hk, tpf, Dh]
    V4 = x[:, v0 : v0 + Hk * Dh].reshape(tpf_all, Hk, Dh).transpose(1, 0, 2)
    cos, sin = rope_tables(H_spatial, W_spatial, frame_t, Dh)
    k_rot = apply_rope(K4, cos[None], sin[None])
    V4 = np.ascontiguousarray(V4)
    if k_scale is not None:
        k_rot = (k_rot.astype(np.float32) * (np.float32(1.0) / np.asarray(k_scale, np.float32))[:, None, None]).astype(np.float32)
    if v_scale is not None:
        V4 = (V4 * (np.float32(1.0) / np.asarray(v_scale, np.float32))[:, None, None]).astype(np.float32)
    k_c = from_f32(k_rot, kv_dtype, reference_quirk=reference_quirk)[:, quilt_offset::quilt_factor, :]
    v_c = from_f32(np.ascontiguousarray(V4), kv_dtype, reference_quirk=reference_quirk)[:, quilt_offset::quilt_factor, :]

    carrier = np.uint16 if kv_dtype == "bf16" else np.uint8
    if K_cache is None:
        K_cache = np.zeros((Hk * cap, Dh), dtype=carrier)
    if Vt_cache is None:
        Vt_cache = np.zeros((Hk * Dh, cap), dtype=carrier)
    Kc = K_cache.reshape(Hk, cap, Dh)
    Vc = Vt_cache.reshape(Hk, Dh, cap)
    Kc[:, L : L + tpf, :] = k_c
    Vc[:, :, L : L + tpf] = v_c.transpose(0, 2, 1)
    if not frozen and frame_t % pinned_dilation == 0:
        slot = ((frame_t + pinned_dilation - 1) // pinned_dilation) % num_buckets
        Kc[:, slot * tpf : (slot + 1) * tpf, :] = k_c
        Vc[:, :, slot * tpf : (slot + 1) * tpf] = v_c.transpose(0, 2, 1)
    segs, n = compute_segments(frame_t, num_buckets, tpf, pinned_dilation, max_segments)
    return K_cache, Vt_cache, segs, np.array([n], dtype=np.int32)


# ---------------------------------------------------------------------------
# owl_attn
# ---------------------------------------------------------------------------


def segment_mask(segments, n_segments: int, capacity: int) -> np.ndarray:
    """Boolean validity mask ``[capacity]`` (src/quark/kernels/owl_attn/reference.py:29-45)."""
    valid = np.zeros(capacity, dtype=bool)
    segs = np.asarray(segments, dtype=np.int64).reshape(-1, 2)
    for i in range(int(n_segments)):
        st, ln = int(segs[i, 0]), int(segs[i, 1])
        end = min(st + ln, capacity)
        if st < end:
            valid[st:end] = True
    return valid


def owl_attn(
    qkv,
    K_cache,
    Vt_cache,
    segments,
    n_segments,
    frame_t: int,
    *,
    n_kv_heads: int,
    gqa_ratio: int,
    H_spatial: int,
    W_spatial: int,
    kv_dtype: str = "bf16",
    Dh: int = 64,
    packed_qkv: bool = True,
    out_dtype: str = "bf16",
    q_quant: str | None = None,
    return_f32: bool = False,
    k_scale=None,
    v_scale=None,
):
    """Segment-masked GQA attention with Q-side RoPE (owl_attn/reference.py:47-111), B = 1.

    ``k_scale`` / ``v_scale`` (f32 ``[n_kv_heads]``, an extension) restate attention over scaled caches:
    ``S = (Q . Kq^T) * k_scale[h] / sqrt(Dh)``, ``O = (P . Vq) * v_scale[h]``.

    Same arithmetic as the reference (f32 scores, exact softmax, f32 ``P @ V``), evaluated one
    Q head at a time over the valid key columns only: masked columns contribute
    ``exp(-inf) = 0`` in the reference, so dropping them changes no result bit except the order
    of the f32 sums.  ``q_quant="e4m3"`` additionally rounds the rotated Q through e4m3, which
    is what the fp8 compute path of the GPU kernels feeds its MMAs (the reference oracle itself
    keeps Q in f32); it is used only for "same quantised operands" comparisons.
    """
    tpf = H_spatial * W_spatial
    Hk = n_kv_heads
    Hq = Hk * gqa_ratio
    cap = K_cache.shape[0] // Hk
    cos, sin = rope_tables(H_spatial, W_spatial, int(frame_t), Dh)
    q = to_f32(qkv, "bf16")
    if packed_qkv:
        Q4 = q[:, : Hq * Dh].reshape(tpf, Hq, Dh).transpose(1, 0, 2)
    else:
        Q4 = q.reshape(Hq, tpf, Dh)
    Q_rot = apply_rope(Q4, cos[None], sin[None])
    if q_quant is not None:
        Q_rot = to_f32(from_f32(Q_rot, q_quant), q_quant)
    Kc = to_f32(K_cache, kv_dtype).reshape(Hk, cap, Dh)
    Vc = to_f32(Vt_cache, kv_dtype).reshape(Hk, Dh, cap)
    valid = segment_mask(segments, int(np.asarray(n_segments).reshape(-1)[0]), cap)
    idx = np.nonzero(valid)[0]
    out = np.zeros((Hq, tpf, Dh), dtype=np.float32)
    scale = np.float32(1.0 / np.sqrt(Dh))
    if idx.size:
        for h in range(Hq):
            kh = h // gqa_ratio
            Ks = Kc[kh][idx]  # [S, Dh]
            Vs = Vc[kh][:, idx]  # [Dh, S]
            s = (Q_rot[h] @ Ks.T) * (scale if k_scale is None else scale * np.float32(k_scale[kh]))
            m = s.max(axis=-1, keepdims=True)
            ex = np.exp(s - m)
            den = ex.sum(axis=-1, keepdims=True)
            out[h] = (ex / den) @ Vs.T
            if v_scale is not None:
                out[h] *= np.float32(v_scale[kh])
    if packed_qkv:
        res = out.transpose(1, 0, 2).reshape(tpf, Hq * Dh)
    else:
        res = out.reshape(Hq * tpf, Dh)
    return res if return_f32 else from_f32(res, out_dtype)


# ---------------------------------------------------------------------------
# GEMM and its epilogue
# ---------------------------------------------------------------------------


def silu_f32(x: np.ndarray) -> np.ndarray:
    return x * (1.0 / (1.0 + np.exp(-x)))


def gemm(
    A,
    B,
    *,
    a_dtype: str = "bf16",
    b_dtype: str = "bf16",
    out_dtype: str = "bf16",
    bias=None,
    activation: str | None = None,
    gate=None,
    residual=None,
    gate_groups: int = 1,
    a_quant: str | None = None,
    return_f32: bool = False,
    a_scale=None,
    w_scale=None,
):
    """``C = A @ B.T`` with the epilogue order (scales ->) bias -> SiLU -> gate*acc + residual -> cast.

    ``a_scale`` (scalar) / ``w_scale`` (f32 ``[N]``), an extension (the reference's e4m3 GEMM is scale free):
    ``C = (Aq . Wq^T) * (a_scale * w_scale[n])`` before the rest of the epilogue.

    Follows ``src/quark/kernels/gemm/reference.py:18-48``.  The reference keeps A in f32 even
    when the kernel computes in e4m3; ``a_quant="e4m3"`` rounds A through e4m3 first so that a
    GPU fp8 result can be compared against the oracle on the same quantised operands.
    """
    a = to_f32(A, a_dtype)
    if a_quant is not None and a_dtype != a_quant:
        a = to_f32(from_f32(a, a_quant), a_quant)
    b = to_f32(B, b_dtype)
    c = a.reshape(-1, a.shape[-1]) @ b.T
    if a_scale is not None or w_scale is not None:
        sa = np.float32(1.0 if a_scale is None else np.asarray(a_scale, np.float32).reshape(-1)[0])
        col = sa if w_scale is None else (sa * np.asarray(w_scale, np.float32)).reshape(1, -1)
        c = (c * col).astype(np.float32)
    if bias is not None:
        c = c + to_f32(bias, out_dtype).reshape(1, -1)
    if activation == "silu":
        c = silu_f32(c)
    elif activation is not None:
        raise ValueError(f"unsupported activation {activation!r}")
    if gate is not None and residual is not None:
        g = to_f32(gate, out_dtype).reshape(gate_groups, -1)
        r = to_f32(residual, out_dtype)
        c = r + np.repeat(g, c.shape[0] // gate_groups, axis=0) * c
    return c if return_f32 else from_f32(c, out_dtype)


def quantize_e4m3(X, src_dtype: str = "bf16", *, reference_quirk: bool = False):
    """Unscaled RN-even, saturating narrow (src/quark/nn/layers.py:291-304, npconv.py:109-148)."""
    return from_f32(to_f32(X, src_dtype), "e4m3", reference_quirk=reference_quirk)


# ---------------------------------------------------------------------------
# norm / elementwise glue
# ---------------------------------------------------------------------------


def quantize_e4m3_rows(X, src_dtype: str = "bf16"):
    """Per-row scaled narrowing (an extension; no reference counterpart): ``scale[r] = max|X[r]| / 448`` (1 for an
    all-zero row), ``q[r] = e4m3(X[r] * (1 / scale[r]))``, every step in f32.  Returns ``(q u8, scale f32[rows])``."""
    x = to_f32(X, src_dtype)
    amax = np.max(np.abs(x), axis=1).astype(np.float32)
    scale = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    return from_f32((x * inv[:, None]).astype(np.float32), "e4m3"), scale


def ada_rmsnorm(X, scale, bias, *, eps: float = 1e-6, activation: str | None = None, dtype: str = "bf16", return_f32=False):
    """``rmsnorm(x) * (1 + scale) + bias`` (+ SiLU) (src/quark/kernels/ada_rmsnorm/reference.py:10-29)."""
    x = to_f32(X, dtype)
    s = to_f32(scale, dtype).reshape(-1, x.shape[-1])
    b = to_f32(bias, dtype).reshape(-1, x.shape[-1])
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    y = x * inv
    rep = x.shape[0] // s.shape[0]
    y = y * (1.0 + np.repeat(s, rep, axis=0)) + np.repeat(b, rep, axis=0)
    if activation == "silu":
        y = silu_f32(y)
    y = y.astype(np.float32)
    return y if return_f32 else from_f32(y, dtype)


def rmsnorm(X, *, eps: float = 1e-6, dtype: str = "bf16"):
    """``x * rsqrt(mean(x^2, last dim) + eps)``, no gain (src/quark/kernels/rmsnorm/reference.py:10-22; the
    model calls it with eps = 1e-6, src/quark/functional/rmsnorm.py:29)."""
    x = to_f32(X, dtype)
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return from_f32((x * inv).astype(np.float32), dtype)


def add(X, Y, *, dtype: str = "bf16"):
    """``x + y`` (src/quark/kernels/elementwise/reference.py:10-19, op "add")."""
    return from_f32(to_f32(X, dtype) + to_f32(Y, dtype), dtype)


def mlp_fusion(X, cond, w_x, w_c, w_2):
    """``fc2(silu(x @ Wx.T + cond @ Wc.T))`` the way the reference runs it (src/quark/nn/layers.py:797-822):
    the cond projection is a GEMM of its own whose bf16 result is fc1_x's bias row, SiLU is a separate op
    on the bf16 GEMM output.  All bf16."""
    h_c = gemm(cond, w_c).reshape(-1)
    h = silu(gemm(X, w_x, bias=h_c))
    return gemm(h, w_2)


def controller_embedding(ctrl_input, w1, w2):
    """``fc2(silu(fc1(ctrl_input)))`` on the padded controller row (src/quark/nn/layers.py:760-794)."""
    return gemm(silu(gemm(ctrl_input, w1)), w2)


def head_rmsnorm(X, *, n_q_heads: int, n_kv_heads: int, Dh: int = 64, eps: float = 1e-6, dtype: str = "bf16"):
    """Per-head RMS norm of the Q and K columns, V copied (head_rmsnorm/reference.py:10-26)."""
    x = to_f32(X, dtype).copy()
    nh = n_q_heads + n_kv_heads
    seg = x[:, : nh * Dh].reshape(x.shape[0], nh, Dh)
    inv = 1.0 / np.sqrt(np.mean(seg * seg, axis=-1, keepdims=True) + eps)
    x[:, : nh * Dh] = (seg * inv).reshape(x.shape[0], nh * Dh)
    return from_f32(x.astype(np.float32), dtype)


def value_residual_packed(QKV_curr, QKV_first, lamb: float, *, v_col_offset: int, v_width: int, dtype: str = "bf16"):
    """``v += lamb * (v_first - v)`` on the V columns (value_residual_packed/reference.py:8-20)."""
    cur = to_f32(QKV_curr, dtype)
    first = to_f32(QKV_first, dtype)
    lam = np.float32(lamb)
    out = cur.copy()
    sl = slice(v_col_offset, v_col_offset + v_width)
    out[:, sl] = cur[:, sl] + lam * (first[:, sl] - cur[:, sl])
    return from_f32(out, dtype)


def ada_gate_residual(X, Y, gate, *, dtype: str = "bf16"):
    """``x + gate * y`` (src/quark/kernels/ada_gate_residual/reference.py:10-22)."""
    x = to_f32(X, dtype)
    y = to_f32(Y, dtype)
    g = to_f32(gate, dtype).reshape(-1, x.shape[-1])
    return from_f32(x + np.repeat(g, x.shape[0] // g.shape[0], axis=0) * y, dtype)


def silu(X, *, dtype: str = "bf16"):
    """``x * sigmoid(x)`` (src/quark/kernels/silu/reference.py:10-18)."""
    return from_f32(silu_f32(to_f32(X, dtype)), dtype)


def euler_step(X, V, dsig: float, *, dtype: str = "bf16"):
    """``x + dsig * v`` (src/quark/functional/euler_step.py:36-41)."""
    return from_f32(to_f32(X, dtype) + np.float32(dsig) * to_f32(V, dtype), dtype)


def patchify(X, W, *, C: int, H: int, Wd: int, ph: int = 2, pw: int = 2, dtype: str = "bf16"):
    """``[1, C*H*W] -> [Hp*Wp, d_model]`` (src/quark/kernels/patchify/reference.py:8-23)."""
    x = to_f32(X, dtype).reshape(1, C, H // ph, ph, Wd // pw, pw).transpose(0, 2, 4, 1, 3, 5)
    x = x.reshape((H // ph) * (Wd // pw), C * ph * pw)
    return from_f32(x @ to_f32(W, dtype).T, dtype)


def unpatchify(X, W, bias, *, C: int, H: int, Wd: int, ph: int = 2, pw: int = 2, dtype: str = "bf16"):
    """``[Hp*Wp, d_model] -> [1, C*H*W]`` (src/quark/kernels/unpatchify/reference.py:8-24)."""
    h = to_f32(X, dtype) @ to_f32(W, dtype).T
    if bias is not None:
        h = h + to_f32(bias, dtype).reshape(1, -1)
    Hp, Wp = H // ph, Wd // pw
    h = h.reshape(1, Hp, Wp, C, ph, pw).transpose(0, 3, 1, 4, 2, 5)
    return from_f32(np.ascontiguousarray(h).reshape(1, C * H * Wd), dtype)


# ---------------------------------------------------------------------------
# randn: Philox4x32-10 + Box-Muller
# ---------------------------------------------------------------------------


def philox4x32_10(counter, key):
    """Philox4x32 with 10 rounds (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11).

    ``counter``: ``uint32 [..., 4]``, ``key``: ``uint32 [..., 2]`` (broadcast together); returns ``uint32 [..., 4]``.
    The round, multipliers and key schedule are those of the reference's kernel
    (``src/quark/kernels/randn/kernel.py:44-48, 130-147``), which are the published ones."""
    c = np.array(np.broadcast_arrays(*[np.asarray(counter, np.uint64)[..., i] for i in range(4)]))
    k = np.array(np.broadcast_arrays(*[np.asarray(key, np.uint64)[..., i] for i in range(2)]), dtype=np.uint64)
    k = [np.broadcast_to(k[0], c[0].shape).copy(), np.broadcast_to(k[1], c[0].shape).copy()]
    c = [x.copy() for x in c]
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c[0]
        p1 = np.uint64(0xCD9E8D57) * c[2]
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
        k = [(k[0] + np.uint64(0x9E3779B9)) & mask, (k[1] + np.uint64(0xBB67AE85)) & mask]
    return np.stack(c, axis=-1).astype(np.uint32)


def randn(n: int, counter_offset: int = 0, *, seed0: int = 0xDEADBEEF, seed1: int = 0xBADC0FFE, counter_stride: int = 1, dtype: str = "f32"):
    """``n`` standard normals in the order the device kernel writes them.

    Restates ``src/quark/kernels/randn/kernel.py:149-254`` at its default tile (128 threads, 2048 outputs per
    block, ``config.py:11-20``): thread ``t`` of block ``b``, pass ``g`` draws Philox counter
    ``(b * 512 + g * 128 + t + offset, 0, seed0, seed1)`` under the key ``(seed0, seed1)``; word ``x`` becomes the
    uniform ``(x >> 8) * 2^-24 + 2^-25``; words (0, 1) and (2, 3) become two normals each,
    ``sqrt(-2 ln u1) * (cos, sin)(2 pi u2)``; the four land at ``b * 2048 + (4 g + k) * 128 + t``.  The reference has
    no value oracle for this op (``reference.py`` returns zeros: "statistical, not bitwise"), and its kernel uses
    approximate log2 / sqrt / sin / cos, so agreement with any implementation is to a tolerance, not bitwise;
    the integers (Philox words) are exact.  ``counter_stride`` multiplies the offset (1 = the reference)."""
    blocks = (n + 2047) // 2048
    b = np.arange(blocks, dtype=np.uint64)[:, None, None]
    g = np.arange(4, dtype=np.uint64)[None, :, None]
    t = np.arange(128, dtype=np.uint64)[None, None, :]
    off = (int(counter_offset) * int(counter_stride)) & 0xFFFFFFFF
    c0 = ((b * np.uint64(512) + g * np.uint64(128) + t + np.uint64(off)) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    ctr = np.stack([c0, np.zeros_like(c0), np.full_like(c0, seed0 & 0xFFFFFFFF), np.full_like(c0, seed1 & 0xFFFFFFFF)], axis=-1)
    w = philox4x32_10(ctr, np.array([seed0 & 0xFFFFFFFF, seed1 & 0xFFFFFFFF], np.uint32))  # [blocks, 4, 128, 4]
    u = (w >> np.uint32(8)).astype(np.float32) * np.float32(2.0**-24) + np.float32(2.0**-25)
    z = np.empty(u.shape, np.float32)
    for h in range(2):
        r = np.sqrt(np.float32(-2.0) * np.log(u[..., 2 * h].astype(np.float64))).astype(np.float32)
        th = (np.float32(2.0 * np.pi) * u[..., 2 * h + 1]).astype(np.float64)
        z[..., 2 * h] = r * np.cos(th).astype(np.float32)
        z[..., 2 * h + 1] = r * np.sin(th).astype(np.float32)
    # [block, g, t, k] -> position block * 2048 + (4 g + k) * 128 + t
    flat = z.transpose(0, 1, 3, 2).reshape(-1)[:n]
    return from_f32(flat, "bf16") if dtype == "bf16" else flat


# ---------------------------------------------------------------------------
# mixture of experts ("correct" routing)
# ---------------------------------------------------------------------------


def moe_route(logits, top_k: int) -> np.ndarray:
    """Dense routing weights ``[E, M]`` f32: per token a softmax over its ``top_k`` largest logits at those experts,
    zero elsewhere (``src/quark/kernels/moe_router_correct/reference.py:38-49``).  Equal logits: the lower index wins, as
    in the reference's kernel, which inserts with a strict ``>`` (``src/quark/kernels/_moe_router_dsl.py:32-66``); its numpy
    reference leaves ties to numpy's unstable ``argsort``."""
    L = to_f32(logits, "bf16")
    M, E = L.shape
    order = np.argsort(-L, axis=1, kind="stable")[:, :top_k]
    score = np.take_along_axis(L, order, axis=1)
    ex = np.exp(score - score.max(axis=-1, keepdims=True))
    w = ex / ex.sum(axis=-1, keepdims=True)
    dense = np.zeros((E, M), np.float32)
    for k in range(top_k):
        dense[order[:, k], np.arange(M)] = w[:, k]
    return dense


def moe_route_slots(logits, top_k: int, *, tile: int = 128, total_slots: int | None = None, order=None):
    """The same routing as slot tables sorted by expert, every expert's run padded to a multiple of ``tile`` rows
    (``src/quark/kernels/moe_router_correct/reference.py:51-108``, whose tile is 32; the GPU library uses 128, its GEMM's row
    tile).  Returns ``slot_token`` (the token in each slot; -1 for padding here, where the reference leaves 0),
    ``slot_weight``, ``tile_expert`` (-1 past the last used tile: the reference's ``work_list[2 i + 1]``), ``token_slot``
    ``[M, top_k]`` (k in order of decreasing logit), ``offsets`` ``[E + 1]`` and ``counts`` ``[E]``.  Within an expert the
    slots follow (token, k) order, as the reference's numpy oracle fills them.  Ties between logits go to the lower
    expert index (see ``moe_route``); ``order`` ``[M, top_k]`` overrides the choice of experts (the golden test passes the
    reference's, whose unstable sort may break a tie the other way), the layout follows from it."""
    L = to_f32(logits, "bf16")
    M, E = L.shape
    if order is None:
        order = np.argsort(-L, axis=1, kind="stable")[:, :top_k]
    order = np.asarray(order, np.int64)
    score = np.take_along_axis(L, order, axis=1)
    ex = np.exp(score - score.max(axis=-1, keepdims=True))
    w = (ex / ex.sum(axis=-1, keepdims=True)).astype(np.float32)
    counts = np.bincount(order.ravel(), minlength=E).astype(np.int32)
    offsets = np.concatenate([[0], np.cumsum((counts + tile - 1) // tile * tile)]).astype(np.int32)
    if total_slots is None:
        total_slots = (M * top_k + E * (tile - 1) + tile - 1) // tile * tile
    if offsets[-1] > total_slots:
        raise ValueError(f"moe_route_slots: {int(offsets[-1])} active slots exceed the {total_slots} provided")
    slot_token = np.full(total_slots, -1, np.int32)
    slot_weight = np.zeros(total_slots, np.float32)
    token_slot = np.zeros((M, top_k), np.int32)
    cursor = offsets[:-1].copy()
    for t in range(M):
        for k in range(top_k):
            e = order[t, k]
            slot_token[cursor[e]] = t
            slot_weight[cursor[e]] = w[t, k]
            token_slot[t, k] = cursor[e]
            cursor[e] += 1
    tile_expert = np.full(total_slots // tile, -1, np.int32)
    for e in range(E):
        tile_expert[offsets[e] // tile : offsets[e + 1] // tile] = e
    return dict(slot_token=slot_token, slot_weight=slot_weight, tile_expert=tile_expert, token_slot=token_slot, offsets=offsets, counts=counts)


def moe(x, router_w, expert_in, expert_out, *, top_k: int, fp8: bool = False, a_quant: str | None = None):
    """``out[m] = sum_k w_k * W_out[e_k] silu(W_in[e_k] x_m)`` with the reference's rounding points
    (``src/quark/nn/moe.py:252-363``): bf16 router logits, bf16 hidden activations, f32 per-expert outputs, one
    narrowing to bf16 after the weighted sum (``kernels/moe_reduce/reference.py:16-33``).  ``router_w [E, D]`` bf16,
    ``expert_in [E * H, D]``, ``expert_out [E * D, H]`` (bf16, or e4m3 with ``fp8``)."""
    E = router_w.shape[0]
    D = router_w.shape[1]
    H = expert_in.shape[0] // E
    wd = "e4m3" if fp8 else "bf16"
    weights = moe_route(gemm(x, router_w), top_k)
    xf = to_f32(x, "bf16")
    acc = np.zeros((xf.shape[0], D), np.float32)
    for e in range(E):
        sel = weights[e] != 0
        if not sel.any():
            continue
        h = gemm(x, expert_in[e * H : (e + 1) * H], b_dtype=wd, a_quant=a_quant, activation="silu")
        y = gemm(h, expert_out[e * D : (e + 1) * D], b_dtype=wd, a_quant=a_quant, return_f32=True)
        acc[sel] += weights[e][sel, None] * y[sel]
    return from_f32(acc, "bf16")
