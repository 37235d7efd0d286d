"""``qf.*``: the reference's functional call surface on ``QuarkTensor``, over the C ABI.

Same names, positional order, keyword names and error behaviour as ``quark.functional``
(``src/quark/functional/__init__.py:20-79``); each wrapper validates shapes and dtypes the way
the reference's ``spec_from_tensors`` does (``ValueError`` / ``TypeError``), picks or allocates the
output, and makes exactly one call into ``libquark_b200.so`` on the active stream.  Calls are
allocation-free once their output and workspace buffers exist, so they can be captured into a
CUDA graph after one eager run.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib
from ..runtime import stream as _stream
from ..runtime.tensor import QuarkTensor

__all__ = [
    "gemm", "owl_attn", "kv_cache_update", "quantize_e4m3", "ada_rmsnorm", "head_rmsnorm", "value_residual_packed",
    "ada_gate_residual", "silu", "euler_step", "patchify", "unpatchify", "increment", "rope_table", "qkv_post", "quantize_e4m3_rows",
]  # fmt: skip


def _p(t) -> C.c_void_p:
    return C.c_void_p(t.data_ptr() if t is not None else None)


def _s() -> C.c_void_p:
    return C.c_void_p(_stream.active_stream())


def _dt(t) -> str:
    d = getattr(t, "dtype", None)
    if not isinstance(d, str):
        raise TypeError(f"expected a QuarkTensor, got {type(t).__name__}")
    return d


def _code(name: str | None, default: str) -> int:
    name = default if name is None else (name.value if hasattr(name, "value") else name)
    if name not in _lib.DTYPE_CODE:
        raise TypeError(f"unsupported dtype {name!r}")
    return _lib.DTYPE_CODE[name]


# ---------------------------------------------------------------------------
# workspace (K-slice partials, tile counters, e4m3 copies of bf16 activations)
# ---------------------------------------------------------------------------

_WS: QuarkTensor | None = None
_ATTN_WS: QuarkTensor | None = None
# Workspaces that were replaced by larger ones.  A CUDA graph captured while a smaller workspace was current
# (an Engine's frame graph, say) still holds that buffer's device address, so a superseded workspace is never
# freed: it stays referenced here for the life of the process (a few MB each, and growth is rare).
_RETIRED_WS: list = []


def _grow(current: QuarkTensor | None, nbytes: int) -> QuarkTensor:
    if current is not None:
        _RETIRED_WS.append(current)
    return QuarkTensor.zeros(int(nbytes), dtype="e4m3")


def _workspace(nbytes: int) -> QuarkTensor | None:
    """One zero-initialised scratch buffer shared by every GEMM call (calls on one stream never overlap).  The
    library keeps the tile counters in a fixed area at its start, whatever the shape, so calls of different
    shapes can share it."""
    global _WS
    if nbytes <= 0:
        return _WS
    if _WS is None or _WS.nbytes < nbytes:
        _WS = _grow(_WS, max(int(nbytes), 1 << 20))
    return _WS


def _attn_workspace(nbytes: int) -> QuarkTensor | None:
    """The attention kernel's own zero-initialised scratch (tickets first; never shared with the GEMM's)."""
    global _ATTN_WS
    if nbytes <= 0:
        return None
    if _ATTN_WS is None or _ATTN_WS.nbytes < nbytes:
        _ATTN_WS = _grow(_ATTN_WS, int(nbytes))
    return _ATTN_WS


_SCRATCH: dict = {}


def _scratch(tag: str, shape, dtype: str) -> QuarkTensor:
    """Persistent intermediate buffers of composed ops, keyed by use and shape (allocated once)."""
    key = (tag, tuple(shape), dtype)
    t = _SCRATCH.get(key)
    if t is None:
        t = QuarkTensor.empty(*shape, dtype=dtype)
        _SCRATCH[key] = t
    return t


# ---------------------------------------------------------------------------
# RoPE tables
# ---------------------------------------------------------------------------

_ROPE: dict[tuple[int, int], QuarkTensor] = {}


def rope_table_numpy(H: int, W: int, Dh: int = 64) -> np.ndarray:
    """f32 ``[H*W, 16]``: 8 cosines then 8 sines of the 4 x- and 4 y-angles of every token.

    Same arithmetic as the reference table (``src/quark/kernels/kv_cache_update/reference.py:61-106``):
    f64 linspace positions narrowed to f32, times f64 pixel frequencies ``linspace(1, 0.4*min(H,W), 4)*pi``,
    narrowed to f32, then numpy's single-precision cos / sin.
    """
    if H <= 0 or W <= 0:
        raise ValueError(f"H_spatial and W_spatial must be > 0; got H={H}, W={W}")
    if Dh != 64:
        raise ValueError("only head_dim 64 is supported")
    freqs = np.linspace(1.0, min(H, W) * 0.8 / 2, Dh // 16) * np.pi
    fx = np.linspace(-1 + 1 / W, 1 - 1 / W, W).astype(np.float32)[:, None] * freqs  # [W, 4] f64
    fy = np.linspace(-1 + 1 / H, 1 - 1 / H, H).astype(np.float32)[:, None] * freqs  # [H, 4] f64
    ang = np.concatenate(
        [np.broadcast_to(fx[None, :, :], (H, W, 4)), np.broadcast_to(fy[:, None, :], (H, W, 4))], axis=-1
    ).reshape(H * W, 8).astype(np.float32)
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def rope_table(H: int, W: int) -> QuarkTensor:
    key = (int(H), int(W))
    t = _ROPE.get(key)
    if t is None:
        t = QuarkTensor.from_numpy(rope_table_numpy(*key))
        _ROPE[key] = t
    return t


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------


def gemm(A, B, out_dtype=None, compute_dtype=None, b_shuffled=False, activation=None, bias=None, gate=None,
         residual=None, gate_groups=1, out=None, *, a_scale=None, w_scale=None, split_k=0, tile_n=0, slice_mode=0,
         b_constant=False):  # fmt: skip
    """``C = A @ B.T`` (+ bias, SiLU, ``residual + gate * C``); ``src/quark/functional/gemm.py:597-635``.

    ``a_scale`` / ``w_scale`` (f32 device tensors) and ``split_k`` / ``tile_n`` / ``slice_mode`` are extensions; left
    at their defaults the call is the reference's.  ``b_constant=True`` promises that no kernel still in
    flight writes ``B`` (a weight matrix): the kernel then fetches its first ``B`` tiles while the kernels
    before it in the stream are still finishing.
    """
    if b_shuffled:
        raise NotImplementedError("qf.gemm: b_shuffled=True is not supported (disabled upstream as well)")
    if A.ndim < 2 or B.ndim != 2:
        raise ValueError(f"qf.gemm: A must be at least rank-2 and B rank-2, got {A.shape} and {B.shape}")
    K = int(A.shape[-1])
    M = A.numel // K
    N = int(B.shape[0])
    if int(B.shape[1]) != K:
        raise ValueError(f"qf.gemm: A is [..., {K}] but B is {B.shape} (expected [N, {K}])")
    a_dt, b_dt = _dt(A), _dt(B)
    cd = compute_dtype.value if hasattr(compute_dtype, "value") else compute_dtype
    if cd is None:
        cd = b_dt if b_dt == "e4m3" else a_dt
    if cd not in ("bf16", "e4m3"):
        raise TypeError(f"qf.gemm: compute_dtype {cd!r} is not supported")
    if activation not in (None, "silu"):
        raise ValueError(f"qf.gemm: unsupported activation {activation!r}")
    if (gate is None) != (residual is None):
        raise ValueError("qf.gemm: gate and residual must be given together")
    od = out_dtype.value if hasattr(out_dtype, "value") else out_dtype
    if od is None:
        od = out.dtype if out is not None else "bf16"
    if out is None:
        out = QuarkTensor.empty(M, N, dtype=od)
    elif out.numel != M * N or out.dtype != od:
        raise ValueError(f"qf.gemm: out is {out.shape} {out.dtype}, expected ({M}, {N}) {od}")
    if bias is not None and bias.numel != N:
        raise ValueError(f"qf.gemm: bias has {bias.numel} elements, expected {N}")
    if gate is not None:
        if gate.numel != gate_groups * N or residual.numel != M * N:
            raise ValueError(f"qf.gemm: gate must be [{gate_groups}, {N}] and residual [{M}, {N}]")
        if M % gate_groups:
            raise ValueError(f"qf.gemm: gate_groups={gate_groups} does not divide M={M}")
    p = _lib.GemmParams(
        M=M, N=N, K=K, a_dtype=_code(a_dt, "bf16"), b_dtype=_code(b_dt, "bf16"), c_dtype=_code(od, "bf16"),
        compute_dtype=_code(cd, "bf16"), activation=1 if activation == "silu" else 0, gate_groups=int(gate_groups),
        split_k=int(split_k), tile_n=int(tile_n), reserved=int(slice_mode) | (2 if b_constant else 0),
        a_scale=a_scale.data_ptr() if a_scale is not None else None,
        w_scale=w_scale.data_ptr() if w_scale is not None else None,
    )  # fmt: skip
    lib = _lib.load()
    need = int(lib.qb_gemm_workspace_bytes(C.byref(p)))
    ws = _workspace(need)
    _lib.check(
        lib.qb_gemm(_p(A), _p(B), _p(out), _p(bias), _p(gate), _p(residual), C.byref(p), _p(ws), ws.nbytes if ws is not None else 0, _s())
    )
    return out


def gemm_tp(A, B, arena, *, compute_dtype=None, b_constant=False):
    """The row-parallel GEMM of a tensor-parallel rank, ``A @ B.T`` in bf16 with no epilogue, whose rows go straight to
    the ranks that sum them: row ``m`` lands in the staging area of rank ``m // (M / world)`` (``runtime.tp.TpArena``;
    plain stores over NVLink).  Follow it with ``arena.reduce(..., schedule=3)`` on every rank.  No reference counterpart."""
    K = int(A.shape[-1])
    M = A.numel // K
    N = int(B.shape[0])
    if int(B.shape[1]) != K or (M, N) != (arena.rows, arena.D):
        raise ValueError(f"qf.gemm_tp: A {tuple(A.shape)} x B {tuple(B.shape)} is not the [{arena.rows}, {arena.D}] partial of the arena")
    a_dt, b_dt = _dt(A), _dt(B)
    cd = compute_dtype or (b_dt if b_dt == "e4m3" else a_dt)
    gp = _lib.GemmParams(
        M=M, N=N, K=K, a_dtype=_code(a_dt, "bf16"), b_dtype=_code(b_dt, "bf16"), c_dtype=_code("bf16", "bf16"), compute_dtype=_code(cd, "bf16"),
        activation=0, gate_groups=1, split_k=1, tile_n=0, reserved=2 if b_constant else 0, a_scale=None, w_scale=None,
    )  # fmt: skip
    tp = arena.params()
    lib = _lib.load()
    ws = _workspace(int(lib.qb_gemm_workspace_bytes(C.byref(gp))))
    _lib.check(lib.qb_gemm_tp(_p(A), _p(B), C.byref(gp), C.byref(tp), _p(ws), ws.nbytes if ws is not None else 0, _s()))


def quantize_e4m3(X, *, out=None):
    """bf16 / f32 -> e4m3, unscaled, RN-even, saturating (``src/quark/functional/quantize_e4m3.py:25-69``)."""
    dt = _dt(X)
    if dt not in ("bf16", "f32"):
        raise TypeError(f"qf.quantize_e4m3: source dtype {dt!r} is not supported")
    if out is None:
        out = QuarkTensor.empty(*X.shape, dtype="e4m3")
    elif out.numel != X.numel or out.dtype != "e4m3":
        raise ValueError("qf.quantize_e4m3: out must be an e4m3 tensor of the same size")
    _lib.check(_lib.load().qb_quantize_e4m3(_p(X), _p(out), X.numel, _lib.DTYPE_CODE[dt], _s()))
    return out


def quantize_e4m3_rows(X, *, out=None, scale_out=None):
    """Per-row scaled narrowing of a bf16 matrix (a weight ``[out, in]``): ``scale[r] = max|X[r]| / 448``,
    ``out[r] = e4m3(X[r] * (1 / scale[r]))``.  Returns ``(out, scale)``; ``scale`` is what ``qf.gemm`` takes as
    ``w_scale``.  An extension: the reference narrows without a scale (``src/quark/nn/layers.py:291-304``)."""
    if _dt(X) != "bf16" or X.ndim != 2:
        raise TypeError("qf.quantize_e4m3_rows: X must be a bf16 matrix")
    rows, cols = int(X.shape[0]), int(X.shape[1])
    if cols % 8:
        raise ValueError(f"qf.quantize_e4m3_rows: {cols} columns (must be a multiple of 8)")
    if out is None:
        out = QuarkTensor.empty(rows, cols, dtype="e4m3")
    if scale_out is None:
        scale_out = QuarkTensor.empty(rows, dtype="f32")
    if out.numel != X.numel or out.dtype != "e4m3" or scale_out.numel != rows or scale_out.dtype != "f32":
        raise ValueError("qf.quantize_e4m3_rows: out must be e4m3 of X's size and scale_out f32 [rows]")
    _lib.check(_lib.load().qb_quantize_e4m3_rows(_p(X), _p(out), _p(scale_out), rows, cols, _s()))
    return out, scale_out


def _head_scales(who, n_kv_heads, k_scale, v_scale):
    for name, t in (("k_scale", k_scale), ("v_scale", v_scale)):
        if t is not None and (_dt(t) != "f32" or t.numel != n_kv_heads):
            raise ValueError(f"{who}: {name} must be an f32 tensor of {n_kv_heads} per-head scales")
    return (k_scale.data_ptr() if k_scale is not None else None, v_scale.data_ptr() if v_scale is not None else None)


def dequantize_e4m3(X, *, out=None):
    """e4m3 -> bf16, exact (every e4m3 value is a bf16 value)."""
    if _dt(X) != "e4m3":
        raise TypeError(f"qf.dequantize_e4m3: source dtype {_dt(X)!r} (expected e4m3)")
    if out is None:
        out = QuarkTensor.empty(*X.shape, dtype="bf16")
    elif out.numel != X.numel or out.dtype != "bf16":
        raise ValueError("qf.dequantize_e4m3: out must be a bf16 tensor of the same size")
    _lib.check(_lib.load().qb_dequantize_e4m3(_p(X), _p(out), X.numel, _s()))
    return out


# ---------------------------------------------------------------------------
# KV cache append and attention
# ---------------------------------------------------------------------------


def _quilt_checks(who: str, tpf: int, quilt_factor: int, quilt_offset: int) -> None:
    if quilt_factor < 1 or (quilt_factor & (quilt_factor - 1)) != 0:
        raise ValueError(f"{who}: quilt_factor must be a power of 2 (>=1), got {quilt_factor}")
    if quilt_offset < 0 or quilt_offset >= quilt_factor:
        raise ValueError(f"{who}: quilt_offset must be in [0, quilt_factor); got offset={quilt_offset} factor={quilt_factor}")
    if tpf % quilt_factor != 0:
        raise ValueError(f"{who}: H_spatial*W_spatial={tpf} must be divisible by quilt_factor={quilt_factor}")


def kv_cache_update(K, V, frame_t, frozen, Vt_cache, segments, n_segments, K_cache, *, B, n_kv_heads, H_spatial,
                    W_spatial, num_buckets, pinned_dilation, kv_dtype=None, max_segments=3, packed_qkv=False,
                    n_q_heads=0, rope_n_frames=1, quilt_factor=1, quilt_offset=0, k_scale=None, v_scale=None):  # fmt: skip
    """In-place RoPE + cache append (``src/quark/functional/kv_cache_update.py:187-265``).

    ``k_scale`` / ``v_scale`` (extension, f32 ``[n_kv_heads]``): the caches receive ``K / k_scale[h]`` and ``V / v_scale[h]``.

    ``K`` is the packed QKV tensor when ``packed_qkv=True`` (``V`` is then ignored, as upstream); otherwise ``K`` and
    ``V`` are head-major ``[B * n_kv_heads * tpf, 64]`` tensors of their own.
    Returns ``(K_cache, Vt_cache, segments, n_segments)``, the very tensors that were passed in.
    """
    del rope_n_frames
    tpf = int(H_spatial) * int(W_spatial)
    _quilt_checks("qf.kv_cache_update", tpf, quilt_factor, quilt_offset)
    if B != 1:
        raise NotImplementedError("qf.kv_cache_update: only B=1 is supported (the model is batch 1)")
    Dh = 64
    if packed_qkv:
        qkv_dim = (n_q_heads + 2 * n_kv_heads) * Dh
        if K.ndim != 2 or tuple(K.shape) != (B * tpf, qkv_dim):
            raise ValueError(f"qf.kv_cache_update: packed QKV shape {tuple(K.shape)} != ({B * tpf}, {qkv_dim})")
    else:
        if K.ndim != 2 or tuple(K.shape) != (B * n_kv_heads * tpf, Dh):
            raise ValueError(f"qf.kv_cache_update: K shape {tuple(K.shape)} != ({B * n_kv_heads * tpf}, {Dh})")
        if V is None or tuple(V.shape) != tuple(K.shape):
            raise ValueError(f"qf.kv_cache_update: V shape {None if V is None else tuple(V.shape)} != K shape {tuple(K.shape)}")
        if _dt(V) != "bf16":
            raise TypeError(f"qf.kv_cache_update: V dtype {_dt(V)!r} (expected bf16)")
    if _dt(K) != "bf16":
        raise TypeError(f"qf.kv_cache_update: input dtype {_dt(K)!r} (expected bf16)")
    cap = (num_buckets + 1) * (tpf // quilt_factor)  # a quilted cache keeps tpf / quilt_factor tokens per frame
    if tuple(K_cache.shape) != (B * n_kv_heads * cap, Dh):
        raise ValueError(f"qf.kv_cache_update: K_cache shape {tuple(K_cache.shape)} != ({B * n_kv_heads * cap}, {Dh})")
    if tuple(Vt_cache.shape) != (B * n_kv_heads * Dh, cap):
        raise ValueError(f"qf.kv_cache_update: Vt_cache shape {tuple(Vt_cache.shape)} != ({B * n_kv_heads * Dh}, {cap})")
    if int(segments.shape[0]) != B * max_segments * 2:
        raise ValueError(f"qf.kv_cache_update: segments shape {tuple(segments.shape)} != ({B * max_segments * 2},)")
    if int(n_segments.shape[0]) != B:
        raise ValueError(f"qf.kv_cache_update: n_segments shape {tuple(n_segments.shape)} != ({B},)")
    kvd = _dt(K_cache)
    want = kv_dtype.value if hasattr(kv_dtype, "value") else kv_dtype
    if want is not None and want != kvd:
        raise TypeError(f"qf.kv_cache_update: kv_dtype={want!r} but the caches are {kvd!r}")
    if _dt(Vt_cache) != kvd or kvd not in ("bf16", "e4m3"):
        raise TypeError(f"qf.kv_cache_update: cache dtypes {kvd!r} / {_dt(Vt_cache)!r}")
    ks, vs = _head_scales("qf.kv_cache_update", n_kv_heads, k_scale, v_scale)
    p = _lib.KvParams(
        n_q_heads=n_q_heads, n_kv_heads=n_kv_heads, H_spatial=H_spatial, W_spatial=W_spatial, num_buckets=num_buckets,
        pinned_dilation=pinned_dilation, kv_dtype=_lib.DTYPE_CODE[kvd], max_segments=max_segments, quilt_factor=quilt_factor,
        packed_qkv=1 if packed_qkv else 0, quilt_offset=quilt_offset, k_scale=ks, v_scale=vs,
    )  # fmt: skip
    tail = (_p(frame_t), _p(frozen), _p(K_cache), _p(Vt_cache), _p(segments), _p(n_segments), _p(rope_table(H_spatial, W_spatial)),
            C.byref(p), _s())  # fmt: skip
    lib = _lib.load()
    _lib.check(lib.qb_kv_cache_update(_p(K), *tail) if packed_qkv else lib.qb_kv_cache_update_kv(_p(K), _p(V), *tail))
    return K_cache, Vt_cache, segments, n_segments


def qkv_post(QKV, QKV_first, lamb, frame_t, frozen, Vt_cache, segments, n_segments, K_cache, *, n_q_heads, n_kv_heads, H_spatial,
             W_spatial, num_buckets, pinned_dilation, eps: float = 1e-6, max_segments=3, out=None, k_scale=None, v_scale=None):  # fmt: skip
    """``head_rmsnorm`` + ``value_residual_packed`` + ``kv_cache_update`` in one launch (no reference
    counterpart as a single call; bit-identical to the three calls of
    ``src/quark/models/waypoint_15.py:398-407``).  ``QKV_first`` / ``lamb`` may both be None.
    Returns the normalised / mixed packed QKV; the caches and segment table are updated in place."""
    _bf16_only("qf.qkv_post", QKV)
    tpf = int(H_spatial) * int(W_spatial)
    qkv_dim = (n_q_heads + 2 * n_kv_heads) * 64
    if QKV.ndim != 2 or tuple(QKV.shape) != (tpf, qkv_dim):
        raise ValueError(f"qf.qkv_post: packed QKV shape {tuple(QKV.shape)} != ({tpf}, {qkv_dim})")
    if (QKV_first is None) != (lamb is None):
        raise ValueError("qf.qkv_post: QKV_first and lamb must be given together")
    if QKV_first is not None and (tuple(QKV_first.shape) != tuple(QKV.shape) or _dt(QKV_first) != "bf16" or _dt(lamb) != "f32"):
        raise ValueError("qf.qkv_post: QKV_first must match QKV (bf16) and lamb must be an f32 tensor")
    cap = num_buckets * tpf + tpf
    if tuple(K_cache.shape) != (n_kv_heads * cap, 64) or tuple(Vt_cache.shape) != (n_kv_heads * 64, cap):
        raise ValueError(f"qf.qkv_post: cache shapes {tuple(K_cache.shape)} / {tuple(Vt_cache.shape)} do not match capacity {cap}")
    if int(segments.shape[0]) != max_segments * 2 or int(n_segments.shape[0]) != 1:
        raise ValueError("qf.qkv_post: segments / n_segments shapes")
    kvd = _dt(K_cache)
    if _dt(Vt_cache) != kvd or kvd not in ("bf16", "e4m3"):
        raise TypeError(f"qf.qkv_post: cache dtypes {kvd!r} / {_dt(Vt_cache)!r}")
    out = _like(QKV, out, "qf.qkv_post")
    ks, vs = _head_scales("qf.qkv_post", n_kv_heads, k_scale, v_scale)
    p = _lib.KvParams(
        n_q_heads=n_q_heads, n_kv_heads=n_kv_heads, H_spatial=H_spatial, W_spatial=W_spatial, num_buckets=num_buckets,
        pinned_dilation=pinned_dilation, kv_dtype=_lib.DTYPE_CODE[kvd], max_segments=max_segments, quilt_factor=1, packed_qkv=1,
        k_scale=ks, v_scale=vs,
    )  # fmt: skip
    _lib.check(
        _lib.load().qb_qkv_post(
            _p(QKV), _p(QKV_first), _p(lamb), _p(out), _p(frame_t), _p(frozen), _p(K_cache), _p(Vt_cache), _p(segments),
            _p(n_segments), _p(rope_table(H_spatial, W_spatial)), C.byref(p), float(eps), _s(),
        )
    )  # fmt: skip
    return out


def gemm_qkv_post(A, B, QKV_first, lamb, frame_t, frozen, Vt_cache, segments, n_segments, K_cache, *, n_q_heads, n_kv_heads,
                  H_spatial, W_spatial, num_buckets, pinned_dilation, compute_dtype=None, eps: float = 1e-6, max_segments=3, out=None,
                  a_scale=None, w_scale=None, k_scale=None, v_scale=None, quilt_factor=1, quilt_offset=0):  # fmt: skip
    """``qkv_post(gemm(A, B))`` in one launch: the QKV projection whose epilogue normalises the Q and K heads,
    mixes V with the first block's, rotates K and appends K / V to the caches (same bytes as the two calls;
    no reference counterpart as a single call).  Returns the packed QKV that ``owl_attn`` reads."""
    K = int(A.shape[-1])
    M = A.numel // K
    N = int(B.shape[0])
    tpf = int(H_spatial) * int(W_spatial)
    if M != tpf or N != (n_q_heads + 2 * n_kv_heads) * 64 or int(B.shape[1]) != K:
        raise ValueError(f"qf.gemm_qkv_post: A {tuple(A.shape)} x B {tuple(B.shape)} is not the [{tpf}, {(n_q_heads + 2 * n_kv_heads) * 64}] projection")
    a_dt, b_dt = _dt(A), _dt(B)
    cd = compute_dtype or (b_dt if b_dt == "e4m3" else a_dt)
    if (QKV_first is None) != (lamb is None):
        raise ValueError("qf.gemm_qkv_post: QKV_first and lamb must be given together")
    if QKV_first is not None and (tuple(QKV_first.shape) != (M, N) or _dt(QKV_first) != "bf16" or _dt(lamb) != "f32"):
        raise ValueError("qf.gemm_qkv_post: QKV_first must be the packed bf16 QKV of the first block and lamb an f32 tensor")
    _quilt_checks("qf.gemm_qkv_post", tpf, quilt_factor, quilt_offset)
    cap = (num_buckets + 1) * (tpf // quilt_factor)  # a quilted cache keeps tpf / quilt_factor tokens per frame
    if tuple(K_cache.shape) != (n_kv_heads * cap, 64) or tuple(Vt_cache.shape) != (n_kv_heads * 64, cap):
        raise ValueError(f"qf.gemm_qkv_post: cache shapes {tuple(K_cache.shape)} / {tuple(Vt_cache.shape)} do not match capacity {cap}")
    if int(segments.shape[0]) != max_segments * 2 or int(n_segments.shape[0]) != 1:
        raise ValueError("qf.gemm_qkv_post: segments / n_segments shapes")
    kvd = _dt(K_cache)
    if _dt(Vt_cache) != kvd or kvd not in ("bf16", "e4m3"):
        raise TypeError(f"qf.gemm_qkv_post: cache dtypes {kvd!r} / {_dt(Vt_cache)!r}")
    if out is None:
        out = QuarkTensor.empty(M, N, dtype="bf16")
    elif out.numel != M * N or out.dtype != "bf16":
        raise ValueError(f"qf.gemm_qkv_post: out is {out.shape} {out.dtype}, expected ({M}, {N}) bf16")
    gp = _lib.GemmParams(
        M=M, N=N, K=K, a_dtype=_code(a_dt, "bf16"), b_dtype=_code(b_dt, "bf16"), c_dtype=_code("bf16", "bf16"),
        compute_dtype=_code(cd, "bf16"), activation=0, gate_groups=1, split_k=1, tile_n=128, reserved=2,
        a_scale=a_scale.data_ptr() if a_scale is not None else None, w_scale=w_scale.data_ptr() if w_scale is not None else None,
    )  # fmt: skip
    if w_scale is not None and (_dt(w_scale) != "f32" or w_scale.numel != N):
        raise ValueError(f"qf.gemm_qkv_post: w_scale must be f32 [{N}]")
    ks, vs = _head_scales("qf.gemm_qkv_post", n_kv_heads, k_scale, v_scale)
    kp = _lib.KvParams(
        n_q_heads=n_q_heads, n_kv_heads=n_kv_heads, H_spatial=H_spatial, W_spatial=W_spatial, num_buckets=num_buckets,
        pinned_dilation=pinned_dilation, kv_dtype=_lib.DTYPE_CODE[kvd], max_segments=max_segments, quilt_factor=quilt_factor, packed_qkv=1,
        quilt_offset=quilt_offset, k_scale=ks, v_scale=vs,
    )  # fmt: skip
    lib = _lib.load()
    ws = _workspace(int(lib.qb_gemm_workspace_bytes(C.byref(gp))))
    _lib.check(
        lib.qb_gemm_qkv_post(
            _p(A), _p(B), _p(out), _p(QKV_first), _p(lamb), _p(frame_t), _p(frozen), _p(K_cache), _p(Vt_cache), _p(segments), _p(n_segments),
            _p(rope_table(H_spatial, W_spatial)), C.byref(gp), C.byref(kp), float(eps), _p(ws), ws.nbytes if ws is not None else 0, _s(),
        )
    )  # fmt: skip
    return out


_DUMMY_FRAME_T: QuarkTensor | None = None


_CAST_SCRATCH: dict = {}


def _cast_scratch(t, dtype: str, which: int):
    key = (tuple(t.shape), dtype, which)
    if key not in _CAST_SCRATCH:
        _CAST_SCRATCH[key] = QuarkTensor.empty(*t.shape, dtype=dtype)
    return _CAST_SCRATCH[key]


def owl_attn(Q, K_cache, Vt_cache, segments, n_segments, B, n_kv_heads, gqa_ratio, H_spatial, W_spatial, num_buckets,
             pinned_dilation, out_dtype=None, compute_dtype=None, max_segments=3, packed_qkv=False, quilt_factor=1,
             quilt_offset=0, frame_t=None, *, out=None, out_q=None, k_scale=None, v_scale=None, kv_splits=0):  # fmt: skip
    """Segment-sparse GQA attention with inline Q RoPE (``src/quark/functional/owl_attn.py:322-394``)."""
    global _DUMMY_FRAME_T
    if Q.ndim != 2:
        raise ValueError(f"qf.owl_attn: Q must be rank-2 (flat), got {Q.shape}")
    tpf = int(H_spatial) * int(W_spatial)
    _quilt_checks("qf.owl_attn", tpf, quilt_factor, quilt_offset)
    if B != 1:
        raise NotImplementedError("qf.owl_attn: only B=1 is supported (the model is batch 1)")
    n_q = n_kv_heads * gqa_ratio
    Dh = 64
    # packed: Q is the QKV projection [tpf, (Hq + 2 Hk) * 64] and the output is [tpf, Hq * 64]; otherwise Q and the
    # output are head-major [Hq * tpf, 64] (src/quark/kernels/owl_attn/kernel.py:248-288)
    q_shape = (B * tpf, (n_q + 2 * n_kv_heads) * 64) if packed_qkv else (B * n_q * tpf, Dh)
    o_shape = (B * tpf, n_q * Dh) if packed_qkv else (B * n_q * tpf, Dh)
    if tuple(Q.shape) != q_shape:
        raise ValueError(f"qf.owl_attn: {'packed QKV' if packed_qkv else 'Q'} shape {tuple(Q.shape)} != {q_shape}")
    cap = (num_buckets + 1) * (tpf // quilt_factor)
    if tuple(K_cache.shape) != (B * n_kv_heads * cap, Dh):
        raise ValueError(f"qf.owl_attn: K_cache shape {tuple(K_cache.shape)} != ({B * n_kv_heads * cap}, {Dh})")
    if tuple(Vt_cache.shape) != (B * n_kv_heads * Dh, cap):
        raise ValueError(f"qf.owl_attn: Vt_cache shape {tuple(Vt_cache.shape)} != ({B * n_kv_heads * Dh}, {cap})")
    if int(segments.shape[0]) != B * max_segments * 2:
        raise ValueError(f"qf.owl_attn: segments shape {tuple(segments.shape)} != ({B * max_segments * 2},)")
    if int(n_segments.shape[0]) != B:
        raise ValueError(f"qf.owl_attn: n_segments shape {tuple(n_segments.shape)} != ({B},)")
    if _dt(Q) != "bf16":
        raise TypeError(f"qf.owl_attn: Q dtype {_dt(Q)!r} (expected bf16)")
    kvd = _dt(K_cache)
    cd = compute_dtype.value if hasattr(compute_dtype, "value") else compute_dtype
    if cd is None:
        cd = "bf16"
    if cd not in ("bf16", "e4m3") or kvd not in ("bf16", "e4m3"):
        raise NotImplementedError(f"qf.owl_attn: compute_dtype={cd!r} with a {kvd!r} cache (bf16 and e4m3 only)")
    if cd != kvd:
        # The reference casts K and V to the compute dtype as it loads them (src/quark/kernels/owl_attn/kernel.py:
        # 342-348).  Here the cast is a pass of its own into a scratch copy of the two caches (one pair per shape,
        # reused by every layer: calls on one stream run in order), after which the kernel for that dtype runs.
        # Same values as casting on load; a cache's worth of extra traffic per call, so not the fast path.
        conv = quantize_e4m3 if cd == "e4m3" else dequantize_e4m3
        Ks, Vs = _cast_scratch(K_cache, cd, 0), _cast_scratch(Vt_cache, cd, 1)
        conv(K_cache, out=Ks)
        conv(Vt_cache, out=Vs)
        K_cache, Vt_cache, kvd = Ks, Vs, cd
    od = out_dtype.value if hasattr(out_dtype, "value") else out_dtype
    if od not in (None, "bf16"):
        raise NotImplementedError(f"qf.owl_attn: out_dtype {od!r} (only bf16)")
    if out is None:
        out = QuarkTensor.empty(*o_shape, dtype="bf16")
    elif out.numel != B * tpf * n_q * Dh or out.dtype != "bf16":
        raise ValueError(f"qf.owl_attn: out is {out.shape} {out.dtype}, expected {o_shape} bf16")
    if out_q is not None and (out_q.dtype != "e4m3" or out_q.numel != out.numel):
        raise ValueError("qf.owl_attn: out_q must be an e4m3 tensor of the output's size")
    if frame_t is None:
        if _DUMMY_FRAME_T is None:
            _DUMMY_FRAME_T = QuarkTensor.zeros(1, dtype="s32")
        frame_t = _DUMMY_FRAME_T
    p = _lib.AttnParams(
        n_kv_heads=n_kv_heads, gqa_ratio=gqa_ratio, H_spatial=H_spatial, W_spatial=W_spatial, num_buckets=num_buckets,
        pinned_dilation=pinned_dilation, kv_dtype=_lib.DTYPE_CODE[kvd], compute_dtype=_lib.DTYPE_CODE[cd],
        max_segments=max_segments, packed_qkv=1 if packed_qkv else 0, quilt_factor=quilt_factor, kv_splits=int(kv_splits),
        k_scale=k_scale.data_ptr() if k_scale is not None else None,
        v_scale=v_scale.data_ptr() if v_scale is not None else None,
    )  # fmt: skip
    lib = _lib.load()
    ws = _attn_workspace(int(lib.qb_owl_attn_workspace_bytes(C.byref(p))))
    _lib.check(
        lib.qb_owl_attn(
            _p(Q), _p(K_cache), _p(Vt_cache), _p(segments), _p(n_segments), _p(frame_t), _p(out), _p(out_q),
            _p(rope_table(H_spatial, W_spatial)), C.byref(p), _p(ws), ws.nbytes if ws is not None else 0, _s(),
        )
    )  # fmt: skip
    return out


# ---------------------------------------------------------------------------
# norm / elementwise ops
# ---------------------------------------------------------------------------


def _like(X, out, who):
    if out is None:
        return QuarkTensor.empty(*X.shape, dtype=X.dtype)
    if out.numel != X.numel or out.dtype != X.dtype:
        raise ValueError(f"{who}: out is {out.shape} {out.dtype}, expected {X.shape} {X.dtype}")
    return out


def _bf16_only(who, *ts):
    for t in ts:
        if _dt(t) != "bf16":
            raise TypeError(f"{who}: dtype {_dt(t)!r} (expected bf16)")


def ada_rmsnorm(X, scale, bias, eps: float = 1e-6, activation: str | None = None, *, out=None, out_q=None, only_q: bool = False):
    """``rmsnorm(x) * (1 + scale) + bias`` (+ SiLU) (``src/quark/functional/ada_rmsnorm.py:61``).

    ``out_q`` (extension): an e4m3 tensor that also receives the result, for a following fp8 GEMM; with ``only_q`` the
    bf16 result is not written at all (``out_q`` is returned).
    """
    _bf16_only("qf.ada_rmsnorm", X, scale, bias)
    D = int(X.shape[-1])
    rows = X.numel // D
    G = scale.numel // D
    if scale.numel != G * D or bias.numel != G * D or G == 0 or rows % G:
        raise ValueError(f"qf.ada_rmsnorm: X {X.shape}, scale {scale.shape}, bias {bias.shape} do not broadcast")
    if activation not in (None, "silu"):
        raise ValueError(f"qf.ada_rmsnorm: unsupported activation {activation!r}")
    if only_q and out_q is None:
        raise ValueError("qf.ada_rmsnorm: only_q needs out_q")
    out = None if only_q else _like(X, out, "qf.ada_rmsnorm")
    if out_q is not None and (out_q.dtype != "e4m3" or out_q.numel != X.numel):
        raise ValueError("qf.ada_rmsnorm: out_q must be an e4m3 tensor of the same size")
    _lib.check(
        _lib.load().qb_ada_rmsnorm(_p(X), _p(scale), _p(bias), _p(out), _p(out_q), rows, D, G, float(eps), 1 if activation == "silu" else 0, _s())
    )
    return out_q if only_q else out


def head_rmsnorm(X, n_q_heads: int, n_kv_heads: int, Dh: int, eps: float = 1e-6, *, out=None):
    """Per-head RMS norm of the Q and K heads of packed QKV (``src/quark/functional/head_rmsnorm.py:33``)."""
    _bf16_only("qf.head_rmsnorm", X)
    if X.ndim != 2 or int(X.shape[1]) != (n_q_heads + 2 * n_kv_heads) * Dh:
        raise ValueError(f"qf.head_rmsnorm: X shape {X.shape} is not [M, (n_q + 2 n_kv) * Dh]")
    out = _like(X, out, "qf.head_rmsnorm")
    _lib.check(_lib.load().qb_head_rmsnorm(_p(X), _p(out), int(X.shape[0]), n_q_heads, n_kv_heads, Dh, float(eps), _s()))
    return out


def value_residual_packed(QKV_curr, QKV_first, lamb, *, v_col_offset, v_width, out=None):
    """``v += lamb * (v_first - v)`` on the V columns; ``lamb`` is an f32 device scalar."""
    _bf16_only("qf.value_residual_packed", QKV_curr, QKV_first)
    if QKV_curr.ndim != 2 or tuple(QKV_curr.shape) != tuple(QKV_first.shape):
        raise ValueError(f"qf.value_residual_packed: shapes {QKV_curr.shape} and {QKV_first.shape}")
    if _dt(lamb) != "f32":
        raise TypeError("qf.value_residual_packed: lamb must be an f32 tensor")
    out = _like(QKV_curr, out, "qf.value_residual_packed")
    _lib.check(
        _lib.load().qb_value_residual_packed(
            _p(QKV_curr), _p(QKV_first), _p(lamb), _p(out), int(QKV_curr.shape[0]), int(QKV_curr.shape[1]), v_col_offset, v_width, _s()
        )
    )
    return out


def ada_gate_residual(X, Y, gate, *, out=None):
    """``x + gate * y`` with the gate broadcast over groups of rows."""
    _bf16_only("qf.ada_gate_residual", X, Y, gate)
    D = int(X.shape[-1])
    rows = X.numel // D
    G = gate.numel // D
    if Y.numel != X.numel or gate.numel != G * D or G == 0 or rows % G:
        raise ValueError(f"qf.ada_gate_residual: X {X.shape}, Y {Y.shape}, gate {gate.shape} do not broadcast")
    out = _like(X, out, "qf.ada_gate_residual")
    _lib.check(_lib.load().qb_ada_gate_residual(_p(X), _p(Y), _p(gate), _p(out), rows, D, G, _s()))
    return out


def silu(X, *, out=None, out_q=None):
    _bf16_only("qf.silu", X)
    out = _like(X, out, "qf.silu")
    if out_q is not None and (out_q.dtype != "e4m3" or out_q.numel != X.numel):
        raise ValueError("qf.silu: out_q must be an e4m3 tensor of the same size")
    _lib.check(_lib.load().qb_silu(_p(X), _p(out), _p(out_q), X.numel, _s()))
    return out


def rmsnorm(X, eps: float = 1e-6, *, out=None):
    """``x * rsqrt(mean(x^2, last dim) + eps)``, no gain (``src/quark/functional/rmsnorm.py:29-45``)."""
    _bf16_only("qf.rmsnorm", X)
    D = int(X.shape[-1])
    out = _like(X, out, "qf.rmsnorm")
    _lib.check(_lib.load().qb_rmsnorm(_p(X), _p(out), X.numel // D, D, float(eps), _s()))
    return out


def add(X, Y, *, out=None):
    """``x + y`` on same-shape bf16 tensors (the reference's ``elemwise_binary("add")``, ``src/quark/nn/layers.py:655-669``)."""
    _bf16_only("qf.add", X, Y)
    if Y.numel != X.numel:
        raise ValueError(f"qf.add: X {X.shape} and Y {Y.shape}")
    out = _like(X, out, "qf.add")
    _lib.check(_lib.load().qb_add(_p(X), _p(Y), _p(out), X.numel, _s()))
    return out


def euler_step(X, V, Dsig, *, out=None):
    """``cast(f32(X) + f32(Dsig[0]) * f32(V), X.dtype)`` (``src/quark/functional/euler_step.py:36-41``)."""
    _bf16_only("qf.euler_step", X, V)
    if V.numel != X.numel:
        raise ValueError(f"qf.euler_step: X {X.shape} and V {V.shape}")
    if _dt(Dsig) != "f32":
        raise TypeError("qf.euler_step: Dsig must be an f32 tensor")
    out = _like(X, out, "qf.euler_step")
    _lib.check(_lib.load().qb_euler_step(_p(X), _p(V), _p(Dsig), _p(out), X.numel, _s()))
    return out


def randn(*, shape, dtype: str = "bf16", counter_offset, out=None, seed0: int = 0xDEADBEEF, seed1: int = 0xBADC0FFE, counter_stride: int = 1):
    """Standard normals of ``shape`` made on the device: Philox4x32-10 + Box-Muller, a pure function of
    ``(counter_offset[0] * counter_stride, seed0, seed1)`` (``src/quark/functional/randn.py:33-82``).

    ``counter_offset`` is a one-element device tensor (four bytes: ``s32`` here, read as unsigned).  The reference
    leaves it to the caller to move it far enough between draws; ``counter_stride`` (an addition) multiplies it on
    the device, so a counter that goes up by one per draw (the frame counter, say) with
    ``counter_stride >= ceil(n / 4)`` gives disjoint Philox counters.  ``out`` makes the call allocation-free."""
    if isinstance(shape, int):
        shape = (shape,)
    n = 1
    for d in shape:
        n *= int(d)
    if n <= 0:
        raise ValueError(f"qf.randn: shape {shape}")
    if dtype not in ("bf16", "f32"):
        raise ValueError(f"qf.randn: dtype must be 'bf16' or 'f32', got {dtype!r}")
    if _dt(counter_offset) not in ("s32", "u32") or counter_offset.numel != 1:
        raise TypeError("qf.randn: counter_offset must be a one-element 32-bit integer tensor")
    if out is None:
        out = QuarkTensor.empty(*shape, dtype=dtype)
    elif out.numel != n or _dt(out) != dtype:
        raise ValueError(f"qf.randn: out is {out.shape} {_dt(out)}, expected {n} elements of {dtype}")
    _lib.check(_lib.load().qb_randn(_p(counter_offset), _p(out), n, _lib.DTYPE_CODE[dtype], int(counter_stride) & 0xFFFFFFFF, seed0 & 0xFFFFFFFF,
                                    seed1 & 0xFFFFFFFF, _s()))  # fmt: skip
    return out


def moe_route(logits, *, top_k: int, out=None):
    """Dense routing weights ``[E, M]`` f32 of the "correct" mixture-of-experts routing: per token a softmax over its
    ``top_k`` largest logits, zero elsewhere (``src/quark/kernels/moe_router_correct/reference.py:38-49``)."""
    if _dt(logits) != "bf16" or logits.ndim != 2:
        raise TypeError("qf.moe_route: logits must be a bf16 [M, E] tensor")
    M, E = int(logits.shape[0]), int(logits.shape[1])
    if out is None:
        out = QuarkTensor.empty(E, M, dtype="f32")
    elif out.numel != E * M or _dt(out) != "f32":
        raise ValueError(f"qf.moe_route: out must be f32 [{E}, {M}]")
    _lib.check(_lib.load().qb_moe_route(_p(logits), _p(out), M, E, int(top_k), _s()))
    return out


def moe_combine(partials, weights, *, out=None):
    """``out[m] = sum_e weights[e, m] * partials[e * M + m]`` in f32, narrowed to bf16 once
    (``src/quark/kernels/moe_reduce/reference.py:16-33``).  ``partials`` f32 ``[E * M, D]``, ``weights`` f32 ``[E, M]``."""
    if _dt(partials) != "f32" or _dt(weights) != "f32":
        raise TypeError("qf.moe_combine: partials and weights must be f32")
    E, M = int(weights.shape[0]), int(weights.shape[1])
    D = int(partials.shape[-1])
    if partials.numel != E * M * D:
        raise ValueError(f"qf.moe_combine: partials {partials.shape} for weights {weights.shape}")
    if out is None:
        out = QuarkTensor.empty(M, D, dtype="bf16")
    elif out.numel != M * D or _dt(out) != "bf16":
        raise ValueError(f"qf.moe_combine: out must be bf16 [{M}, {D}]")
    _lib.check(_lib.load().qb_moe_combine(_p(partials), _p(weights), _p(out), M, D, E, _s()))
    return out


def kv_cast_appended(K_cache, Vt_cache, K_shadow, Vt_shadow, frame_t, frozen, *, n_kv_heads, H_spatial, W_spatial, num_buckets, pinned_dilation,
                     quilt_factor=1, **_ignored):
    """Brings the rows the last append wrote (tail slot; ring slot on a write frame) over into a second pair of caches in
    the other dtype, so that ``K_shadow == cast(K_cache)`` stays true: the reference's cast on load for a cache whose dtype
    differs from the attention's compute dtype (``src/quark/kernels/owl_attn/kernel.py:342-348``), done per appended row."""
    kvd = _dt(K_cache)
    other = "bf16" if kvd == "e4m3" else "e4m3"
    if kvd not in ("bf16", "e4m3") or _dt(Vt_cache) != kvd or _dt(K_shadow) != other or _dt(Vt_shadow) != other:
        raise TypeError("qf.kv_cast_appended: the shadow pair must have the other of the two cache dtypes")
    if K_shadow.numel != K_cache.numel or Vt_shadow.numel != Vt_cache.numel:
        raise ValueError("qf.kv_cast_appended: the shadow pair must have the caches' shapes")
    p = _lib.KvParams(
        n_q_heads=0, n_kv_heads=n_kv_heads, H_spatial=H_spatial, W_spatial=W_spatial, num_buckets=num_buckets, pinned_dilation=pinned_dilation,
        kv_dtype=_lib.DTYPE_CODE[kvd], max_segments=3, quilt_factor=quilt_factor, packed_qkv=1, quilt_offset=0, k_scale=None, v_scale=None,
    )  # fmt: skip
    _lib.check(_lib.load().qb_kv_cast_appended(_p(K_cache), _p(Vt_cache), _p(K_shadow), _p(Vt_shadow), _p(frame_t), _p(frozen), C.byref(p), _s()))


def moe_slots(M: int, E: int, top_k: int) -> int:
    """Rows of the slot tables of ``moe_route_slots``: every expert's run padded to whole 128-row tiles."""
    return int(_lib.load().qb_moe_slots(int(M), int(E), int(top_k)))


def moe_route_slots(logits, *, top_k: int, slot_token=None, slot_weight=None, tile_expert=None, token_slot=None, counts=None):
    """The "correct" routing as slot tables sorted by expert (``src/quark/kernels/moe_router_correct/reference.py:51-120``;
    row tile 128 here).  Returns ``(slot_token, slot_weight, tile_expert, token_slot)``."""
    if _dt(logits) != "bf16" or logits.ndim != 2:
        raise TypeError("qf.moe_route_slots: logits must be a bf16 [M, E] tensor")
    M, E = int(logits.shape[0]), int(logits.shape[1])
    n = moe_slots(M, E, top_k)
    slot_token = slot_token if slot_token is not None else QuarkTensor.empty(n, dtype="s32")
    slot_weight = slot_weight if slot_weight is not None else QuarkTensor.empty(n, dtype="f32")
    tile_expert = tile_expert if tile_expert is not None else QuarkTensor.empty(n // 128, dtype="s32")
    token_slot = token_slot if token_slot is not None else QuarkTensor.empty(M, int(top_k), dtype="s32")
    if slot_token.numel != n or slot_weight.numel != n or tile_expert.numel != n // 128 or token_slot.numel != M * int(top_k):
        raise ValueError(f"qf.moe_route_slots: tables must hold {n} slots, {n // 128} tiles and [{M}, {top_k}] token slots")
    _lib.check(_lib.load().qb_moe_route_slots(_p(logits), _p(slot_token), _p(slot_weight), _p(tile_expert), _p(token_slot), _p(counts), M, E,
                                              int(top_k), _s()))  # fmt: skip
    return slot_token, slot_weight, tile_expert, token_slot


def moe_gather(x, slot_token, *, out=None):
    """``out[s] = x[slot_token[s]]`` (zeros for padding slots): the activations in slot order."""
    D = int(x.shape[-1])
    n = slot_token.numel
    es = {"bf16": 2, "e4m3": 1, "f32": 4}[_dt(x)]
    if out is None:
        out = QuarkTensor.empty(n, D, dtype=_dt(x))
    elif out.numel != n * D or _dt(out) != _dt(x):
        raise ValueError(f"qf.moe_gather: out must be {_dt(x)} [{n}, {D}]")
    _lib.check(_lib.load().qb_moe_gather(_p(x), _p(slot_token), _p(out), n, D * es, _s()))
    return out


def gemm_grouped(A, B, tile_expert, *, n_experts: int, out_dtype="bf16", compute_dtype=None, activation=None, out=None, b_constant=False):
    """``C[tile i] = A[tile i] @ B[expert(i)].T`` over 128-row tiles of slot-sorted rows; tiles whose expert is -1 are skipped.
    ``B`` is ``[n_experts * N, K]``.  Replaces ``qf.moe_inproj`` / ``qf.moe_outproj`` (``src/quark/nn/moe.py:307-338``)."""
    K = int(A.shape[-1])
    M = A.numel // K
    if int(B.shape[0]) % int(n_experts) or int(B.shape[1]) != K:
        raise ValueError(f"qf.gemm_grouped: B {tuple(B.shape)} is not [{n_experts} * N, {K}]")
    N = int(B.shape[0]) // int(n_experts)
    if M % 128 or tile_expert.numel != M // 128:
        raise ValueError(f"qf.gemm_grouped: {M} rows need {M // 128} whole tiles, the table has {tile_expert.numel}")
    if activation not in (None, "silu"):
        raise ValueError(f"qf.gemm_grouped: unsupported activation {activation!r}")
    a_dt, b_dt = _dt(A), _dt(B)
    cd = compute_dtype or (b_dt if b_dt == "e4m3" else a_dt)
    if out is None:
        out = QuarkTensor.empty(M, N, dtype=out_dtype)
    elif out.numel != M * N or _dt(out) != out_dtype:
        raise ValueError(f"qf.gemm_grouped: out must be {out_dtype} [{M}, {N}]")
    p = _lib.GemmParams(
        M=M, N=N, K=K, a_dtype=_code(a_dt, "bf16"), b_dtype=_code(b_dt, "bf16"), c_dtype=_code(out_dtype, "bf16"), compute_dtype=_code(cd, "bf16"),
        activation=1 if activation == "silu" else 0, gate_groups=1, split_k=1, tile_n=0, reserved=2 if b_constant else 0, a_scale=None, w_scale=None,
    )  # fmt: skip
    lib = _lib.load()
    ws = _workspace(int(lib.qb_gemm_grouped_workspace_bytes(C.byref(p))))
    _lib.check(lib.qb_gemm_grouped(_p(A), _p(B), _p(out), _p(tile_expert), int(n_experts), C.byref(p), _p(ws), ws.nbytes if ws is not None else 0, _s()))
    return out


def moe_reduce(partials, slot_weight, token_slot, *, out=None):
    """``out[m] = sum_k slot_weight[s] * partials[s]``, ``s = token_slot[m, k]``, in f32, narrowed to bf16 once
    (``src/quark/kernels/moe_reduce/reference.py:16-33``)."""
    if _dt(partials) != "f32" or _dt(slot_weight) != "f32" or _dt(token_slot) != "s32":
        raise TypeError("qf.moe_reduce: partials and slot_weight must be f32, token_slot s32")
    M, top_k = int(token_slot.shape[0]), int(token_slot.shape[1])
    D = int(partials.shape[-1])
    if out is None:
        out = QuarkTensor.empty(M, D, dtype="bf16")
    elif out.numel != M * D or _dt(out) != "bf16":
        raise ValueError(f"qf.moe_reduce: out must be bf16 [{M}, {D}]")
    _lib.check(_lib.load().qb_moe_reduce(_p(partials), _p(slot_weight), _p(token_slot), _p(out), M, D, top_k, _s()))
    return out


def increment(counter):
    if _dt(counter) != "s32":
        raise TypeError("qf.increment: counter must be an s32 tensor")
    _lib.check(_lib.load().qb_increment(_p(counter), _s()))
    return counter


def patchify(X, W, *, B: int, C: int, H: int, W_spatial: int, ph: int = 2, pw: int = 2, out=None):
    """``[B, C*H*W] -> [B*Hp*Wp, d_model]`` (``src/quark/nn/layers.py:524-550``)."""
    _bf16_only("qf.patchify", X, W)
    if B != 1:
        raise NotImplementedError("qf.patchify: only B=1 is supported")
    if H % ph or W_spatial % pw:
        raise ValueError(f"qf.patchify: H={H} W={W_spatial} not divisible by patch ({ph},{pw})")
    d_model = int(W.shape[0])
    if X.numel != C * H * W_spatial or int(W.shape[1]) != C * ph * pw:
        raise ValueError(f"qf.patchify: X {X.shape} / W {W.shape} do not match C={C}, H={H}, W={W_spatial}")
    tokens = (H // ph) * (W_spatial // pw)
    if out is None:
        out = QuarkTensor.empty(tokens, d_model, dtype="bf16")
    elif out.numel != tokens * d_model:
        raise ValueError(f"qf.patchify: out is {out.shape}, expected ({tokens}, {d_model})")
    K = C * ph * pw
    if K % 16 == 0 and d_model % 8 == 0:  # tensor-core route: gather the patches, then one GEMM
        tmp = _scratch("patchify", (tokens, K), "bf16")
        _lib.check(_lib.load().qb_patch_gather(_p(X), _p(tmp), C, H, W_spatial, ph, pw, _s()))
        return gemm(tmp, W, out_dtype="bf16", out=out.reshape(tokens, d_model), b_constant=True)
    _lib.check(_lib.load().qb_patchify(_p(X), _p(W), _p(out), C, H, W_spatial, ph, pw, d_model, _s()))
    return out


def unpatchify(X, weight, bias, *, B: int, C: int, H: int, W: int, ph: int = 2, pw: int = 2, out=None):
    """``[M, d_model] -> [B, C*H*W]`` (``src/quark/functional/unpatchify.py:18-20``)."""
    _bf16_only("qf.unpatchify", X, weight)
    if B != 1:
        raise NotImplementedError("qf.unpatchify: only B=1 is supported")
    if H % ph or W % pw:
        raise ValueError(f"qf.unpatchify: H={H} W={W} not divisible by patch ({ph},{pw})")
    d_model = int(weight.shape[1])
    tokens = (H // ph) * (W // pw)
    if X.numel != tokens * d_model or int(weight.shape[0]) != C * ph * pw:
        raise ValueError(f"qf.unpatchify: X {X.shape} / weight {weight.shape} do not match C={C}, H={H}, W={W}")
    if bias is not None and bias.numel != C * ph * pw:
        raise ValueError(f"qf.unpatchify: bias has {bias.numel} elements, expected {C * ph * pw}")
    if out is None:
        out = QuarkTensor.empty(B, C * H * W, dtype="bf16")
    elif out.numel != C * H * W:
        raise ValueError(f"qf.unpatchify: out is {out.shape}, expected ({B}, {C * H * W})")
    n_out = C * ph * pw
    if d_model % 16 == 0 and n_out % 8 == 0:  # tensor-core route: one GEMM (bias in its epilogue), then scatter
        tmp = _scratch("unpatchify", (tokens, n_out), "bf16")
        gemm(X.reshape(tokens, d_model), weight, out_dtype="bf16", bias=bias, out=tmp, b_constant=True)
        _lib.check(_lib.load().qb_patch_scatter(_p(tmp), _p(out), C, H, W, ph, pw, _s()))
        return out
    _lib.check(_lib.load().qb_unpatchify(_p(X), _p(weight), _p(bias), _p(out), C, H, W, ph, pw, d_model, _s()))
    return out
