"""Chained CPU reference: conditioning tables, one block, one NFE, one generated frame.

Test infrastructure (see ``oracle/__init__.py``).  The per-kernel references of ``oracle/ops.py``
are chained exactly as the reference model chains its kernels:

* ``noise_embedding`` / ``cond_rows`` / ``out_norm_rows``
                       follow ``src/quark/models/_waypoint_15_io.py:385-478``
* ``block_forward``    follows ``TransformerBlock.forward`` (``src/quark/models/waypoint_15.py:389-440``)
* ``nfe_forward``      follows ``Waypoint15.forward``        (``src/quark/models/waypoint_15.py:626-661``)
* ``gen_frame``        follows ``GenerateFrame.forward``     (``src/quark/models/waypoint_15.py:755-766``)

``cfg`` is any object with the attribute names of the reference's ``Waypoint15Config``
(``src/quark/models/waypoint_15.py:79-171``).  ``params`` is a dict of numpy carrier arrays:

    patchify.weight [d, C*ph*pw]   unpatchify.weight [C*ph*pw, d]   unpatchify.bias [C*ph*pw]
    out_norm.lut    list over sigma of (scale_row, bias_row)
    blocks[i]: qkv.weight, out.weight, fc1.weight, fc2.weight (bf16 or e4m3 carriers),
               lamb (python float), lut = list over sigma of (s0, b0, g0, s1, b1, g1)

``state`` is a list over layers of dicts ``K_cache, Vt_cache, segments, n_segments`` that are
updated in place, like the device caches.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import ops
from .codec import from_f32, to_f32


@dataclass(frozen=True)
class Quant:
    """Mirror of the reference's ``QuantConfig`` (waypoint_15.py:46-76) for the chained oracle.

    ``mirror_operand_rounding`` additionally rounds GEMM activations and the rotated Q through
    e4m3 where the GPU kernels must (tensor cores take both operands in 8 bits).  The reference
    oracles keep those operands in f32 (gemm/reference.py:1-10).
    """

    linear: str = "bf16"
    kv_cache: str = "bf16"
    attn_compute: str = "bf16"
    mirror_operand_rounding: bool = True


def is_global(cfg, layer: int) -> bool:
    return (layer - cfg.global_attn_offset) % cfg.global_attn_period == 0


def num_buckets(cfg, layer: int) -> int:
    return cfg.global_window // cfg.global_pinned_dilation if is_global(cfg, layer) else cfg.local_window


def pinned_dilation(cfg, layer: int) -> int:
    return cfg.global_pinned_dilation if is_global(cfg, layer) else 1


# ---------------------------------------------------------------------------
# conditioning tables (host-side numpy in the reference as well)
# ---------------------------------------------------------------------------


def noise_embedding(sigmas, fourier_dim: int, w1_f32: np.ndarray, w2_f32: np.ndarray) -> np.ndarray:
    """``[n_sigma, d]`` f32 (``compute_noise_emb_numpy``, _waypoint_15_io.py:385-427)."""
    half = fourier_dim // 2
    freqs = np.array([10000.0 ** (-i / max(half - 1, 1)) for i in range(half)], dtype=np.float32)
    n = len(sigmas)
    fourier = np.zeros((n, 2 * half), dtype=np.float32)
    sqrt2 = math.sqrt(2.0)
    for i, s in enumerate(sigmas):
        phase = np.array([float(s) * 1000.0 * f for f in freqs], dtype=np.float32)
        fourier[i, :half] = sqrt2 * np.sin(phase)
        fourier[i, half:] = sqrt2 * np.cos(phase)
    h = fourier @ w1_f32.T
    h = h * (1.0 / (1.0 + np.exp(-h)))
    return h @ w2_f32.T


def cond_rows(emb_f32, attn_bias_f32, mlp_bias_f32, proj_ws_f32):
    """Six bf16 rows ``(s0, b0, g0, s1, b1, g1)`` for one sigma (_waypoint_15_io.py:445-463)."""
    h_attn = emb_f32 + attn_bias_f32
    h_attn = h_attn * (1.0 / (1.0 + np.exp(-h_attn)))
    h_mlp = emb_f32 + mlp_bias_f32
    h_mlp = h_mlp * (1.0 / (1.0 + np.exp(-h_mlp)))
    rows = [(h_attn if j < 3 else h_mlp) @ proj_ws_f32[j].T for j in range(6)]
    return tuple(from_f32(r.reshape(1, -1).astype(np.float32), "bf16") for r in rows)


def out_norm_rows(emb_f32, on_w_f32):
    """``(scale_row, bias_row)`` bf16 for the output norm (_waypoint_15_io.py:465-477)."""
    d = emb_f32.shape[0]
    h = emb_f32 * (1.0 / (1.0 + np.exp(-emb_f32)))
    ab = h @ on_w_f32.T
    return (
        from_f32(ab[:d].reshape(1, d).astype(np.float32), "bf16"),
        from_f32(ab[d:].reshape(1, d).astype(np.float32), "bf16"),
    )


# ---------------------------------------------------------------------------
# state
# ---------------------------------------------------------------------------


def new_state(cfg, quant: Quant):
    """Zeroed caches and the initial segment table (src/quark/nn/layers.py:879-884)."""
    tpf = cfg.height * cfg.width // getattr(cfg, "quilt_factor", 1)  # tokens of a frame that a cache keeps
    Dh = cfg.d_model // cfg.n_heads
    carrier = np.uint8 if quant.kv_cache == "fp8" else np.uint16
    st = []
    for i in range(cfg.n_layers):
        nb = num_buckets(cfg, i)
        cap = nb * tpf + tpf
        st.append(
            dict(
                K_cache=np.zeros((cfg.n_kv_heads * cap, Dh), dtype=carrier),
                Vt_cache=np.zeros((cfg.n_kv_heads * Dh, cap), dtype=carrier),
                segments=np.array([0, 0, nb * tpf, tpf, 0, 0], dtype=np.int32),
                n_segments=np.array([2], dtype=np.int32),
            )
        )
    return st


# ---------------------------------------------------------------------------
# block / NFE / frame
# ---------------------------------------------------------------------------


def _linear(x, blk, name, quant: Quant, **epi):
    """``blk[name]`` is the weight; ``blk[name + ".scale"]`` (optional) its per-output-channel scales (the scaled-e4m3
    extension: the reference's weights are narrowed without a scale)."""
    w = blk[name]
    if quant.linear == "fp8":
        return ops.gemm(x, w, b_dtype="e4m3", a_quant="e4m3" if quant.mirror_operand_rounding else None, w_scale=blk.get(name + ".scale"), **epi)
    return ops.gemm(x, w, **epi)


def block_forward(cfg, layer: int, blk: dict, st: dict, x, sigma_idx: int, frame_t: int, *, qkv_first, frozen: bool, quant: Quant,
                  tp_world: int = 1, reduce=None, ctrl_emb=None):  # fmt: skip
    """One transformer block; returns ``(x, qkv)`` (waypoint_15.py:389-440, ctrl_emb=None).

    ``tp_world > 1`` restates one rank of the sharding by KV-head group: ``blk`` holds that rank's weight
    slices, ``st`` its heads' caches, and ``reduce(partial_bf16) -> summed_bf16`` stands for the sum over
    the ranks after each row-parallel GEMM; gate and residual are applied once, after the sum.
    """
    s0, b0, g0, s1, b1, g1 = blk["lut"][sigma_idx]
    Hq, Hk = cfg.n_heads // tp_world, cfg.n_kv_heads // tp_world
    Dh = cfg.d_model // cfg.n_heads
    kv_dtype = "e4m3" if quant.kv_cache == "fp8" else "bf16"
    geo = dict(H_spatial=cfg.height, W_spatial=cfg.width)

    # per-KV-head cache scales of the scaled-e4m3 extension (absent: the reference's scale-free caches)
    ks, vs = (blk.get("k_scale"), blk.get("v_scale")) if quant.kv_cache == "fp8" else (None, None)
    h = ops.ada_rmsnorm(x, s0, b0)
    qkv = _linear(h, blk, "qkv.weight", quant)
    qkv = ops.head_rmsnorm(qkv, n_q_heads=Hq, n_kv_heads=Hk, Dh=Dh)
    if getattr(cfg, "value_residual", True) and qkv_first is not None:
        qkv = ops.value_residual_packed(qkv, qkv_first, blk["lamb"], v_col_offset=(Hq + Hk) * Dh, v_width=Hk * Dh)
    _, _, segs, nseg = ops.kv_cache_update(
        qkv,
        frame_t,
        int(frozen),
        n_kv_heads=Hk,
        n_q_heads=Hq,
        num_buckets=num_buckets(cfg, layer),
        pinned_dilation=pinned_dilation(cfg, layer),
        kv_dtype=kv_dtype,
        Dh=Dh,
        K_cache=st["K_cache"],
        Vt_cache=st["Vt_cache"],
        # each layer's cache keeps one residue class of the tokens, taking turns over the layers (waypoint_15.py:311-316)
        quilt_factor=getattr(cfg, "quilt_factor", 1),
        quilt_offset=layer % getattr(cfg, "quilt_factor", 1),
        k_scale=ks,
        v_scale=vs,
        **geo,
    )
    st["segments"][:] = segs
    st["n_segments"][:] = nseg
    Kc, Vc, attn_kv_dtype = st["K_cache"], st["Vt_cache"], kv_dtype
    if quant.kv_cache == "bf16" and quant.attn_compute == "fp8" and quant.mirror_operand_rounding:
        # e4m3 arithmetic over a bf16 cache: K and V are narrowed as they are loaded (kernels/owl_attn/kernel.py:342-348).
        # The opposite mix (e4m3 cache, bf16 arithmetic) needs nothing here: widening e4m3 is exact.
        Kc, Vc, attn_kv_dtype = from_f32(to_f32(Kc, "bf16"), "e4m3"), from_f32(to_f32(Vc, "bf16"), "e4m3"), "e4m3"
    attn = ops.owl_attn(
        qkv,
        Kc,
        Vc,
        st["segments"],
        st["n_segments"],
        frame_t,
        n_kv_heads=Hk,
        gqa_ratio=Hq // Hk,
        kv_dtype=attn_kv_dtype,
        Dh=Dh,
        q_quant="e4m3" if (quant.attn_compute == "fp8" and quant.mirror_operand_rounding) else None,
        k_scale=ks,
        v_scale=vs,
        **geo,
    )
    if reduce is None:
        x = _linear(attn, blk, "out.weight", quant, gate=g0, residual=x)
    else:
        x = ops.ada_gate_residual(x, reduce(_linear(attn, blk, "out.weight", quant)), g0)
    if ctrl_emb is not None and "ctrl.fc1_x.weight" in blk:
        # controller conditioning on every ctrl_conditioning_period-th block (waypoint_15.py:419-424); bf16 throughout
        x = ops.add(x, ops.mlp_fusion(ops.rmsnorm(x), ops.rmsnorm(ctrl_emb), blk["ctrl.fc1_x.weight"], blk["ctrl.fc1_c.weight"],
                                      blk["ctrl.fc2.weight"]))  # fmt: skip
    h = ops.ada_rmsnorm(x, s1, b1)
    if getattr(cfg, "moe", False):
        fp8 = getattr(quant, "moe", quant.linear) == "fp8"
        y = ops.moe(h, blk["moe.router.weight"], blk["moe.expert_in"], blk["moe.expert_out"], top_k=cfg.moe_top_k, fp8=fp8,
                    a_quant="e4m3" if (fp8 and quant.mirror_operand_rounding) else None)  # fmt: skip
        return ops.ada_gate_residual(x, y, g1), qkv
    h = ops.silu(_linear(h, blk, "fc1.weight", quant))
    if reduce is None:
        x = _linear(h, blk, "fc2.weight", quant, gate=g1, residual=x)
    else:
        x = ops.ada_gate_residual(x, reduce(_linear(h, blk, "fc2.weight", quant)), g1)
    return x, qkv


def nfe_forward(cfg, params: dict, state: list, latent, sigma_idx: int, frame_t: int, *, frozen: bool, quant: Quant, ctrl_emb=None):
    """One network evaluation on a ``[1, C*2H*2W]`` bf16 latent (waypoint_15.py:626-661)."""
    ph, pw = cfg.patch
    H2, W2 = cfg.height * ph, cfg.width * pw
    x = ops.patchify(latent, params["patchify.weight"], C=cfg.channels, H=H2, Wd=W2, ph=ph, pw=pw)
    qkv_first = None
    for li in range(cfg.n_layers):
        x, qkv = block_forward(cfg, li, params["blocks"][li], state[li], x, sigma_idx, frame_t, qkv_first=qkv_first, frozen=frozen, quant=quant,
                               ctrl_emb=ctrl_emb)  # fmt: skip
        if li == 0 and getattr(cfg, "value_residual", True):
            qkv_first = qkv
    s_on, b_on = params["out_norm.lut"][sigma_idx]
    x = ops.ada_rmsnorm(x, s_on, b_on, activation="silu")
    return ops.unpatchify(x, params["unpatchify.weight"], params["unpatchify.bias"], C=cfg.channels, H=H2, Wd=W2, ph=ph, pw=pw)


def gen_frame(cfg, params: dict, state: list, noise_latent, frame_t: int, *, quant: Quant, ctrl_input=None):
    """Four Euler denoise steps plus the commit pass; returns ``(latent, frame_t + 1)``.  ``ctrl_input`` is the
    padded controller row; it is embedded once per frame (waypoint_15.py:597-611, :755-766)."""
    sig = cfg.scheduler_sigmas
    x = noise_latent
    n = len(sig) - 1
    ctrl_emb = None
    if ctrl_input is not None and "ctrl_emb.fc1.weight" in params:
        ctrl_emb = ops.controller_embedding(ctrl_input, params["ctrl_emb.fc1.weight"], params["ctrl_emb.fc2.weight"])
    for si in range(n):
        v = nfe_forward(cfg, params, state, x, si, frame_t, frozen=True, quant=quant, ctrl_emb=ctrl_emb)
        x = ops.euler_step(x, v, float(sig[si + 1] - sig[si]))
    nfe_forward(cfg, params, state, x, n, frame_t, frozen=False, quant=quant, ctrl_emb=ctrl_emb)
    return x, frame_t + 1
