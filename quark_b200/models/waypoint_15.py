"""Waypoint-1.5 DiT: config, block wiring, one NFE, one generated frame.

Mirrors ``src/quark/models/waypoint_15.py``: ``QuantConfig`` (``:46-76``), ``Waypoint15Config``
(``:79-171``), ``TransformerBlock`` (``:259-440``), ``Waypoint15`` (``:448-661``) and
``GenerateFrame`` (``:664-766``) with the same field and method names.  Not carried over: the
capacity-bounded MoE routings, checkpoint download from a hub.  Weights come from ``make_params`` (seeded random init),
from a local checkpoint (``checkpoint.load_checkpoint``) or any dict of the same layout, through
``Waypoint15.load_params``.
"""

from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field

import numpy as np

from .. import functional as qf
from .. import nn
from ..runtime import stream as _stream
from ..runtime.tensor import QuarkTensor
from . import _cond


@dataclass(frozen=True)
class QuantConfig:
    """Per-component ``"fp8"`` / ``"bf16"`` switches (``src/quark/models/waypoint_15.py:46-76``)."""

    linear: str = "fp8"
    kv_cache: str = "fp8"
    attn_compute: str = "fp8"
    moe: str = "fp8"

    def __post_init__(self) -> None:
        for name in ("linear", "kv_cache", "attn_compute", "moe"):
            v = getattr(self, name)
            if v not in ("fp8", "bf16"):
                raise ValueError(f"QuantConfig.{name}: must be 'fp8' or 'bf16', got {v!r}")

    @classmethod
    def all_bf16(cls) -> "QuantConfig":
        return cls(linear="bf16", kv_cache="bf16", attn_compute="bf16", moe="bf16")

    @classmethod
    def all_fp8(cls) -> "QuantConfig":
        return cls()


@dataclass(frozen=True)
class Waypoint15Config:
    d_model: int = 2048
    n_layers: int = 24
    n_heads: int = 32
    n_kv_heads: int = 16
    mlp_ratio: int = 4
    channels: int = 32
    patch: tuple[int, int] = (2, 2)
    height: int = 16
    width: int = 32
    local_window: int = 16
    global_window: int = 128
    global_pinned_dilation: int = 8
    global_attn_period: int = 4
    global_attn_offset: int = -1
    value_residual: bool = True
    fourier_dim: int = 512
    scheduler_sigmas: tuple[float, ...] = (1.0, 0.9, 0.75, 0.3, 0.0)
    # Controller conditioning (mouse / buttons / scroll folded into every ctrl_conditioning_period-th block,
    # ref: src/quark/models/waypoint_15.py:98-100, :349-366).  The reference's default is on; random-init
    # benchmark configurations run with ctrl_emb = None, so the default here is off.
    ctrl_conditioning: bool = False
    ctrl_conditioning_period: int = 3
    n_buttons: int = 256
    quant: QuantConfig = field(default_factory=QuantConfig.all_bf16)
    quilt_factor: int = 1
    # Mixture-of-experts MLP (src/quark/models/waypoint_15.py:113-130): moe_n_experts experts of width
    # mlp_dim / moe_top_k, each token using its top moe_top_k.  Only moe_routing = "correct" is implemented.
    moe: bool = False
    moe_n_experts: int = 8
    moe_top_k: int = 2
    moe_routing: str = "correct"
    # Fold `x + gate * y` into the out-proj / fc2 GEMM epilogue (upstream field, default off there).
    fuse_gate_residual: bool = True
    # Fold SiLU into fc1's epilogue (upstream does on its PTX / Metal GEMMs, not on the cuBLAS route).
    fuse_silu: bool = True
    # head_rmsnorm + value residual + KV append as one launch (bit-identical to the three).
    fuse_qkv_post: bool = True
    # ... and that launch folded into the QKV projection's epilogue (same bytes again); needs fuse_qkv_post.
    fuse_qkv_gemm: bool = True
    # Scaled e4m3 (an extension; the reference's e4m3 is scale free): linear weights narrowed with one scale per
    # output channel (amax / 448), the caches with one scale per KV head (`k_scale` / `v_scale` of each block's
    # parameters).  Only meaningful where quant says fp8; the mixture-of-experts weights stay unscaled.
    fp8_scales: bool = False
    # Tensor parallelism by KV-head group: rank `tp_rank` of `tp_world` owns n_kv_heads / tp_world KV heads
    # with their Q heads (QKV and fc1 column-parallel, out-proj and fc2 row-parallel, partial outputs summed
    # over the ranks).  The reference is single-GPU; tp_world = 1 is its wiring.
    tp_world: int = 1
    tp_rank: int = 0

    def __post_init__(self):
        if self.ctrl_conditioning and (self.ctrl_conditioning_period < 1 or self.n_buttons < 0):
            raise ValueError("Waypoint15Config: ctrl_conditioning_period must be positive and n_buttons non-negative")
        if self.moe:
            if self.moe_routing != "correct":
                raise NotImplementedError(f"Waypoint15Config: moe_routing {self.moe_routing!r} is not implemented (only 'correct')")
            if self.tp_world > 1:
                raise NotImplementedError("Waypoint15Config: MoE with tp_world > 1 is not implemented")
            # the router is a GEMM with one output column per expert: a multiple of 8 columns
            if not (1 <= self.moe_top_k <= self.moe_n_experts <= 32) or self.moe_n_experts % 8 or (self.d_model * self.mlp_ratio) % (8 * self.moe_top_k):
                raise ValueError(f"Waypoint15Config: moe_top_k {self.moe_top_k} of {self.moe_n_experts} experts over an MLP of {self.d_model * self.mlp_ratio}")
        q = self.quilt_factor
        if q < 1 or q & (q - 1) or (self.height * self.width) % q:
            raise ValueError(f"Waypoint15Config: quilt_factor {q} must be a power of two that divides height * width")
        if self.d_model // self.n_heads != 64:
            raise NotImplementedError("Waypoint15Config: only head_dim 64 is supported")
        if self.tp_world < 1 or not (0 <= self.tp_rank < self.tp_world):
            raise ValueError(f"Waypoint15Config: tp_rank {self.tp_rank} of tp_world {self.tp_world}")
        if self.n_kv_heads % self.tp_world or (self.d_model * self.mlp_ratio) % (128 * self.tp_world):
            raise ValueError(f"Waypoint15Config: {self.n_kv_heads} KV heads / MLP width do not divide over {self.tp_world} ranks")

    @property
    def Dh(self):
        return self.d_model // self.n_heads

    @property
    def mlp_dim(self):
        return self.d_model * self.mlp_ratio

    @property
    def gqa_ratio(self):
        return self.n_heads // self.n_kv_heads

    @property
    def tpf(self):
        return self.height * self.width

    @property
    def qkv_dim(self):
        return (self.n_heads + 2 * self.n_kv_heads) * self.Dh

    @property
    def v_col_offset(self):
        return (self.n_heads + self.n_kv_heads) * self.Dh

    @property
    def v_width(self):
        return self.n_kv_heads * self.Dh

    # ---- this rank's share (everything when tp_world == 1)
    @property
    def n_heads_local(self):
        return self.n_heads // self.tp_world

    @property
    def n_kv_heads_local(self):
        return self.n_kv_heads // self.tp_world

    @property
    def qkv_dim_local(self):
        return (self.n_heads_local + 2 * self.n_kv_heads_local) * self.Dh

    @property
    def mlp_dim_local(self):
        return self.mlp_dim // self.tp_world

    @property
    def ctrl_input_width(self):
        """Controller row: mouse x, mouse y, one flag per button, scroll wheel, padded to a multiple of 16."""
        return (self.n_buttons + 3 + 15) // 16 * 16

    def has_ctrl(self, layer):
        return self.ctrl_conditioning and layer % self.ctrl_conditioning_period == 0

    @property
    def latent_numel(self):
        return self.channels * self.height * self.patch[0] * self.width * self.patch[1]

    def is_global(self, layer):
        return (layer - self.global_attn_offset) % self.global_attn_period == 0

    def num_buckets(self, layer):
        return self.global_window // self.global_pinned_dilation if self.is_global(layer) else self.local_window

    def pinned_dilation(self, layer):
        return self.global_pinned_dilation if self.is_global(layer) else 1

    _YAML_SCALARS = ("d_model", "n_layers", "n_heads", "n_kv_heads", "mlp_ratio", "channels", "height", "width", "local_window",
                     "global_window", "global_pinned_dilation", "global_attn_period", "global_attn_offset", "value_residual",
                     "fourier_dim", "n_buttons", "ctrl_conditioning_period", "moe", "moe_n_experts", "moe_top_k", "moe_routing",
                     "quilt_factor")  # fmt: skip

    @classmethod
    def from_dict(cls, raw: dict, **overrides) -> "Waypoint15Config":
        """From the mapping of a training ``config.yaml`` (``src/quark/models/waypoint_15.py:173-219``): known
        fields are taken, the rest (autoencoder URI, prompt conditioning, frame rate ...) is the caller's concern;
        ``ctrl_conditioning`` there is the controller specification, and only whether it is present matters."""
        kw = {k: raw[k] for k in cls._YAML_SCALARS if k in raw}
        if "patch" in raw:
            kw["patch"] = tuple(raw["patch"])
        if "scheduler_sigmas" in raw:
            kw["scheduler_sigmas"] = tuple(float(s) for s in raw["scheduler_sigmas"])
        if "ctrl_conditioning" in raw:
            kw["ctrl_conditioning"] = raw["ctrl_conditioning"] is not None
        kw.update(overrides)
        return cls(**kw)

    @classmethod
    def from_yaml(cls, model_uri, **overrides) -> "Waypoint15Config":
        """``model_uri``: a ``config.yaml`` or a directory holding one.  A hub repository id cannot be resolved
        (no download client here) and raises ``FileNotFoundError``."""
        from .checkpoint import load_yaml_config

        return cls.from_dict(load_yaml_config(model_uri), **overrides)


# ---------------------------------------------------------------------------
# seeded random-init parameters (host numpy, bf16 carriers)
# ---------------------------------------------------------------------------


def _randn_bf16(rng, shape, std):
    a = rng.standard_normal(shape, dtype=np.float32)
    a *= np.float32(std)
    return _cond._bf16(a)


def make_params(cfg: Waypoint15Config, seed: int = 0, *, weight_std: float = 0.02, threads: int = 8) -> dict:
    """Random-init parameters of the hot path, as host arrays.

    Linear weights are N(0, ``weight_std``) in bf16; the per-sigma noise embedding is a seeded
    N(0, 1) vector of d_model; the conditioning rows follow from it through random-init cond heads
    with the reference's host arithmetic (``_cond.block_rows``).  Layer ``i`` uses the generator
    ``default_rng([seed, i])`` so layers are independent and reproducible one at a time.

    Layout: ``patchify.weight``, ``unpatchify.weight``, ``unpatchify.bias``, ``out_norm.lut`` (list over
    sigma of two rows) and ``blocks`` (list of dicts: ``qkv.weight``, ``out.weight``, ``fc1.weight``,
    ``fc2.weight``, ``lamb``, ``lut`` = list over sigma of six rows).
    """
    d, ns = cfg.d_model, len(cfg.scheduler_sigmas)
    kpatch = cfg.channels * cfg.patch[0] * cfg.patch[1]
    r0 = np.random.default_rng([seed, 1_000_000])
    emb = r0.standard_normal((ns, d), dtype=np.float32)
    params = {
        "patchify.weight": _randn_bf16(r0, (d, kpatch), weight_std),
        "unpatchify.weight": _randn_bf16(r0, (kpatch, d), weight_std),
        "unpatchify.bias": _randn_bf16(r0, (kpatch,), weight_std),
    }
    on_w = _cond.bf16_to_f32(_randn_bf16(r0, (2 * d, d), weight_std))
    params["out_norm.lut"] = [_cond.out_norm_rows(emb[si], on_w) for si in range(ns)]

    def one_layer(i):
        r = np.random.default_rng([seed, i])
        blk = {
            "qkv.weight": _randn_bf16(r, (cfg.qkv_dim, d), weight_std),
            "out.weight": _randn_bf16(r, (d, cfg.n_heads * cfg.Dh), weight_std),
            "fc1.weight": _randn_bf16(r, (cfg.mlp_dim, d), weight_std),
            "fc2.weight": _randn_bf16(r, (d, cfg.mlp_dim), weight_std),
            "lamb": 0.5,
        }
        if cfg.fp8_scales:  # per-KV-head cache scales: what a calibration run would leave (K is RMS-normalised: |k| <= 8)
            rs = np.random.default_rng([seed, i, 13])
            blk["k_scale"] = ((8.0 / 448.0) * (1.0 + 0.25 * rs.random(cfg.n_kv_heads))).astype(np.float32)
            blk["v_scale"] = ((6.0 / 448.0) * (1.0 + 0.25 * rs.random(cfg.n_kv_heads))).astype(np.float32)
        if cfg.moe:  # a generator of its own; layouts of src/quark/nn/moe.py:35-38
            rm = np.random.default_rng([seed, i, 11])
            E, Hm = cfg.moe_n_experts, cfg.mlp_dim // cfg.moe_top_k
            blk["moe.router.weight"] = _randn_bf16(rm, (E, d), 10 * weight_std)  # spread logits, so routing is not a coin toss
            blk["moe.expert_in"] = _randn_bf16(rm, (E * Hm, d), weight_std)
            blk["moe.expert_out"] = _randn_bf16(rm, (E * d, Hm), weight_std)
        ab = _cond.bf16_to_f32(_randn_bf16(r, (d,), weight_std))
        mb = _cond.bf16_to_f32(_randn_bf16(r, (d,), weight_std))
        projs = [_cond.bf16_to_f32(_randn_bf16(r, (d, d), weight_std)) for _ in range(6)]
        blk["lut"] = [_cond.block_rows(emb[si], ab, mb, projs) for si in range(ns)]
        if cfg.has_ctrl(i):  # a generator of its own: the weights above do not depend on this switch
            rc = np.random.default_rng([seed, i, 7])
            for k in ("ctrl.fc1_x.weight", "ctrl.fc1_c.weight", "ctrl.fc2.weight"):
                blk[k] = _randn_bf16(rc, (d, d), weight_std)
        return blk

    if cfg.ctrl_conditioning:
        rc = np.random.default_rng([seed, 2_000_000])
        params["ctrl_emb.fc1.weight"] = _randn_bf16(rc, (cfg.mlp_dim, cfg.ctrl_input_width), weight_std)
        params["ctrl_emb.fc2.weight"] = _randn_bf16(rc, (d, cfg.mlp_dim), weight_std)
    with ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
        params["blocks"] = list(ex.map(one_layer, range(cfg.n_layers)))
    return params


def shard_block_params(cfg: Waypoint15Config, blk: dict) -> dict:
    """The slices of one block's weights that rank ``cfg.tp_rank`` owns.

    QKV rows are regrouped as ``[Q heads | K heads | V heads]`` of the rank's KV-head group, so the
    packed layout (and with it every kernel) is the single-GPU one with fewer heads; out-proj keeps the
    columns of the rank's Q heads, fc1 a row block, fc2 the matching column block.  Conditioning rows,
    ``lamb`` and everything outside the blocks are replicated.
    """
    G, r, Dh = cfg.tp_world, cfg.tp_rank, cfg.Dh
    if G == 1:
        return blk
    nq, nk = cfg.n_heads_local * Dh, cfg.n_kv_heads_local * Dh
    k0, v0 = cfg.n_heads * Dh, (cfg.n_heads + cfg.n_kv_heads) * Dh
    w = np.asarray(blk["qkv.weight"])
    out = dict(blk)
    out["qkv.weight"] = np.ascontiguousarray(np.concatenate([w[r * nq : (r + 1) * nq], w[k0 + r * nk : k0 + (r + 1) * nk], w[v0 + r * nk : v0 + (r + 1) * nk]]))
    out["out.weight"] = np.ascontiguousarray(np.asarray(blk["out.weight"])[:, r * nq : (r + 1) * nq])
    m = cfg.mlp_dim_local
    out["fc1.weight"] = np.ascontiguousarray(np.asarray(blk["fc1.weight"])[r * m : (r + 1) * m])
    out["fc2.weight"] = np.ascontiguousarray(np.asarray(blk["fc2.weight"])[:, r * m : (r + 1) * m])
    for k in ("k_scale", "v_scale"):
        if blk.get(k) is not None:
            out[k] = np.ascontiguousarray(np.asarray(blk[k])[r * cfg.n_kv_heads_local : (r + 1) * cfg.n_kv_heads_local])
    return out


# ---------------------------------------------------------------------------
# model
# ---------------------------------------------------------------------------


class TransformerBlock(nn.Module):
    def __init__(self, cfg: Waypoint15Config, layer_idx: int, comm=None):
        d = cfg.d_model
        self._cfg = cfg
        self._comm = comm
        if cfg.tp_world > 1 and (comm is None or comm.world != cfg.tp_world or comm.rank != cfg.tp_rank):
            raise ValueError("TransformerBlock: tp_world > 1 needs a communicator of that size and rank")
        self._cond_lut: list[tuple] = []
        nq, nk = cfg.n_heads_local, cfg.n_kv_heads_local  # heads of this rank
        self.pre_attn_norm = nn.AdaRMSNorm()
        self.qkv_proj = nn.Linear(d, cfg.qkv_dim_local, out_dtype="bf16")
        self.head_norm = nn.HeadRMSNorm(nq, nk, cfg.Dh)
        if cfg.value_residual:
            self.v_residual = nn.ValueResidualPacked((nq + nk) * cfg.Dh, nk * cfg.Dh)
        kv_dt = "e4m3" if cfg.quant.kv_cache == "fp8" else "bf16"
        geo = dict(B=1, n_kv_heads=nk, H_spatial=cfg.height, W_spatial=cfg.width, num_buckets=cfg.num_buckets(layer_idx),
                   pinned_dilation=cfg.pinned_dilation(layer_idx), packed_qkv=True)  # fmt: skip
        if cfg.quilt_factor > 1:
            # each layer's cache keeps one residue class of the frame's tokens, the classes taking turns over the
            # layers (src/quark/models/waypoint_15.py:311-316)
            geo.update(quilt_factor=cfg.quilt_factor, quilt_offset=layer_idx % cfg.quilt_factor)
        self.kv_cache = nn.KVCacheUpdate(n_q_heads=nq, Dh=cfg.Dh, dtype=kv_dt, **geo)
        self.attn = nn.OwlAttn(gqa_ratio=cfg.gqa_ratio, compute_dtype="e4m3" if cfg.quant.attn_compute == "fp8" else None, **geo)
        self.out_proj = nn.Linear(nq * cfg.Dh, d, out_dtype="bf16")
        self.attn_gate = nn.AdaGateResidual()
        if cfg.has_ctrl(layer_idx):
            if cfg.tp_world > 1:
                raise NotImplementedError("TransformerBlock: controller conditioning with tp_world > 1 is not implemented")
            # bf16 end to end, also under fp8 (src/quark/models/waypoint_15.py:349-366)
            self.ctrl_fusion = nn.MLPFusion(d, out_dtype="bf16")
            self.ctrl_x_norm = nn.RMSNorm()
            self.ctrl_emb_norm = nn.RMSNorm()
            self.ctrl_residual = nn.Add()
        self.pre_mlp_norm = nn.AdaRMSNorm()
        if cfg.moe:
            self.mlp = nn.MoE(cfg.tpf, d, cfg.mlp_dim // cfg.moe_top_k, cfg.moe_n_experts, cfg.moe_top_k, routing=cfg.moe_routing)
        else:
            self.mlp = nn.MLP(d, cfg.mlp_dim_local, d, out_dtype="bf16", fuse_silu=cfg.fuse_silu)
        self.mlp_gate = nn.AdaGateResidual()

    def forward(self, x, sigma_idx: int, frame_t, *, qkv_first, ctrl_emb=None, frozen: bool = False, x_out=None, h_in=None, next_norm=None):
        """Returns ``(x, qkv)`` (``src/quark/models/waypoint_15.py:389-440``).

        Tensor-parallel ranks with a fused reduction (``comm.fused``): the sum over the ranks, gate + residual and the
        AdaRMSNorm that follows are one kernel, so the pre-MLP norm never runs as a launch of its own, and the norm that
        follows the block (``next_norm = (scale, bias, activation, emit_e4m3)``: the next block's pre-attention norm, or
        the output norm) is produced by this block's last reduction and left in ``self.h_next``; ``h_in`` is what the
        previous block left there."""
        s0, b0, g0, s1, b1, g1 = self._cond_lut[sigma_idx]
        fp8 = self.qkv_proj.weight.data.dtype == "e4m3"
        tp = self._cfg.tp_world > 1
        tp_fused = tp and getattr(self._comm, "fused", False)
        # row-parallel partial outputs are summed over the ranks before gate and residual are applied (once)
        fuse = self._cfg.fuse_gate_residual and not tp
        self.h_next = None
        arena = self._comm.arena(x.numel // int(x.shape[-1]), int(x.shape[-1])) if tp_fused else None

        h0 = h_in if h_in is not None else self.pre_attn_norm(x, s0, b0, emit_e4m3=fp8)
        use_first = hasattr(self, "v_residual") and qkv_first is not None
        # the stand-alone fused post-processing kernel appends every token; a quilted cache goes through the GEMM epilogue
        # (which knows the quilt) or the plain kernels.  The epilogue stores whole 16-byte vectors of cached V tokens per
        # 128-token tile, which bounds the quilt factor it takes (8 for e4m3 caches, 16 for bf16)
        quilted = self._cfg.quilt_factor > 1
        kc = self.kv_cache
        quilt_fits = self._cfg.quilt_factor * (16 if kc.K_cache.dtype == "e4m3" else 8) <= 128
        if self._cfg.fuse_qkv_post and self._cfg.fuse_qkv_gemm and quilt_fits:
            kc = self.kv_cache
            qkv = qf.gemm_qkv_post(
                h0, self.qkv_proj.weight.data, qkv_first if use_first else None, self.v_residual.lamb.data if use_first else None,
                frame_t if frame_t is not None else kc.frame_t, kc._frozen[1 if frozen else 0], kc.Vt_cache, kc.segments, kc.n_segments,
                kc.K_cache, n_q_heads=self._cfg.n_heads_local, n_kv_heads=self._cfg.n_kv_heads_local, H_spatial=self._cfg.height,
                W_spatial=self._cfg.width, num_buckets=kc._kw["num_buckets"], pinned_dilation=kc._kw["pinned_dilation"],
                out=nn._cached(self, "qkv_post", (h0.numel // int(h0.shape[-1]), self._cfg.qkv_dim_local), "bf16"),
                w_scale=self.qkv_proj.w_scale, k_scale=kc.k_scale, v_scale=kc.v_scale,
                quilt_factor=kc._kw["quilt_factor"], quilt_offset=kc._kw["quilt_offset"],
            )  # fmt: skip
        elif self._cfg.fuse_qkv_post and not quilted:
            qkv = self.qkv_proj(h0)
            kc = self.kv_cache
            qkv = qf.qkv_post(
                qkv, qkv_first if use_first else None, self.v_residual.lamb.data if use_first else None,
                frame_t if frame_t is not None else kc.frame_t, kc._frozen[1 if frozen else 0], kc.Vt_cache, kc.segments, kc.n_segments,
                kc.K_cache, n_q_heads=self._cfg.n_heads_local, n_kv_heads=self._cfg.n_kv_heads_local, H_spatial=self._cfg.height,
                W_spatial=self._cfg.width, num_buckets=kc._kw["num_buckets"], pinned_dilation=kc._kw["pinned_dilation"],
                out=nn._cached(self, "qkv_post", qkv.shape, "bf16"), k_scale=kc.k_scale, v_scale=kc.v_scale,
            )  # fmt: skip
        else:
            qkv = self.head_norm(self.qkv_proj(h0))
            if use_first:
                qkv = self.v_residual(qkv, qkv_first)
            self.kv_cache(qkv, frame_t, frozen=frozen)
        attn_out = self.attn(qkv, self.kv_cache, frame_t, emit_e4m3=fp8, frozen=frozen)
        h = None
        if fuse:
            x = self.out_proj(attn_out, gate=g0, residual=x, gate_groups=int(g0.shape[0]))
        elif tp_fused:
            sched = self._comm.tp_schedule
            pushed = sched == 3 and self.out_proj.w_scale is None  # scaled weights need the GEMM's epilogue: keep the partial local
            if pushed:
                self.out_proj(attn_out, tp_arena=arena)  # every row of the partial goes straight to the rank that sums it
            else:
                self.out_proj(attn_out, out=arena.y[0])  # the partial goes into this rank's peer-mapped buffer
            x, h = arena.reduce(x, g0, s1, b1, x_slot=0, emit_e4m3=fp8, schedule=sched if pushed or sched != 3 else 0)
        else:
            y = self.out_proj(attn_out)
            if tp:
                self._comm.all_reduce_sum(y)
            x = self.attn_gate(x, y, g0)
        if ctrl_emb is not None and hasattr(self, "ctrl_fusion"):
            x = self.ctrl_residual(x, self.ctrl_fusion(self.ctrl_x_norm(x), self.ctrl_emb_norm(ctrl_emb)))
        moe = self._cfg.moe
        if h is None:
            h = self.pre_mlp_norm(x, s1, b1, emit_e4m3=fp8 and not moe)  # the router reads bf16; MoE narrows for its experts itself
        if moe:
            x = self.mlp_gate(x, self.mlp(h), g1)
        elif fuse:
            x = self.mlp(h, gate=g1, residual=x, gate_groups=int(g1.shape[0]), out=x_out)
        elif tp_fused:
            if pushed:
                self.mlp(h, tp_arena=arena)
            else:
                self.mlp(h, out=arena.y[1])
            ns, nb_, act, emit = next_norm if next_norm is not None else (None, None, None, False)
            x, self.h_next = arena.reduce(x, g1, ns, nb_, activation=act, x_slot=1, emit_e4m3=emit, schedule=sched if pushed or sched != 3 else 0)
        else:
            y = self.mlp(h)
            if tp:
                self._comm.all_reduce_sum(y)
            x = self.mlp_gate(x, y, g1)
        return x, qkv


class Waypoint15(nn.Module):
    def __init__(self, cfg: Waypoint15Config | None = None, comm=None):
        self.cfg = cfg = cfg or Waypoint15Config()
        self.comm = comm
        ph, pw = cfg.patch
        self.patchify = nn.Patchify(cfg.channels, cfg.d_model, cfg.height * ph, cfg.width * pw, ph, pw)
        self.blocks = nn.ModuleList([TransformerBlock(cfg, i, comm) for i in range(cfg.n_layers)])
        self.out_norm = nn.AdaRMSNorm()
        self.unpatchify = nn.Unpatchify(cfg.d_model, cfg.channels, cfg.height * ph, cfg.width * pw, ph, pw)
        if cfg.ctrl_conditioning:
            self.ctrl_emb = nn.ControllerInputEmbedding(cfg.n_buttons, cfg.d_model, cfg.mlp_ratio, out_dtype="bf16")
        self._out_norm_luts: list[tuple] = []
        # Two residual-stream buffers used alternately by consecutive blocks when the gate/residual
        # epilogue is fused: a GEMM must not write the tensor it reads its residual from.
        self._x_bufs = None

    def load_params(self, params: dict) -> "Waypoint15":
        """Upload a ``make_params``-style dict (full-size weights; a tensor-parallel rank keeps its slices);
        call ``prepare()`` afterwards."""
        up = lambda a: QuarkTensor.from_numpy(np.asarray(a), dtype="bf16")  # noqa: E731
        self.patchify.weight.data = up(params["patchify.weight"])
        self.unpatchify.weight.data = up(params["unpatchify.weight"])
        self.unpatchify.bias.data = up(params["unpatchify.bias"])
        self._out_norm_luts = [tuple(up(r) for r in rows) for rows in params["out_norm.lut"]]
        if hasattr(self, "ctrl_emb"):
            self.ctrl_emb.fc1.weight.data = up(params["ctrl_emb.fc1.weight"])
            self.ctrl_emb.fc2.weight.data = up(params["ctrl_emb.fc2.weight"])
        for blk, p in zip(self.blocks, params["blocks"]):
            p = shard_block_params(self.cfg, p)
            blk.qkv_proj.weight.data = up(p["qkv.weight"])
            blk.out_proj.weight.data = up(p["out.weight"])
            if self.cfg.moe:
                blk.mlp.router.weight.data = up(p["moe.router.weight"])
                blk.mlp.expert_in.data = up(p["moe.expert_in"])
                blk.mlp.expert_out.data = up(p["moe.expert_out"])
            else:
                blk.mlp.fc1.weight.data = up(p["fc1.weight"])
                blk.mlp.fc2.weight.data = up(p["fc2.weight"])
            if hasattr(blk, "ctrl_fusion"):
                blk.ctrl_fusion.fc1_x.weight.data = up(p["ctrl.fc1_x.weight"])
                blk.ctrl_fusion.fc1_c.weight.data = up(p["ctrl.fc1_c.weight"])
                blk.ctrl_fusion.fc2.weight.data = up(p["ctrl.fc2.weight"])
            if hasattr(blk, "v_residual"):
                blk.v_residual.lamb.data = QuarkTensor.from_numpy(np.array([p["lamb"]], dtype=np.float32))
            if self.cfg.fp8_scales and self.cfg.quant.kv_cache == "fp8":
                blk.kv_cache.set_scales(p.get("k_scale"), p.get("v_scale"))
            blk._cond_lut = [tuple(up(r) for r in rows) for rows in p["lut"]]
        return self

    def prepare(self, **kwargs):
        """Quantise linear weights when ``cfg.quant.linear == "fp8"`` (``waypoint_15.py:502-535``)."""
        kwargs.setdefault("fp8", self.cfg.quant.linear == "fp8")
        kwargs.setdefault("fp8_scaled", self.cfg.fp8_scales)
        for blk in self.blocks:
            for lin in (blk.qkv_proj, blk.out_proj) + (() if self.cfg.moe else (blk.mlp.fc1, blk.mlp.fc2)):
                lin.prepare(**kwargs)
            if self.cfg.moe:  # the experts follow quant.moe, independently of the other linears (waypoint_15.py:505-517)
                blk.mlp.prepare(moe_fp8=self.cfg.quant.moe == "fp8")
        _stream.synchronize()

    def encode_ctrl(self, ctrl_input):
        """The padded controller row ``[1, ctrl_input_width]`` (bf16) -> ``ctrl_emb [1, d_model]``, once per frame;
        None without controller conditioning or without an input (``src/quark/models/waypoint_15.py:597-611``)."""
        if ctrl_input is None or not hasattr(self, "ctrl_emb"):
            return None
        if ctrl_input.dtype != "bf16" or tuple(ctrl_input.shape) != (1, self.cfg.ctrl_input_width):
            raise TypeError(f"encode_ctrl: expected a bf16 [1, {self.cfg.ctrl_input_width}] row, got {ctrl_input.dtype} {ctrl_input.shape}")
        return self.ctrl_emb(ctrl_input)

    def set_frame_t(self, value: int) -> None:
        for blk in self.blocks:
            blk.kv_cache.set_frame_t(value)

    def reset(self) -> None:
        for blk in self.blocks:
            blk.kv_cache.reset()

    def forward(self, latent, sigma_idx: int, frame_t=None, ctrl_emb=None, frozen: bool = False):
        """One NFE on a ``[1, C*2H*2W]`` bf16 latent (``src/quark/models/waypoint_15.py:626-661``)."""
        if latent.dtype != "bf16" or latent.numel != self.cfg.latent_numel:
            raise TypeError(f"Waypoint15: latent must be bf16 with {self.cfg.latent_numel} elements, got {latent.dtype} {latent.shape}")
        s_on, b_on = self._out_norm_luts[sigma_idx]
        x = self.patchify(latent)
        if self._x_bufs is None:
            self._x_bufs = (QuarkTensor.empty(*x.shape, dtype="bf16"), QuarkTensor.empty(*x.shape, dtype="bf16"))
        qkv_first = None
        fp8 = self.cfg.quant.linear == "fp8"
        h_in = None
        for li, block in enumerate(self.blocks):
            # what follows this block's last reduction (used by tensor-parallel ranks with the fused reduction only)
            if li + 1 < len(self.blocks):
                nlut = self.blocks[li + 1]._cond_lut[sigma_idx]
                next_norm = (nlut[0], nlut[1], None, fp8)
            else:
                next_norm = (s_on, b_on, "silu", False)
            x, qkv = block(x, sigma_idx, frame_t, qkv_first=qkv_first, ctrl_emb=ctrl_emb, frozen=frozen, x_out=self._x_bufs[li & 1], h_in=h_in,
                           next_norm=next_norm)  # fmt: skip
            h_in = block.h_next
            if li == 0 and self.cfg.value_residual:
                qkv_first = qkv
        x = h_in if h_in is not None else self.out_norm(x, s_on, b_on, activation="silu")
        return self.unpatchify(x)


class GenerateFrame(nn.Module):
    """encode (none) -> 4 Euler denoise steps -> commit pass -> ``frame_t += 1`` (``waypoint_15.py:664-766``).

    ``prepare_graph`` runs the frame once eagerly (so every cached buffer exists), captures it into
    one CUDA graph, and rewinds ``frame_t``; afterwards ``__call__`` copies the noise into the
    captured input buffer and replays.
    """

    def __init__(self, model: Waypoint15):
        self.model = model
        sig = model.cfg.scheduler_sigmas
        self.n_denoise = len(sig) - 1
        self.dsig_tensors = [QuarkTensor.from_numpy(np.array([float(sig[i + 1] - sig[i])], dtype=np.float32)) for i in range(self.n_denoise)]
        self.euler_steps = nn.ModuleList([nn.EulerStep() for _ in range(self.n_denoise)])
        self.frame_t = QuarkTensor.zeros(1, dtype="s32")
        self._graph = None
        self._ctrl_in = None
        self._in = None
        self._out = None
        self.launches_per_frame = 0  # kernels in the captured frame graph

    def set_frame_t(self, value: int) -> None:
        self.frame_t.copy_from_numpy(np.array([value], dtype=np.int32))

    def reset(self) -> None:
        self.model.reset()
        self.set_frame_t(0)

    def forward(self, latent, ctrl_input=None):
        ft = self.frame_t
        x = latent
        ctrl_emb = self.model.encode_ctrl(ctrl_input)
        for si in range(self.n_denoise):
            v = self.model(x, sigma_idx=si, frame_t=ft, ctrl_emb=ctrl_emb, frozen=True)
            x = self.euler_steps[si](x, v, self.dsig_tensors[si])
        self.model(x, sigma_idx=self.n_denoise, frame_t=ft, ctrl_emb=ctrl_emb)
        qf.increment(ft)
        return x

    def prepare_graph(self, example_latent, example_ctrl_input=None, *, start_frame_t: int = 0) -> None:
        """Warm up and capture.  The KV state after this call is what the warm-up and capture
        passes left (two commits of the example latent at ``start_frame_t``); callers that care
        restore or reset the caches afterwards."""
        self._in = QuarkTensor.empty(*example_latent.shape, dtype="bf16")
        self._in.copy_from(example_latent)
        self._ctrl_in = example_ctrl_input  # a persistent device row the caller refills per frame
        self.set_frame_t(start_frame_t)
        self.forward(self._in, self._ctrl_in)
        _stream.synchronize()
        self.set_frame_t(start_frame_t)
        from .. import _lib

        n0 = _lib.kernel_launch_count()
        with _stream.capture_graph() as cap:
            self._out = self.forward(self._in, self._ctrl_in)
        self.launches_per_frame = _lib.kernel_launch_count() - n0
        self._graph = cap.graph
        self.set_frame_t(start_frame_t)
        _stream.synchronize()

    def __call__(self, latent, ctrl_input=None):
        if self._graph is None:
            return self.forward(latent, ctrl_input)
        if ctrl_input is not None and ctrl_input is not self._ctrl_in:
            raise ValueError("GenerateFrame: the captured graph reads the controller row given to prepare_graph; refill that tensor")
        self._in.copy_from(latent)
        self._graph.launch()
        return self._out
