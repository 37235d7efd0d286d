"""``quark.nn`` modules on the hot path, same class names and constructor keywords.

Mirrors ``src/quark/nn/module.py:145-465`` (``Module`` / ``Parameter``) and the layers the
Waypoint-1.5 block uses (``src/quark/nn/layers.py``): ``Linear``, ``MLP``, ``AdaRMSNorm``,
``HeadRMSNorm``, ``ValueResidualPacked``, ``KVCacheUpdate``, ``OwlAttn``, ``AdaGateResidual``,
``Patchify``, ``Unpatchify``, ``EulerStep``, ``SiLU``.  Every module owns its output buffer, so a
forward pass allocates nothing after the first call and can be captured into a CUDA graph.
"""

from __future__ import annotations

from collections import OrderedDict

import numpy as np

from .. import functional as qf
from ..runtime.tensor import QuarkTensor


class Parameter:
    """A tensor that appears in ``state_dict()`` (``src/quark/nn/module.py:129-142``)."""

    __slots__ = ("data",)

    def __init__(self, data):
        self.data = data


class Module:
    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def _members(self):
        for k, v in self.__dict__.items():
            if isinstance(v, (Parameter, Module)):
                yield k, v

    def named_parameters(self, prefix: str = ""):
        for name, v in self._members():
            full = f"{prefix}.{name}" if prefix else name
            if isinstance(v, Parameter):
                yield full, v
            else:
                yield from v.named_parameters(full)

    def named_modules(self, prefix: str = ""):
        yield prefix, self
        for name, v in self._members():
            if isinstance(v, Module):
                yield from v.named_modules(f"{prefix}.{name}" if prefix else name)

    def state_dict(self):
        return OrderedDict((k, p.data) for k, p in self.named_parameters())

    def load_state_dict(self, sd: dict, strict: bool = True):
        """Copy host arrays (carrier dtypes) or tensors into the parameters by name."""
        own = dict(self.named_parameters())
        missing = [k for k in own if k not in sd]
        unexpected = [k for k in sd if k not in own]
        if strict and (missing or unexpected):
            raise KeyError(f"load_state_dict: missing {missing[:5]}, unexpected {unexpected[:5]}")
        for k, p in own.items():
            if k not in sd:
                continue
            v = sd[k]
            if isinstance(v, QuarkTensor):
                p.data = v
            else:
                v = np.asarray(v)
                if v.size != p.data.numel:
                    raise ValueError(f"load_state_dict: {k} has {v.size} elements, expected {p.data.numel}")
                p.data = QuarkTensor.from_numpy(v.reshape(p.data.shape), dtype=p.data.dtype)

    def prepare(self, **kwargs):
        for _, v in self._members():
            if isinstance(v, Module):
                v.prepare(**kwargs)


class ModuleList(Module):
    def __init__(self, modules=()):
        self._list = list(modules)

    def _members(self):
        for i, m in enumerate(self._list):
            yield str(i), m

    def __iter__(self):
        return iter(self._list)

    def __len__(self):
        return len(self._list)

    def __getitem__(self, i):
        return self._list[i]


def _cached(module, key: str, shape, dtype) -> QuarkTensor:
    """Per-module output buffers keyed by (name, shape, dtype) (``src/quark/nn/layers.py:236-258``)."""
    cache = module.__dict__.setdefault("_bufs", {})
    k = (key, tuple(shape), dtype)
    buf = cache.get(k)
    if buf is None:
        buf = QuarkTensor.empty(*shape, dtype=dtype)
        cache[k] = buf
    return buf


class Linear(Module):
    """``y = x @ weight.T`` through ``qf.gemm`` (``src/quark/nn/layers.py:261-467``).

    ``prepare(fp8=True)`` narrows the bf16 weight to unscaled e4m3 with ``qf.quantize_e4m3`` like
    the reference (``layers.py:291-304``).  Unlike the reference there is no per-call memset of
    the output: split-K partials live in the workspace, not in the output buffer.
    """

    def __init__(self, in_features: int, out_features: int, *, bias: bool = False, out_dtype: str = "bf16", fp8_skip: bool = False):
        self.weight = Parameter(QuarkTensor.zeros(out_features, in_features, dtype="bf16"))
        self._has_bias = bias
        self._out_dtype = out_dtype
        self._fp8_skip = fp8_skip
        self._fp8 = False
        self.w_scale = None  # f32 [out_features] after prepare(fp8=True, fp8_scaled=True)
        if bias:
            self.bias = Parameter(QuarkTensor.zeros(out_features, dtype="bf16"))

    def prepare(self, *, shuffle: bool = False, fp8: bool = False, fp8_scaled: bool = False, **kwargs):
        """``fp8_scaled`` (extension): narrow with one scale per output channel (``amax / 448``) instead of unscaled;
        the scales stay with the layer and are applied in the GEMM's epilogue."""
        if shuffle:
            raise RuntimeError("weight shuffling is not supported (it is disabled upstream as well)")
        if fp8 and not self._fp8_skip and not self._fp8:
            if fp8_scaled:
                self.weight.data, self.w_scale = qf.quantize_e4m3_rows(self.weight.data)
            else:
                self.weight.data = qf.quantize_e4m3(self.weight.data)
            self._fp8 = True

    def forward(self, x, *, activation=None, bias=None, gate=None, residual=None, gate_groups: int = 1, out_dtype=None, out=None, tp_arena=None):
        """``tp_arena``: a row-parallel linear of a tensor-parallel rank; the partial output is stored straight into the
        staging areas of the ranks that sum it (``qf.gemm_tp``) and nothing is returned."""
        a_dt = x.dtype
        if tp_arena is not None:
            if activation is not None or bias is not None or gate is not None or self._has_bias or self.w_scale is not None:
                raise ValueError("Linear: a partial output sent to its reducers takes no epilogue")
            b_dt = self.weight.data.dtype
            return qf.gemm_tp(x, self.weight.data, tp_arena, compute_dtype=b_dt if b_dt == "e4m3" else None, b_constant=True)
        if a_dt not in ("bf16", "e4m3"):
            raise TypeError(f"Linear: activation dtype {a_dt!r} not in ('bf16', 'e4m3'). Insert a cast upstream.")
        fused_gate = gate is not None and residual is not None
        if fused_gate and bias is not None:
            raise ValueError("Linear.forward: gate/residual fusion is incompatible with bias")
        if self._has_bias and bias is not None:
            raise ValueError("Linear: call-time bias= conflicts with a layer constructed with bias=True")
        b_dt = self.weight.data.dtype
        if a_dt == "e4m3" and b_dt != "e4m3":
            raise TypeError("Linear: an e4m3 activation needs an e4m3 weight (call prepare(fp8=True))")
        od = out_dtype or self._out_dtype
        M = x.numel // int(x.shape[-1])
        N = int(self.weight.data.shape[0])
        if out is None:
            out = _cached(self, "out", (M, N), od)
        return qf.gemm(
            x, self.weight.data, out_dtype=od, compute_dtype=b_dt if b_dt == "e4m3" else None, activation=activation,
            bias=self.bias.data if self._has_bias else bias, gate=gate, residual=residual, gate_groups=gate_groups, out=out,
            w_scale=self.w_scale,
            b_constant=True,  # a Parameter: written by load_params only, never by a kernel of the forward pass
        )  # fmt: skip


class MoE(Module):
    """Top-k mixture of expert MLPs, ``routing="correct"`` of the reference (``src/quark/nn/moe.py:103-363``): every
    token goes to its own ``top_k`` experts with a softmax over their logits as weights,
    ``out = sum_k w_k * W_out[e_k] silu(W_in[e_k] x)``.

    Same parameters and layouts as upstream (``router.weight [E, D]``, ``expert_in [E * H, D]``, ``expert_out
    [E * D, H]``), same rounding points (bf16 logits, bf16 hidden activations, f32 partial outputs, one narrowing after
    the weighted sum), and the reference's schedule: the router emits slot tables sorted by expert (every expert's run
    padded to whole 128-row tiles), the tokens are gathered into slot order, the two expert projections are grouped
    GEMMs over ``M * top_k`` (+ padding) rows, and a reduction gathers each token's ``top_k`` partial rows.
    ``schedule="dense"`` keeps the earlier form (every expert over every token, routing weights zero outside a token's
    top k: E / top_k times the flops, no data-dependent tables).  The capacity-bounded ``"balanced"`` and
    ``"shared_experts"`` routings are rejected, as upstream's own ``forward`` does (``src/quark/nn/moe.py:340-347``)."""

    def __init__(self, M: int, d_model: int, d_intermediate: int, n_experts: int, top_k: int, *, routing: str = "correct", out_dtype: str = "bf16",
                 schedule: str = "sorted"):  # fmt: skip
        if routing != "correct":
            raise NotImplementedError(f"MoE: routing {routing!r} is not implemented (only 'correct')")
        if schedule not in ("sorted", "dense"):
            raise ValueError(f"MoE: schedule {schedule!r} (sorted or dense)")
        if not (1 <= top_k <= n_experts <= 32) or n_experts % 8:
            raise ValueError(f"MoE: top_k {top_k} of {n_experts} experts (8, 16, 24 or 32: the router is a GEMM with one column per expert)")
        self._M, self._D, self._H, self._E, self._K = M, d_model, d_intermediate, n_experts, top_k
        self._schedule = schedule
        self.router = Linear(d_model, n_experts, out_dtype="bf16", fp8_skip=True)  # stays bf16: few columns, precision matters
        self.expert_in = Parameter(QuarkTensor.zeros(n_experts * d_intermediate, d_model, dtype="bf16"))
        self.expert_out = Parameter(QuarkTensor.zeros(n_experts * d_model, d_intermediate, dtype="bf16"))
        self._fp8 = False

    def prepare(self, *, fp8: bool = False, moe_fp8: bool | None = None, **kwargs):
        use = fp8 if moe_fp8 is None else moe_fp8
        if use and not self._fp8:
            self.expert_in.data = qf.quantize_e4m3(self.expert_in.data)
            self.expert_out.data = qf.quantize_e4m3(self.expert_out.data)
            self._fp8 = True

    def forward(self, x):
        M, D, H, E = x.numel // int(x.shape[-1]), self._D, self._H, self._E
        cd = "e4m3" if self._fp8 else None
        logits = self.router(x)
        xq = qf.quantize_e4m3(x, out=_cached(self, "xq", (M, D), "e4m3")) if self._fp8 else x  # once, not per expert
        if self._schedule == "sorted":
            n = qf.moe_slots(M, E, self._K)
            slot_token, slot_weight, tile_expert, token_slot = qf.moe_route_slots(
                logits, top_k=self._K, slot_token=_cached(self, "slot_token", (n,), "s32"), slot_weight=_cached(self, "slot_weight", (n,), "f32"),
                tile_expert=_cached(self, "tile_expert", (n // 128,), "s32"), token_slot=_cached(self, "token_slot", (M, self._K), "s32"),
            )  # fmt: skip
            xs = qf.moe_gather(xq, slot_token, out=_cached(self, "xs", (n, D), xq.dtype))
            if not getattr(self, "_partials_cleared", False):
                # rows of padding tiles are never written nor read; start them from zero once so the buffer holds no junk
                self._partials_cleared = True
                _cached(self, "h_s", (n, H), "bf16").zero_()
                _cached(self, "partials_s", (n, D), "f32").zero_()
            h = qf.gemm_grouped(xs, self.expert_in.data, tile_expert, n_experts=E, compute_dtype=cd, activation="silu",
                                out=_cached(self, "h_s", (n, H), "bf16"), b_constant=True)  # fmt: skip
            partials = qf.gemm_grouped(h, self.expert_out.data, tile_expert, n_experts=E, out_dtype="f32", compute_dtype=cd,
                                       out=_cached(self, "partials_s", (n, D), "f32"), b_constant=True)  # fmt: skip
            return qf.moe_reduce(partials, slot_weight, token_slot, out=_cached(self, "out", (M, D), "bf16"))
        weights = qf.moe_route(logits, top_k=self._K, out=_cached(self, "weights", (E, M), "f32"))
        h = _cached(self, "h", (M, H), "bf16")
        partials = _cached(self, "partials", (E * M, D), "f32")
        for e in range(E):
            qf.gemm(xq, self.expert_in.data.rows(e * H, (e + 1) * H), compute_dtype=cd, activation="silu", out=h, b_constant=True)
            qf.gemm(h, self.expert_out.data.rows(e * D, (e + 1) * D), out_dtype="f32", compute_dtype=cd, out=partials.rows(e * M, (e + 1) * M),
                    b_constant=True)  # fmt: skip
        return qf.moe_combine(partials, weights, out=_cached(self, "out", (M, D), "bf16"))


class SiLU(Module):
    def forward(self, x, *, emit_e4m3: bool = False):
        out = _cached(self, "out", x.shape, x.dtype)
        out_q = _cached(self, "out_q", x.shape, "e4m3") if emit_e4m3 else None
        qf.silu(x, out=out, out_q=out_q)
        return out_q if emit_e4m3 else out


class MLP(Module):
    """``fc2(silu(fc1(x)))`` with the optional gate/residual epilogue on fc2 (``layers.py:700-757``).

    ``fuse_silu=True`` folds SiLU into fc1's epilogue (the reference does so on its PTX and Metal
    GEMMs, ``src/quark/kernels/gemm/spec.py:54-59``); otherwise SiLU is its own launch as on the
    reference's cuBLAS route.  With an fp8 fc2 the hidden activation is handed over in e4m3.
    """

    def __init__(self, d_in: int, d_mid: int, d_out: int, out_dtype: str = "bf16", *, hidden_out_dtype: str | None = None, fuse_silu: bool = False):
        self.fc1 = Linear(d_in, d_mid, out_dtype=hidden_out_dtype or out_dtype)
        self.fc2 = Linear(d_mid, d_out, out_dtype=out_dtype)
        self.silu = SiLU()
        self._fuse_silu = fuse_silu

    def forward(self, x, *, gate=None, residual=None, gate_groups: int = 1, out=None, tp_arena=None):
        fp8 = self.fc2.weight.data.dtype == "e4m3"
        if self._fuse_silu:
            h = self.fc1(x, activation="silu", out_dtype="e4m3" if fp8 else None)
        else:
            h = self.silu(self.fc1(x), emit_e4m3=fp8)
        if tp_arena is not None:
            return self.fc2(h, tp_arena=tp_arena)
        return self.fc2(h, gate=gate, residual=residual, gate_groups=gate_groups, out=out)


class AdaRMSNorm(Module):
    """Stateless ``rmsnorm(x) * (1 + scale) + bias`` (``layers.py:609-619``)."""

    def forward(self, x, scale, bias, *, activation=None, emit_e4m3: bool = False):
        if emit_e4m3:  # the bf16 copy has no reader: only the e4m3 result is written
            return qf.ada_rmsnorm(x, scale, bias, activation=activation, out_q=_cached(self, "out_q", x.shape, "e4m3"), only_q=True)
        return qf.ada_rmsnorm(x, scale, bias, activation=activation, out=_cached(self, "out", x.shape, x.dtype))


class RMSNorm(Module):
    """Plain RMSNorm, no gain; caches its output (``layers.py:645-652``)."""

    def forward(self, x):
        return qf.rmsnorm(x, out=_cached(self, "out", x.shape, x.dtype))


class Add(Module):
    """``x + y`` into a cached buffer (``layers.py:655-669``)."""

    def forward(self, x, y):
        return qf.add(x, y, out=_cached(self, "out", x.shape, x.dtype))


class MLPFusion(Module):
    """``y = fc2(silu(x @ Wx.T + cond @ Wc.T))``: the cond projection enters fc1_x as its bias row
    (``layers.py:797-822``).  bf16 throughout, also when the model's other linears are e4m3."""

    def __init__(self, d_model: int, out_dtype: str = "bf16"):
        self.fc1_x = Linear(d_model, d_model, out_dtype=out_dtype)
        self.fc1_c = Linear(d_model, d_model, out_dtype=out_dtype)
        self.fc2 = Linear(d_model, d_model, out_dtype=out_dtype)

    def forward(self, x, cond):
        h_c = self.fc1_c(cond).reshape(-1)
        return self.fc2(self.fc1_x(x, bias=h_c, activation="silu"))


class ControllerInputEmbedding(Module):
    """``[mouse(2) | buttons one-hot | scroll]`` padded to a multiple of 16 -> fc1 -> SiLU -> fc2 -> ``[1, d_model]``
    (``layers.py:760-794``).  bf16 throughout."""

    def __init__(self, n_buttons: int, d_model: int, mlp_ratio: int = 4, out_dtype: str = "bf16"):
        self._raw_in = n_buttons + 3
        self._padded_in = (self._raw_in + 15) // 16 * 16
        self.fc1 = Linear(self._padded_in, d_model * mlp_ratio, out_dtype=out_dtype)
        self.fc2 = Linear(d_model * mlp_ratio, d_model, out_dtype=out_dtype)

    def forward(self, ctrl_input):
        return self.fc2(self.fc1(ctrl_input, activation="silu"))


class AdaGateResidual(Module):
    def forward(self, x, y, gate):
        return qf.ada_gate_residual(x, y, gate, out=_cached(self, "out", x.shape, x.dtype))


class HeadRMSNorm(Module):
    def __init__(self, n_q_heads: int, n_kv_heads: int, Dh: int):
        self._nq, self._Hk, self._Dh = n_q_heads, n_kv_heads, Dh

    def forward(self, qkv):
        return qf.head_rmsnorm(qkv, n_q_heads=self._nq, n_kv_heads=self._Hk, Dh=self._Dh, out=_cached(self, "out", qkv.shape, qkv.dtype))


class ValueResidualPacked(Module):
    """``v += lamb * (v_first - v)`` with a learnable f32 scalar (``layers.py:825-843``)."""

    def __init__(self, v_col_offset: int, v_width: int, lamb: float = 0.5):
        self._vo, self._vw = v_col_offset, v_width
        self.lamb = Parameter(QuarkTensor.from_numpy(np.array([lamb], dtype=np.float32)))

    def forward(self, qkv, qkv_first):
        return qf.value_residual_packed(
            qkv, qkv_first, self.lamb.data, v_col_offset=self._vo, v_width=self._vw, out=_cached(self, "out", qkv.shape, qkv.dtype)
        )


class EulerStep(Module):
    def forward(self, x, v, dsig):
        return qf.euler_step(x, v, dsig, out=_cached(self, "out", x.shape, x.dtype))


class Patchify(Module):
    def __init__(self, C: int, d_model: int, H: int, W: int, ph: int = 2, pw: int = 2):
        self.weight = Parameter(QuarkTensor.zeros(d_model, C * ph * pw, dtype="bf16"))
        self._C, self._H, self._W, self._ph, self._pw = C, H, W, ph, pw

    def forward(self, x):
        d_model = int(self.weight.data.shape[0])
        rows = (self._H // self._ph) * (self._W // self._pw)
        out = _cached(self, "out", (rows, d_model), "bf16")
        return qf.patchify(x, self.weight.data, B=1, C=self._C, H=self._H, W_spatial=self._W, ph=self._ph, pw=self._pw, out=out)


class Unpatchify(Module):
    def __init__(self, d_model: int, C: int, H: int, W: int, ph: int = 2, pw: int = 2):
        self.weight = Parameter(QuarkTensor.zeros(C * ph * pw, d_model, dtype="bf16"))
        self.bias = Parameter(QuarkTensor.zeros(C * ph * pw, dtype="bf16"))
        self._C, self._H, self._W, self._ph, self._pw = C, H, W, ph, pw

    def forward(self, x, B: int = 1):
        out = _cached(self, "out", (B, self._C * self._H * self._W), "bf16")
        return qf.unpatchify(x, self.weight.data, self.bias.data, B=B, C=self._C, H=self._H, W=self._W, ph=self._ph, pw=self._pw, out=out)


class KVCacheUpdate(Module):
    """Per-layer cache state and its append (``src/quark/nn/layers.py:846-970``)."""

    def __init__(self, *, B: int, n_kv_heads: int, n_q_heads: int, H_spatial: int, W_spatial: int, Dh: int, num_buckets: int,
                 pinned_dilation: int, packed_qkv: bool, rope_n_frames: int = 1, dtype: str = "bf16", quilt_factor: int = 1,
                 quilt_offset: int = 0):  # fmt: skip
        tpf = H_spatial * W_spatial
        if tpf % quilt_factor != 0:
            raise ValueError(f"KVCacheUpdate: tpf={tpf} not divisible by quilt_factor={quilt_factor}")
        tpf //= quilt_factor  # tokens of a frame that the cache keeps (src/quark/kernels/kv_cache_update/spec.py:66-76)
        L = num_buckets * tpf
        cap = L + tpf
        self.K_cache = QuarkTensor.zeros(B * n_kv_heads * cap, Dh, dtype=dtype)
        self.Vt_cache = QuarkTensor.zeros(B * n_kv_heads * Dh, cap, dtype=dtype)
        self.segments = QuarkTensor.from_numpy(np.array([0, 0, L, tpf, 0, 0], dtype=np.int32))
        self.n_segments = QuarkTensor.from_numpy(np.array([2], dtype=np.int32))
        self.frame_t = QuarkTensor.zeros(1, dtype="s32")
        # frozen = 1 and frozen = 0 as two constant device scalars: no per-call memset in the graph
        self._frozen = (QuarkTensor.from_numpy(np.array([0], dtype=np.int32)), QuarkTensor.from_numpy(np.array([1], dtype=np.int32)))
        self._L, self._tpf = L, tpf
        # optional per-head quantisation scales (f32 [n_kv_heads]); None = the reference's scale-free caches
        self.k_scale = self.v_scale = None
        self._kw = dict(B=B, n_kv_heads=n_kv_heads, H_spatial=H_spatial, W_spatial=W_spatial, num_buckets=num_buckets,
                        pinned_dilation=pinned_dilation, packed_qkv=packed_qkv, n_q_heads=n_q_heads, quilt_factor=quilt_factor,
                        quilt_offset=quilt_offset)  # fmt: skip

    def forward(self, qkv, frame_t=None, frozen: bool = False):
        ft = frame_t if frame_t is not None else self.frame_t
        qf.kv_cache_update(qkv, qkv, ft, self._frozen[1 if frozen else 0], self.Vt_cache, self.segments, self.n_segments, self.K_cache,
                           k_scale=self.k_scale, v_scale=self.v_scale, **self._kw)  # fmt: skip

    # ---- a second pair of caches in the attention's compute dtype, when that differs from the cache dtype
    def shadow(self, dtype: str, frame_t=None, frozen: bool = False):
        """``(K, Vt)`` equal to ``cast(K_cache), cast(Vt_cache)`` in ``dtype``, to be called after the append of the step:
        the rows that append wrote are converted (``qf.kv_cast_appended``); if the caches were written from the host since
        the last call (loaded, restored, reset) or this is the first call, everything is.  The reference casts as the
        attention loads (``src/quark/kernels/owl_attn/kernel.py:342-348``): same values."""
        if dtype == self.K_cache.dtype:
            return self.K_cache, self.Vt_cache
        if getattr(self, "_shadow", None) is None or self._shadow[0].dtype != dtype:
            self._shadow = (QuarkTensor.empty(*self.K_cache.shape, dtype=dtype), QuarkTensor.empty(*self.Vt_cache.shape, dtype=dtype))
            self._shadow_seen = None
        seen = (self.K_cache._storage.host_writes, self.Vt_cache._storage.host_writes)
        if self._shadow_seen != seen:
            self.refresh_shadow()
        else:
            qf.kv_cast_appended(self.K_cache, self.Vt_cache, self._shadow[0], self._shadow[1], frame_t if frame_t is not None else self.frame_t,
                                self._frozen[1 if frozen else 0], **self._kw)  # fmt: skip
        return self._shadow

    def refresh_shadow(self) -> None:
        """Converts both caches whole (after the caches were written by anything but the append)."""
        if getattr(self, "_shadow", None) is None:
            return
        conv = qf.quantize_e4m3 if self._shadow[0].dtype == "e4m3" else qf.dequantize_e4m3
        conv(self.K_cache, out=self._shadow[0])
        conv(self.Vt_cache, out=self._shadow[1])
        self._shadow_seen = (self.K_cache._storage.host_writes, self.Vt_cache._storage.host_writes)

    def set_scales(self, k_scale, v_scale) -> None:
        """Per-KV-head scales as host arrays (or None): the caches then hold ``K / k_scale[h]`` and ``V / v_scale[h]``."""
        up = lambda a: None if a is None else QuarkTensor.from_numpy(np.ascontiguousarray(a, dtype=np.float32))  # noqa: E731
        self.k_scale, self.v_scale = up(k_scale), up(v_scale)

    def set_frame_t(self, value: int) -> None:
        self.frame_t.copy_from_numpy(np.array([value], dtype=np.int32))

    def reset(self) -> None:
        self.K_cache.zero_()
        self.Vt_cache.zero_()
        self.segments.copy_from_numpy(np.array([0, 0, self._L, self._tpf, 0, 0], dtype=np.int32))
        self.n_segments.copy_from_numpy(np.array([2], dtype=np.int32))
        self.set_frame_t(0)
        self.refresh_shadow()


class OwlAttn(Module):
    """Carries the per-layer attention keywords (``src/quark/nn/layers.py:973-1038``)."""

    def __init__(self, *, B: int, n_kv_heads: int, gqa_ratio: int, H_spatial: int, W_spatial: int, num_buckets: int,
                 pinned_dilation: int, packed_qkv: bool, rope_n_frames: int = 1, compute_dtype: str | None = "e4m3",
                 quilt_factor: int = 1, quilt_offset: int = 0):  # fmt: skip
        self._kw = dict(B=B, n_kv_heads=n_kv_heads, gqa_ratio=gqa_ratio, H_spatial=H_spatial, W_spatial=W_spatial,
                        num_buckets=num_buckets, pinned_dilation=pinned_dilation, packed_qkv=packed_qkv,
                        quilt_factor=quilt_factor, quilt_offset=quilt_offset)  # fmt: skip
        self._compute_dtype = compute_dtype

    def forward(self, qkv, kv_cache: KVCacheUpdate, frame_t=None, *, emit_e4m3: bool = False, frozen: bool = False):
        """``frozen``: what the append of this step was called with (it decides which rows a shadow cache has to take over)."""
        n_kv, gqa = self._kw["n_kv_heads"], self._kw["gqa_ratio"]
        n_q = n_kv * gqa
        Dh = int(qkv.shape[1]) // (n_q + 2 * n_kv)
        out = _cached(self, "out", (int(qkv.shape[0]), n_q * Dh), qkv.dtype)
        out_q = _cached(self, "out_q", out.shape, "e4m3") if emit_e4m3 else None
        cd = self._compute_dtype or "bf16"  # as qf.owl_attn reads it
        K, Vt = kv_cache.shadow(cd, frame_t, frozen)  # the caches themselves unless the attention computes in another dtype
        qf.owl_attn(qkv, K, Vt, kv_cache.segments, kv_cache.n_segments, frame_t=frame_t,
                    out=out, out_q=out_q, compute_dtype=self._compute_dtype, k_scale=kv_cache.k_scale, v_scale=kv_cache.v_scale, **self._kw)  # fmt: skip
        return out_q if emit_e4m3 else out
