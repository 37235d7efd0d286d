"""The scaled-e4m3 mode: per-output-channel weight scales, per-KV-head cache scales.

The reference's e4m3 is scale free everywhere (``src/quark/runtime/cublas.py:151-158``: one device ``1.0`` serves as the A
and B scale; ``src/quark/nn/layers.py:291-304``: weights are narrowed without a scale), so this mode has no reference
oracle of its own.  Its oracle is the restated formula, in ``oracle/ops.py``:

    C = (Aq . Wq^T) * (a_scale * w_scale[n])      Kq = e4m3(RoPE(K) * (1 / k_scale[h]))      Vq = e4m3(V * (1 / v_scale[h]))
    S = (Q . Kq^T) * k_scale[h] / 8               O = (P . Vq) * v_scale[h]

Held to the same bars as the scale-free path: e4m3 bytes exact given equal scales (V and weights exact; K up to the
one-code flips of the temporal sine / cosine), cosine >= 0.999 per output tensor; NULL scales and scales of exactly 1
give the scale-free bytes.
"""

import copy

import numpy as np
import pytest

from oracle import codec
from oracle import model as omodel
from oracle import ops
from tests import util
from tests.test_gpu_model import compare, small_cfg
from tests.util import bf16_randn, e4m3_randn, f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def qb():
    import quark_b200 as q

    q._lib.require_device(0)
    yield q
    q.runtime.synchronize()
    assert q._lib.device_status() == 0


def T(qb, arr, dtype=None):
    return qb.QuarkTensor.from_numpy(np.asarray(arr), dtype=dtype)


def scaled_oracle_params(params):
    """The oracle's view of a scaled-fp8 model: weights narrowed per output channel, the scales kept beside them."""
    p = copy.copy(params)
    p["blocks"] = []
    for b in params["blocks"]:
        nb = dict(b)
        for k in ("qkv.weight", "out.weight", "fc1.weight", "fc2.weight"):
            nb[k], nb[k + ".scale"] = ops.quantize_e4m3_rows(b[k])
        p["blocks"].append(nb)
    return p


def test_row_scaled_narrowing_is_bit_exact(qb):
    r = util.rng(70)
    x = (r.standard_normal((96, 512)) * np.exp2(r.integers(-12, 6, size=(96, 1)))).astype(np.float32)
    x[5] = 0.0  # an all-zero row keeps scale 1
    x[6, 3] = 3.0e4  # one outlier sets the row's scale
    xb = codec.f32_to_bf16_rne(x)
    q, s = qb.qf.quantize_e4m3_rows(T(qb, xb, "bf16"))
    wq, ws = ops.quantize_e4m3_rows(xb)
    np.testing.assert_array_equal(s.to_numpy(), ws)
    np.testing.assert_array_equal(q.to_numpy(), wq)
    assert ws[5] == 1.0 and not wq[5].any()
    assert np.all(np.max(np.abs(codec.e4m3_to_f32(wq[ws != 1.0])), axis=1) == 448.0)  # every row uses the top code


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
def test_cache_append_with_per_head_scales(qb, kv_dt):
    """All three append paths (stand-alone kernel, fused post-processing, GEMM epilogue) write the same bytes, and
    those are the oracle's: V exact, K up to rare one-code flips; scales of exactly 1 give the scale-free bytes."""
    r = util.rng(71)
    H, W, Hq, Hk, nb, pd, ft, frozen = 16, 8, 8, 4, 4, 1, 6, 0
    tpf, cap, D, Kd = H * W, (nb + 1) * H * W, (Hq + 2 * Hk) * 64, 256
    ks = np.array([0.02, 0.5, 1.75, 0.011], np.float32)
    vs = np.array([2.0, 0.0625, 0.4, 0.013], np.float32)
    qf = qb.qf
    x = bf16_randn(r, (tpf, Kd))
    A = T(qb, codec.f32_to_e4m3(f32(x, "bf16")), "e4m3")
    Wb = bf16_randn(r, (D, Kd), 0.1)
    Wq, wsc = qf.quantize_e4m3_rows(T(qb, Wb, "bf16"))
    first = T(qb, bf16_randn(r, (tpf, D)), "bf16")
    lam = T(qb, np.array([0.37], np.float32))
    ftt, frz = T(qb, np.array([ft], np.int32)), T(qb, np.array([frozen], np.int32))
    carrier = np.uint16 if kv_dt == "bf16" else np.uint8

    def state():
        return (T(qb, np.zeros((Hk * cap, 64), carrier), kv_dt), T(qb, np.zeros((Hk * 64, cap), carrier), kv_dt),
                T(qb, np.full(6, -7, np.int32)), T(qb, np.array([-7], np.int32)))  # fmt: skip

    kw = dict(n_q_heads=Hq, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd)
    sc = dict(k_scale=T(qb, ks), v_scale=T(qb, vs))
    # (a) projection (scaled weights), the three reference ops, the stand-alone append
    raw = qf.gemm(A, Wq, out_dtype="bf16", compute_dtype="e4m3", tile_n=128, w_scale=wsc)
    q0 = qf.value_residual_packed(qf.head_rmsnorm(raw, Hq, Hk, 64), first, lam, v_col_offset=(Hq + Hk) * 64, v_width=Hk * 64)
    Ka, Va, sa, na = state()
    qf.kv_cache_update(q0, None, ftt, frz, Va, sa, na, Ka, B=1, packed_qkv=True, **kw, **sc)
    # (b) the fused post-processing kernel, (c) the GEMM with that as its epilogue
    Kb, Vb, sb, nb_ = state()
    q1 = qf.qkv_post(raw, first, lam, ftt, frz, Vb, sb, nb_, Kb, **kw, **sc)
    Kc, Vc, s_c, nc = state()
    q2 = qf.gemm_qkv_post(A, Wq, first, lam, ftt, frz, Vc, s_c, nc, Kc, w_scale=wsc, **kw, **sc)
    for q in (q1, q2):
        np.testing.assert_array_equal(q.to_numpy(), q0.to_numpy())
    for K, V in ((Kb, Vb), (Kc, Vc)):
        np.testing.assert_array_equal(K.to_numpy(), Ka.to_numpy())
        np.testing.assert_array_equal(V.to_numpy(), Va.to_numpy())
    # against the restated formula, fed the device's own packed QKV
    with codec.bf16_rounding("rne"):
        wK, wV, _, _ = ops.kv_cache_update(q0.to_numpy(), ft, frozen, n_kv_heads=Hk, n_q_heads=Hq, H_spatial=H, W_spatial=W, num_buckets=nb,
                                           pinned_dilation=pd, kv_dtype=kv_dt, k_scale=ks, v_scale=vs)  # fmt: skip
    gK, gV = Ka.to_numpy(), Va.to_numpy()
    np.testing.assert_array_equal(gV, wV)
    diff = gK != wK
    if kv_dt == "e4m3":
        assert diff.mean() <= 2e-3 and np.all(np.abs(gK.astype(np.int16)[diff] - wK.astype(np.int16)[diff]) <= 1)
    else:
        assert np.max(util.bf16_ulp_diff(gK, wK)[np.abs(f32(wK, "bf16")) > 1e-3]) <= 2
    # the scaled projection against the oracle's GEMM with the same scales
    wraw = ops.gemm(x, Wq.to_numpy(), b_dtype="e4m3", a_quant="e4m3", w_scale=wsc.to_numpy(), return_f32=True)
    g = f32(raw.to_numpy(), "bf16")
    assert util.cosine(g, wraw) >= util.COS_MIN and util.max_rel(g, wraw) <= util.BF16_MAX_REL
    # scales of exactly one: the scale-free bytes
    one = dict(k_scale=T(qb, np.ones(Hk, np.float32)), v_scale=T(qb, np.ones(Hk, np.float32)))
    Kd1, Vd1, s1, n1 = state()
    qf.gemm_qkv_post(A, Wq, first, lam, ftt, frz, Vd1, s1, n1, Kd1, w_scale=wsc, **kw, **one)
    Kd0, Vd0, s0, n0 = state()
    qf.gemm_qkv_post(A, Wq, first, lam, ftt, frz, Vd0, s0, n0, Kd0, w_scale=wsc, **kw)
    np.testing.assert_array_equal(Kd1.to_numpy(), Kd0.to_numpy())
    np.testing.assert_array_equal(Vd1.to_numpy(), Vd0.to_numpy())
    assert np.any(Kd0.to_numpy() != Ka.to_numpy())  # and the scales above did change what is stored


@pytest.mark.parametrize("use_graph", [False, True])
def test_scaled_fp8_session_matches_the_restated_oracle(qb, use_graph):
    """A session with every linear and both caches scaled: appended and generated frames against the chained
    oracle of the restated formulas, cache bytes of the first layer after the first append against the oracle's."""
    from quark_b200.models import Waypoint15Config, make_params

    base = small_cfg(qb, "fp8")
    cfg = Waypoint15Config(**{**base.__dict__, "fp8_scales": True})
    params = make_params(cfg, seed=17, weight_std=0.08)
    assert params["blocks"][0]["k_scale"].shape == (cfg.n_kv_heads,)
    eng = qb.Engine(cfg=cfg, quant=cfg.quant, params=params, use_graph=use_graph)
    assert eng.model.blocks[0].qkv_proj.w_scale is not None and eng.model.blocks[0].kv_cache.k_scale is not None
    op = scaled_oracle_params(params)
    for li, blk in enumerate(eng.model.blocks):  # the device narrowing of every weight is the oracle's, bit for bit
        for name, lin in (("qkv.weight", blk.qkv_proj), ("out.weight", blk.out_proj), ("fc1.weight", blk.mlp.fc1), ("fc2.weight", blk.mlp.fc2)):
            np.testing.assert_array_equal(lin.weight.data.to_numpy(), op["blocks"][li][name])
            np.testing.assert_array_equal(lin.w_scale.to_numpy(), op["blocks"][li][name + ".scale"])
    oq = omodel.Quant(linear="fp8", kv_cache="fp8", attn_compute="fp8")
    r = util.rng(72)
    lats = [codec.f32_to_bf16(r.standard_normal((1, cfg.latent_numel)).astype(np.float32)) for _ in range(3)]
    noises = [r.standard_normal((1, cfg.latent_numel)).astype(np.float32) for _ in range(2)]
    with codec.bf16_rounding("rne"):
        state, ft, want = omodel.new_state(cfg, oq), 0, []
        for lat in lats:
            omodel.nfe_forward(cfg, op, state, lat, len(cfg.scheduler_sigmas) - 1, ft, frozen=False, quant=oq)
            if ft == 0:
                first_K = state[0]["K_cache"].copy()
            ft += 1
        for nz in noises:
            w, ft = omodel.gen_frame(cfg, op, state, codec.f32_to_bf16(nz), ft, quant=oq)
            want.append(w)
    eng.append_frame(lats[0])
    gK = eng.model.blocks[0].kv_cache.K_cache.to_numpy()
    np.testing.assert_array_equal(gK.any(axis=1), first_K.any(axis=1))
    assert util.cosine(f32(gK, "e4m3"), f32(first_K, "e4m3")) >= util.COS_MIN
    for lat in lats[1:]:
        eng.append_frame(lat)
    for k, nz in enumerate(noises):
        compare(eng.gen_frame(noise=nz).reshape(-1), want[k].reshape(-1), f"scaled fp8 gen_frame {k} graph={use_graph}", True)
    # the scales matter: the scale-free session of the same parameters is a different (equally valid) computation
    plain = qb.Engine(cfg=base, quant=base.quant, params=params, use_graph=False)
    plain.append_frame(lats[0])
    assert np.any(plain.model.blocks[0].kv_cache.K_cache.to_numpy() != gK)
