"""GPU parity of every kernel against the CPU oracle, through the qf.* layer and the C ABI.

Inputs are seeded; small shapes come from the golden fixtures (so the CUDA result is also tied
to what the reference's own numpy oracles produced), large shapes are the BASELINE shapes
(360p: 128 tokens, 720p: 512 tokens; d_model 2048, 32 Q / 16 KV heads of 64).
"""

from pathlib import Path

import numpy as np
import pytest

from oracle import codec, ops
from tests import util
from tests.util import assert_close_bf16, bf16_randn, e4m3_randn, f32

pytestmark = pytest.mark.gpu
G = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def qb():
    import quark_b200 as q

    q._lib.require_device(0)
    yield q
    q.runtime.synchronize()
    assert q._lib.device_status() == 0, "a kernel reported a timed-out wait or a bad segment table"


def T(qb, arr, dtype=None):
    return qb.QuarkTensor.from_numpy(np.asarray(arr), dtype=dtype)


# --------------------------------------------------------------------------- e4m3 narrowing


def test_quantize_e4m3_every_bf16_value_bit_exact(qb):
    allb = np.arange(65536, dtype=np.uint16)
    got = qb.qf.quantize_e4m3(T(qb, allb, "bf16")).to_numpy()
    want = codec.f32_to_e4m3(codec.bf16_to_f32(allb))
    nan = np.isnan(codec.bf16_to_f32(allb))
    np.testing.assert_array_equal(got[~nan], want[~nan])
    assert np.all((got[nan] & 0x7F) == 0x7F)
    # the reference's own encoder differs only in its documented subnormal band
    ref = np.load(G / "codec.npz")["e4m3_of_all_bf16"]
    assert int(np.count_nonzero(got[~nan] != ref[~nan])) == 32


def test_quantize_e4m3_from_f32_and_ragged_tail(qb):
    r = util.rng(1)
    x = (r.standard_normal(1000 + 13) * 30).astype(np.float32)
    x[:6] = [0.0, -0.0, 448.0, 1e9, -1e9, 0.0146484375]
    got = qb.qf.quantize_e4m3(T(qb, x)).to_numpy()
    np.testing.assert_array_equal(got, codec.f32_to_e4m3(x))


# --------------------------------------------------------------------------- glue ops


@pytest.mark.parametrize("rows,D", [(32, 256), (128, 2048), (512, 2048)])
@pytest.mark.parametrize("act", [None, "silu"])
def test_ada_rmsnorm(qb, rows, D, act):
    r = util.rng(2)
    X, s, b = bf16_randn(r, (rows, D)), bf16_randn(r, (1, D), 0.1), bf16_randn(r, (1, D), 0.1)
    outq = qb.QuarkTensor.empty(rows, D, dtype="e4m3")
    got = qb.qf.ada_rmsnorm(T(qb, X, "bf16"), T(qb, s, "bf16"), T(qb, b, "bf16"), activation=act, out_q=outq).to_numpy()
    want = ops.ada_rmsnorm(X, s, b, activation=act)
    assert_close_bf16(got, want, "ada_rmsnorm")
    assert np.percentile(util.bf16_ulp_diff(got, want), 99.9) <= 1
    # the e4m3 side output is the narrowing of the bf16 output, byte for byte
    np.testing.assert_array_equal(outq.to_numpy(), codec.f32_to_e4m3(codec.bf16_to_f32(got)))


def test_glue_ops_against_golden_inputs(qb):
    z = np.load(G / "glue.npz")
    qf = qb.qf
    X, Y, sc = T(qb, z["X"], "bf16"), T(qb, z["Y"], "bf16"), T(qb, z["scale"], "bf16")
    assert_close_bf16(qf.silu(X).to_numpy().ravel(), z["silu"].ravel(), "silu")
    assert_close_bf16(qf.ada_gate_residual(X, Y, sc).to_numpy(), z["ada_gate_residual"], "ada_gate_residual")
    assert_close_bf16(qf.ada_rmsnorm(X, sc, T(qb, z["bias"], "bf16")).to_numpy(), z["ada_rmsnorm"], "ada_rmsnorm")
    QKV, QKV0 = T(qb, z["QKV"], "bf16"), T(qb, z["QKV0"], "bf16")
    got = qf.head_rmsnorm(QKV, n_q_heads=2, n_kv_heads=1, Dh=64).to_numpy()
    assert_close_bf16(got, z["head_rmsnorm"], "head_rmsnorm")
    np.testing.assert_array_equal(got[:, 192:], z["QKV"][:, 192:])  # V columns are copied
    lam = T(qb, np.array([0.37], dtype=np.float32))
    got = qf.value_residual_packed(QKV, QKV0, lam, v_col_offset=192, v_width=64).to_numpy()
    assert_close_bf16(got, z["value_residual_packed"], "value_residual_packed")
    np.testing.assert_array_equal(got[:, :192], z["QKV"][:, :192])  # Q and K columns are copied
    got = qf.patchify(T(qb, z["lat"], "bf16"), T(qb, z["Wp"], "bf16"), B=1, C=4, H=8, W_spatial=12, ph=2, pw=2).to_numpy()
    assert_close_bf16(got, z["patchify"], "patchify")
    got = qf.unpatchify(T(qb, z["tok"], "bf16"), T(qb, z["Wu"], "bf16"), T(qb, z["bu"], "bf16"), B=1, C=4, H=8, W=12).to_numpy()
    assert_close_bf16(got, z["unpatchify"], "unpatchify")


def test_glue_ops_at_model_size(qb):
    r = util.rng(3)
    qf = qb.qf
    tpf, d = 512, 2048
    X, Y, g = bf16_randn(r, (tpf, d)), bf16_randn(r, (tpf, d)), bf16_randn(r, (1, d))
    assert_close_bf16(qf.ada_gate_residual(T(qb, X, "bf16"), T(qb, Y, "bf16"), T(qb, g, "bf16")).to_numpy(), ops.ada_gate_residual(X, Y, g), "gate")
    H1 = bf16_randn(r, (tpf, 8192), 2.0)
    oq = qb.QuarkTensor.empty(tpf, 8192, dtype="e4m3")
    got = qf.silu(T(qb, H1, "bf16"), out_q=oq).to_numpy()
    assert_close_bf16(got, ops.silu(H1), "silu")
    np.testing.assert_array_equal(oq.to_numpy(), codec.f32_to_e4m3(codec.bf16_to_f32(got)))
    QKV, QKV0 = bf16_randn(r, (tpf, 4096)), bf16_randn(r, (tpf, 4096))
    assert_close_bf16(qf.head_rmsnorm(T(qb, QKV, "bf16"), 32, 16, 64).to_numpy(), ops.head_rmsnorm(QKV, n_q_heads=32, n_kv_heads=16), "head_rmsnorm")
    lam = T(qb, np.array([0.5], dtype=np.float32))
    got = qf.value_residual_packed(T(qb, QKV, "bf16"), T(qb, QKV0, "bf16"), lam, v_col_offset=3072, v_width=1024).to_numpy()
    assert_close_bf16(got, ops.value_residual_packed(QKV, QKV0, 0.5, v_col_offset=3072, v_width=1024), "value_residual")
    lat, v = bf16_randn(r, (1, 32 * 32 * 64)), bf16_randn(r, (1, 32 * 32 * 64))
    ds = T(qb, np.array([-0.15], dtype=np.float32))
    assert_close_bf16(qf.euler_step(T(qb, lat, "bf16"), T(qb, v, "bf16"), ds).to_numpy(), ops.euler_step(lat, v, -0.15), "euler")
    Wp = bf16_randn(r, (d, 128), 0.02)
    got = qf.patchify(T(qb, lat, "bf16"), T(qb, Wp, "bf16"), B=1, C=32, H=32, W_spatial=64, ph=2, pw=2).to_numpy()
    assert_close_bf16(got, ops.patchify(lat, Wp, C=32, H=32, Wd=64), "patchify")
    Wu, bu = bf16_randn(r, (128, d), 0.02), bf16_randn(r, (128,), 0.1)
    got = qf.unpatchify(T(qb, X, "bf16"), T(qb, Wu, "bf16"), T(qb, bu, "bf16"), B=1, C=32, H=32, W=64).to_numpy()
    assert_close_bf16(got, ops.unpatchify(X, Wu, bu, C=32, H=32, Wd=64), "unpatchify")
    c = T(qb, np.array([41], dtype=np.int32))
    qf.increment(c)
    assert c.to_numpy().tolist() == [42]


def test_controller_conditioning_ops_against_golden_and_oracle(qb):
    """Plain RMSNorm, add, MLPFusion and the controller embedding: against the fixtures made from the reference's
    oracles, and at model width against the oracle."""
    from quark_b200 import nn

    z = np.load(G / "ctrl.npz")
    qf = qb.qf
    X, Y, cond = T(qb, z["X"], "bf16"), T(qb, z["Y"], "bf16"), T(qb, z["cond"], "bf16")
    assert_close_bf16(qf.rmsnorm(X).to_numpy(), z["rmsnorm"], "rmsnorm")
    assert np.percentile(util.bf16_ulp_diff(qf.rmsnorm(X).to_numpy(), z["rmsnorm"]), 99.9) <= 1
    assert_close_bf16(qf.rmsnorm(cond).to_numpy(), z["rmsnorm_row"], "rmsnorm row")
    got_add = qf.add(X, Y).to_numpy()
    assert util.bf16_ulp_diff(got_add, z["add"]).max() <= 1  # the reference's oracle truncates to bf16, the kernel rounds to nearest
    with codec.bf16_rounding("rne"):
        np.testing.assert_array_equal(got_add, ops.add(z["X"], z["Y"]))
    fus = nn.MLPFusion(256)
    fus.fc1_x.weight.data, fus.fc1_c.weight.data, fus.fc2.weight.data = T(qb, z["Wx"], "bf16"), T(qb, z["Wc"], "bf16"), T(qb, z["W2"], "bf16")
    assert_close_bf16(fus(X, cond).to_numpy(), z["mlp_fusion"], "MLPFusion")
    emb = nn.ControllerInputEmbedding(29, 64)
    emb.fc1.weight.data, emb.fc2.weight.data = T(qb, z["We1"], "bf16"), T(qb, z["We2"], "bf16")
    assert_close_bf16(emb(T(qb, z["ctrl_input"], "bf16")).to_numpy(), z["ctrl_emb"], "ControllerInputEmbedding")
    # model width: 512 tokens x 2048, ragged tail for add
    r = util.rng(17)
    x = bf16_randn(r, (512, 2048), 3.0)
    assert_close_bf16(qf.rmsnorm(T(qb, x, "bf16")).to_numpy(), ops.rmsnorm(x), "rmsnorm 512 x 2048")
    a, b = bf16_randn(r, (1, 8 * 1000 + 5)), bf16_randn(r, (1, 8 * 1000 + 5))
    with codec.bf16_rounding("rne"):
        np.testing.assert_array_equal(qf.add(T(qb, a, "bf16"), T(qb, b, "bf16")).to_numpy(), ops.add(a, b))


def test_rope_table_device_builder_matches_numpy(qb):
    import ctypes as C

    for H, W in [(16, 8), (8, 16), (32, 16), (8, 8)]:
        want = qb.qf.rope_table_numpy(H, W)
        t = qb.QuarkTensor.empty(H * W, 16, dtype="f32")
        qb._lib.check(qb._lib.load().qb_rope_table_build(C.c_void_p(t.data_ptr()), H, W, C.c_void_p(qb.runtime.active_stream())))
        got = t.to_numpy()
        assert np.max(np.abs(got - want)) <= 2.5e-7, (H, W)
        # and the host table equals the oracle's table column for column
        c, s = ops.rope_tables(H, W, 0)
        np.testing.assert_array_equal(want[:, :8], c[:, 0:16:2])
        np.testing.assert_array_equal(want[:, 8:], s[:, 0:16:2])


# --------------------------------------------------------------------------- KV-cache append


def _kv_run(qb, qkv, ft, frozen, *, Hq, Hk, H, W, nb, pd, kv_dt, prefill=None, quilt=1, qoff=0):
    tpf, cap = H * W, (nb + 1) * (H * W // quilt)
    carrier = np.uint16 if kv_dt == "bf16" else np.uint8
    K0 = np.zeros((Hk * cap, 64), carrier) if prefill is None else np.full((Hk * cap, 64), prefill, carrier)
    V0 = np.zeros((Hk * 64, cap), carrier) if prefill is None else np.full((Hk * 64, cap), prefill, carrier)
    Kc, Vc = T(qb, K0, kv_dt), T(qb, V0, kv_dt)
    segs, nseg = T(qb, np.full(6, -7, np.int32)), T(qb, np.array([-7], np.int32))
    out = qb.qf.kv_cache_update(
        T(qb, qkv, "bf16"), None, T(qb, np.array([ft], np.int32)), T(qb, np.array([frozen], np.int32)), Vc, segs, nseg, Kc,
        B=1, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd, packed_qkv=True, n_q_heads=Hq,
        quilt_factor=quilt, quilt_offset=qoff,
    )  # fmt: skip
    assert out[0] is Kc and out[1] is Vc
    return Kc.to_numpy(), Vc.to_numpy(), segs.to_numpy(), nseg.to_numpy()


def _check_kv(K, Vt, segs, nseg, qkv, ft, frozen, *, Hq, Hk, H, W, nb, pd, kv_dt, quilt=1, qoff=0):
    wK, wV, wsegs, wn = ops.kv_cache_update(
        qkv, ft, frozen, n_kv_heads=Hk, n_q_heads=Hq, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd, kv_dtype=kv_dt,
        quilt_factor=quilt, quilt_offset=qoff,
    )  # fmt: skip
    np.testing.assert_array_equal(segs, wsegs)
    np.testing.assert_array_equal(nseg, wn)
    np.testing.assert_array_equal(Vt != 0, wV != 0)  # slot indexing: exactly the same cells written
    if kv_dt == "e4m3":
        np.testing.assert_array_equal(Vt, wV)  # e4m3 encodings of given values: bit-exact
        # K bytes depend on sin/cos of the temporal angle: allow the encoding to flip by one step
        # where the rotated value sits on a rounding boundary, nothing more, and only rarely
        diff = K != wK
        assert diff.mean() <= 2e-3, f"{diff.sum()} of {K.size} K bytes differ"
        assert np.all(np.abs(K.astype(np.int16)[diff] - wK.astype(np.int16)[diff]) <= 1)
    else:
        np.testing.assert_array_equal(Vt, wV)  # a bf16 V value is copied
        assert np.max(util.bf16_ulp_diff(K, wK)[np.abs(f32(wK, "bf16")) > 1e-2]) <= 2  # RN on the GPU, truncation in the oracle
        assert_close_bf16(K, wK, "K_cache")
    np.testing.assert_array_equal(K.any(axis=1), wK.any(axis=1))  # same rows written


def test_kv_cache_update_golden_cases(qb):
    z = np.load(G / "kv_cache_update.npz")
    Hq, Hk, H, W, nb = (int(v) for v in z["geometry"])
    for tag in z["cases"].tolist():
        kv_dt, pd, ft, frozen = tag.split("_")
        geo = dict(Hq=Hq, Hk=Hk, H=H, W=W, nb=nb, pd=int(pd), kv_dt=kv_dt)
        K, Vt, segs, nseg = _kv_run(qb, z["qkv"], int(ft), int(frozen), **geo)
        _check_kv(K, Vt, segs, nseg, z["qkv"], int(ft), int(frozen), **geo)
        np.testing.assert_array_equal(segs, z[f"{tag}.segments"])  # and against the reference's own output
        np.testing.assert_array_equal(nseg, z[f"{tag}.n_segments"])


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("H,W,pd,ft,frozen", [(16, 8, 1, 16, 1), (16, 8, 8, 128, 0), (8, 16, 8, 129, 0), (32, 16, 1, 5, 0), (32, 16, 8, 1000, 1)])
def test_kv_cache_update_model_geometry(qb, kv_dt, H, W, pd, ft, frozen):
    r = util.rng(ft)
    geo = dict(Hq=32, Hk=16, H=H, W=W, nb=16, pd=pd, kv_dt=kv_dt)
    qkv = bf16_randn(r, (H * W, 4096))
    K, Vt, segs, nseg = _kv_run(qb, qkv, ft, frozen, **geo)
    _check_kv(K, Vt, segs, nseg, qkv, ft, frozen, **geo)


def test_kv_cache_update_is_read_modify_write(qb):
    r = util.rng(5)
    geo = dict(Hq=4, Hk=2, H=8, W=8, nb=4, pd=1, kv_dt="bf16")
    qkv = bf16_randn(r, (64, 512))
    K, Vt, _, _ = _kv_run(qb, qkv, 3, 0, prefill=0x1234, **geo)
    cap = 5 * 64
    written = np.zeros(cap, bool)
    written[3 * 64 : 4 * 64] = True
    written[4 * 64 :] = True
    assert np.all(K.reshape(2, cap, 64)[:, ~written] == 0x1234)
    assert np.all(Vt.reshape(2, 64, cap)[:, :, ~written] == 0x1234)
    assert not np.any(K.reshape(2, cap, 64)[:, written] == 0x1234)


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("H,W,Hq,Hk,nb,pd,ft,frozen,with_first", [(8, 8, 4, 2, 4, 1, 6, 0, True), (16, 8, 32, 16, 16, 8, 128, 0, True),
                                                                  (32, 16, 32, 16, 16, 1, 129, 1, True), (8, 16, 32, 16, 16, 8, 64, 0, False)])  # fmt: skip
def test_qkv_post_is_bit_identical_to_the_three_kernels(qb, kv_dt, H, W, Hq, Hk, nb, pd, ft, frozen, with_first):
    r = util.rng(H * W + ft)
    qf = qb.qf
    tpf, cap, D = H * W, (nb + 1) * H * W, (Hq + 2 * Hk) * 64
    raw, first = bf16_randn(r, (tpf, D), 3.0), bf16_randn(r, (tpf, D))
    lam = T(qb, np.array([0.37], np.float32))
    geo = dict(B=1, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd, packed_qkv=True, n_q_heads=Hq)

    def state():
        carrier = np.uint16 if kv_dt == "bf16" else np.uint8
        return (T(qb, np.full((Hk * cap, 64), 0x11, carrier), kv_dt), T(qb, np.full((Hk * 64, cap), 0x22, carrier), kv_dt),
                T(qb, np.full(6, -7, np.int32)), T(qb, np.array([-7], np.int32)))  # fmt: skip

    ftt, frz = T(qb, np.array([ft], np.int32)), T(qb, np.array([frozen], np.int32))
    Ka, Va, sa, na = state()
    q1 = qf.head_rmsnorm(T(qb, raw, "bf16"), Hq, Hk, 64)
    if with_first:
        q1 = qf.value_residual_packed(q1, T(qb, first, "bf16"), lam, v_col_offset=(Hq + Hk) * 64, v_width=Hk * 64)
    qf.kv_cache_update(q1, None, ftt, frz, Va, sa, na, Ka, **geo)
    Kb, Vb, sb, nb_ = state()
    q2 = qf.qkv_post(T(qb, raw, "bf16"), T(qb, first, "bf16") if with_first else None, lam if with_first else None, ftt, frz, Vb, sb, nb_, Kb,
                     n_q_heads=Hq, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd)  # fmt: skip
    np.testing.assert_array_equal(q2.to_numpy(), q1.to_numpy())
    np.testing.assert_array_equal(Kb.to_numpy(), Ka.to_numpy())
    np.testing.assert_array_equal(Vb.to_numpy(), Va.to_numpy())
    np.testing.assert_array_equal(sb.to_numpy(), sa.to_numpy())
    np.testing.assert_array_equal(nb_.to_numpy(), na.to_numpy())


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("lin", ["bf16", "e4m3"])
@pytest.mark.parametrize("H,W,Hq,Hk,nb,pd,ft,frozen,with_first", [(8, 8, 4, 2, 4, 1, 6, 0, True), (8, 8, 2, 1, 4, 2, 9, 0, True),
                                                                  (16, 8, 32, 16, 16, 8, 128, 0, True), (32, 16, 32, 16, 16, 1, 129, 1, True),
                                                                  (8, 16, 32, 16, 16, 8, 64, 0, False)])  # fmt: skip
def test_gemm_qkv_post_is_bit_identical_to_gemm_then_qkv_post(qb, kv_dt, lin, H, W, Hq, Hk, nb, pd, ft, frozen, with_first):
    """The QKV projection with the fused epilogue writes the bytes of the projection followed by qkv_post
    (itself pinned to the three reference ops above): packed QKV, both caches, the segment table."""
    r = util.rng(H * W + ft + 1)
    qf = qb.qf
    tpf, cap, D, Kd = H * W, (nb + 1) * H * W, (Hq + 2 * Hk) * 64, 256
    x = bf16_randn(r, (tpf, Kd))
    first = bf16_randn(r, (tpf, D))
    if lin == "e4m3":
        A, Wt = T(qb, codec.f32_to_e4m3(f32(x, "bf16")), "e4m3"), T(qb, e4m3_randn(r, (D, Kd), 0.5), "e4m3")
    else:
        A, Wt = T(qb, x, "bf16"), T(qb, bf16_randn(r, (D, Kd), 0.1), "bf16")
    lam = T(qb, np.array([0.37], np.float32))

    def state():
        carrier = np.uint16 if kv_dt == "bf16" else np.uint8
        return (T(qb, np.full((Hk * cap, 64), 0x11, carrier), kv_dt), T(qb, np.full((Hk * 64, cap), 0x22, carrier), kv_dt),
                T(qb, np.full(6, -7, np.int32)), T(qb, np.array([-7], np.int32)))  # fmt: skip

    ftt, frz = T(qb, np.array([ft], np.int32)), T(qb, np.array([frozen], np.int32))
    kw = dict(n_q_heads=Hq, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd)
    fa, la = (T(qb, first, "bf16"), lam) if with_first else (None, None)
    Ka, Va, sa, na = state()
    raw = qf.gemm(A, Wt, out_dtype="bf16", compute_dtype="e4m3" if lin == "e4m3" else None, tile_n=128)
    q1 = qf.qkv_post(raw, fa, la, ftt, frz, Va, sa, na, Ka, **kw)
    Kb, Vb, sb, nb_ = state()
    q2 = qf.gemm_qkv_post(A, Wt, fa, la, ftt, frz, Vb, sb, nb_, Kb, **kw)
    np.testing.assert_array_equal(q2.to_numpy(), q1.to_numpy())
    np.testing.assert_array_equal(Kb.to_numpy(), Ka.to_numpy())
    np.testing.assert_array_equal(Vb.to_numpy(), Va.to_numpy())
    np.testing.assert_array_equal(sb.to_numpy(), sa.to_numpy())
    np.testing.assert_array_equal(nb_.to_numpy(), na.to_numpy())


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("lin", ["bf16", "e4m3"])
@pytest.mark.parametrize("H,W,Hq,Hk,nb,pd,quilt,qoff,ft,frozen", [(16, 8, 4, 2, 4, 1, 2, 1, 6, 0), (16, 16, 4, 2, 4, 2, 4, 2, 10, 0), (32, 16, 32, 16, 16, 8, 8, 5, 128, 0),
                                                                  (32, 16, 32, 16, 16, 1, 2, 0, 129, 1)])  # fmt: skip
def test_gemm_qkv_post_with_a_quilted_cache(qb, kv_dt, lin, H, W, Hq, Hk, nb, pd, quilt, qoff, ft, frozen):
    """quilt_factor > 1 in the fused QKV epilogue (src/quark/models/waypoint_15.py:108-112, :315-330: each layer's cache
    keeps one residue class of the frame's tokens): the bytes of the projection followed by head norm, value residual
    and the stand-alone append with the same quilt, which is pinned to the reference's quilted append elsewhere."""
    r = util.rng(H * W + ft + quilt)
    qf = qb.qf
    tpf, D, Kd = H * W, (Hq + 2 * Hk) * 64, 256
    cap = (nb + 1) * (tpf // quilt)
    x = bf16_randn(r, (tpf, Kd))
    first = T(qb, bf16_randn(r, (tpf, D)), "bf16")
    if lin == "e4m3":
        A, Wt = T(qb, codec.f32_to_e4m3(f32(x, "bf16")), "e4m3"), T(qb, e4m3_randn(r, (D, Kd), 0.5), "e4m3")
    else:
        A, Wt = T(qb, x, "bf16"), T(qb, bf16_randn(r, (D, Kd), 0.1), "bf16")
    lam = T(qb, np.array([0.37], np.float32))

    def state():
        carrier = np.uint16 if kv_dt == "bf16" else np.uint8
        return (T(qb, np.full((Hk * cap, 64), 0x11, carrier), kv_dt), T(qb, np.full((Hk * 64, cap), 0x22, carrier), kv_dt),
                T(qb, np.full(6, -7, np.int32)), T(qb, np.array([-7], np.int32)))  # fmt: skip

    ftt, frz = T(qb, np.array([ft], np.int32)), T(qb, np.array([frozen], np.int32))
    geo = dict(n_q_heads=Hq, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd)
    Ka, Va, sa, na = state()
    raw = qf.gemm(A, Wt, out_dtype="bf16", compute_dtype="e4m3" if lin == "e4m3" else None, tile_n=128)
    q1 = qf.value_residual_packed(qf.head_rmsnorm(raw, Hq, Hk, 64), first, lam, v_col_offset=(Hq + Hk) * 64, v_width=Hk * 64)
    qf.kv_cache_update(q1, None, ftt, frz, Va, sa, na, Ka, B=1, packed_qkv=True, quilt_factor=quilt, quilt_offset=qoff, **geo)
    Kb, Vb, sb, nb_ = state()
    q2 = qf.gemm_qkv_post(A, Wt, first, lam, ftt, frz, Vb, sb, nb_, Kb, quilt_factor=quilt, quilt_offset=qoff, **geo)
    np.testing.assert_array_equal(q2.to_numpy(), q1.to_numpy())
    np.testing.assert_array_equal(Kb.to_numpy(), Ka.to_numpy())
    np.testing.assert_array_equal(Vb.to_numpy(), Va.to_numpy())
    np.testing.assert_array_equal(sb.to_numpy(), sa.to_numpy())
    np.testing.assert_array_equal(nb_.to_numpy(), na.to_numpy())
    assert np.any(Ka.to_numpy() != 0x11)


# --------------------------------------------------------------------------- GEMM


def _gemm_case(qb, M, N, K, *, fp8=False, a_fp8=False, bias=False, act=None, gate_groups=0, split_k=0, tile_n=0, slice_mode=0, out_dtype="bf16", seed=0):
    r = util.rng(seed)
    A = bf16_randn(r, (M, K))
    if fp8:
        B = e4m3_randn(r, (N, K), 0.5)
        Aq = codec.f32_to_e4m3(f32(A, "bf16"))
    else:
        B = bf16_randn(r, (N, K), 0.05)
    kw, okw = {}, {}
    if bias:
        b = bf16_randn(r, (N,))
        kw["bias"], okw["bias"] = T(qb, b, "bf16"), b
    if gate_groups:
        g, res = bf16_randn(r, (gate_groups, N)), bf16_randn(r, (M, N))
        kw.update(gate=T(qb, g, "bf16"), residual=T(qb, res, "bf16"), gate_groups=gate_groups)
        okw.update(gate=g, residual=res, gate_groups=gate_groups)
    a_dev = T(qb, Aq, "e4m3") if (fp8 and a_fp8) else T(qb, A, "bf16")
    got = qb.qf.gemm(a_dev, T(qb, B, "e4m3" if fp8 else "bf16"), out_dtype=out_dtype, compute_dtype="e4m3" if fp8 else None,
                     activation=act, split_k=split_k, tile_n=tile_n, slice_mode=slice_mode, **kw)  # fmt: skip
    want32 = ops.gemm(A, B, b_dtype="e4m3" if fp8 else "bf16", a_quant="e4m3" if fp8 else None, activation=act, return_f32=True, **okw)
    return got, want32


def _check_gemm(got, want32, what, fp8):
    if got.dtype == "bf16":
        g = f32(got.to_numpy(), "bf16")
    elif got.dtype == "f32":
        g = got.to_numpy()
    else:
        g = f32(got.to_numpy(), "e4m3")
    assert np.all(np.isfinite(g)), what
    cs, mr = util.cosine(g, want32), util.max_rel(g, want32)
    if got.dtype == "e4m3":
        assert cs >= 0.995, f"{what}: cosine={cs:.6f}"  # 3 mantissa bits in the output itself
    elif fp8:
        assert cs >= util.COS_MIN and mr <= util.BF16_MAX_REL, f"{what}: cosine={cs:.6f} max_rel={mr:.3e}"
    else:
        assert mr <= util.BF16_MAX_REL and cs >= util.COS_MIN, f"{what}: max_rel={mr:.3e} cosine={cs:.6f}"


SMALL = [(64, 128, 256), (32, 64, 128), (128, 128, 256), (32, 64, 64), (200, 72, 80), (1, 8, 16), (130, 264, 2048 + 64)]


@pytest.mark.parametrize("M,N,K", SMALL)
@pytest.mark.parametrize("fp8", [False, True])
def test_gemm_small_and_ragged_shapes(qb, M, N, K, fp8):
    got, want = _gemm_case(qb, M, N, K, fp8=fp8, seed=M + N + K)
    _check_gemm(got, want, f"gemm {M}x{N}x{K} fp8={fp8}", fp8)


@pytest.mark.parametrize("fp8", [False, True])
def test_gemm_epilogues(qb, fp8):
    for kw in [dict(bias=True), dict(act="silu"), dict(bias=True, act="silu"), dict(gate_groups=1), dict(gate_groups=4),
               dict(out_dtype="f32"), dict(out_dtype="e4m3", act="silu"), dict(a_fp8=True)]:  # fmt: skip
        if kw.get("a_fp8") and not fp8:
            continue
        got, want = _gemm_case(qb, 128, 256, 512, fp8=fp8, seed=11, **kw)
        _check_gemm(got, want, f"epilogue {kw} fp8={fp8}", fp8)


def test_gemm_matches_golden_fixture(qb):
    z = np.load(G / "gemm.npz")
    A, B = T(qb, z["A"], "bf16"), T(qb, z["B"], "bf16")
    qf = qb.qf
    assert_close_bf16(qf.gemm(A, B).to_numpy(), z["plain"], "plain")
    assert_close_bf16(qf.gemm(A, B, bias=T(qb, z["bias"], "bf16"), activation="silu").to_numpy(), z["bias_silu"], "bias_silu")
    assert_close_bf16(qf.gemm(A, B, gate=T(qb, z["gate"][:1], "bf16"), residual=T(qb, z["resid"], "bf16")).to_numpy(), z["gate1"], "gate1")
    assert_close_bf16(qf.gemm(A, B, gate=T(qb, z["gate"], "bf16"), residual=T(qb, z["resid"], "bf16"), gate_groups=4).to_numpy(), z["gate4"], "gate4")


@pytest.mark.parametrize("M", [128, 512])
@pytest.mark.parametrize("name,N,K,extra", [("qkv", 4096, 2048, {}), ("out", 2048, 2048, dict(gate_groups=1)), ("fc1", 8192, 2048, {}), ("fc2", 2048, 8192, dict(gate_groups=1))])
@pytest.mark.parametrize("fp8", [False, True])
def test_gemm_production_shapes(qb, M, name, N, K, extra, fp8):
    got, want = _gemm_case(qb, M, N, K, fp8=fp8, seed=7, **extra)
    _check_gemm(got, want, f"{name} M={M} fp8={fp8}", fp8)


@pytest.mark.parametrize("split_k,tile_n,slice_mode", [(1, 64, 0), (1, 128, 0), (1, 256, 0), (2, 128, 0), (4, 64, 0), (8, 256, 0), (3, 128, 0),
                                                       (2, 256, 1), (4, 128, 1), (4, 256, 0), (2, 64, 0)])  # fmt: skip
@pytest.mark.parametrize("fp8", [False, True])
def test_gemm_forced_tiles_and_k_slices_agree(qb, split_k, tile_n, slice_mode, fp8):
    """K slices summed inside a thread-block cluster (2, 4, 8 slices, mode 0) or through the workspace."""
    got, want = _gemm_case(qb, 256, 512, 2048, fp8=fp8, gate_groups=1, split_k=split_k, tile_n=tile_n, slice_mode=slice_mode, seed=3)
    _check_gemm(got, want, f"split_k={split_k} tile_n={tile_n}", fp8)
    again, _ = _gemm_case(qb, 256, 512, 2048, fp8=fp8, gate_groups=1, split_k=split_k, tile_n=tile_n, slice_mode=slice_mode, seed=3)
    np.testing.assert_array_equal(got.to_numpy(), again.to_numpy())  # slice order is fixed: run-to-run identical


def test_gemm_scales_extension(qb):
    r = util.rng(9)
    A, B = bf16_randn(r, (128, 256)), e4m3_randn(r, (64, 256))
    ws = (0.5 + r.random(64)).astype(np.float32)
    got = qb.qf.gemm(T(qb, A, "bf16"), T(qb, B, "e4m3"), compute_dtype="e4m3", a_scale=T(qb, np.array([0.25], np.float32)), w_scale=T(qb, ws))
    want = ops.gemm(A, B, b_dtype="e4m3", a_quant="e4m3", return_f32=True) * 0.25 * ws[None, :]
    _check_gemm(got, want, "scaled fp8", True)


# --------------------------------------------------------------------------- owl_attn


def _attn_run(qb, qkv, Kc, Vc, segs, nseg, ft, *, Hk, gqa, H, W, nb, pd, kv_dt):
    return qb.qf.owl_attn(
        T(qb, qkv, "bf16"), T(qb, Kc, kv_dt), T(qb, Vc, kv_dt), T(qb, np.asarray(segs, np.int32)), T(qb, np.asarray(nseg, np.int32).reshape(1)),
        1, Hk, gqa, H, W, nb, pd, compute_dtype="e4m3" if kv_dt == "e4m3" else None, packed_qkv=True, frame_t=T(qb, np.array([ft], np.int32)),
    ).to_numpy()  # fmt: skip


def _attn_check(got, want_u16, what, fp8):
    g, w = f32(got, "bf16"), f32(want_u16, "bf16")
    assert np.all(np.isfinite(g)), what
    cs, mr = util.cosine(g, w), util.max_rel(g, w)
    if fp8:
        assert cs >= util.COS_MIN, f"{what}: cosine={cs:.6f} max_rel={mr:.3e}"
    else:
        assert mr <= util.BF16_MAX_REL and cs >= util.COS_MIN, f"{what}: max_rel={mr:.3e} cosine={cs:.6f}"


def test_owl_attn_golden_cases(qb):
    z = np.load(G / "owl_attn.npz")
    Hk, gqa, H, W, nb = (int(v) for v in z["geometry"])
    for tag in z["cases"].tolist():
        kv_dt, pd, ft = tag.split("_")
        got = _attn_run(qb, z["qkv"], z[f"K_{kv_dt}"], z[f"Vt_{kv_dt}"], z[f"{tag}.segments"], z[f"{tag}.n_segments"], int(ft),
                        Hk=Hk, gqa=gqa, H=H, W=W, nb=nb, pd=int(pd), kv_dt=kv_dt)  # fmt: skip
        _attn_check(got, z[f"{tag}.out"], f"golden {tag}", kv_dt == "e4m3")


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("H,W,pd,ft", [(16, 8, 1, 16), (16, 8, 8, 129), (8, 16, 1, 3), (32, 16, 8, 128), (32, 16, 1, 129)])
def test_owl_attn_model_geometry(qb, kv_dt, H, W, pd, ft):
    r = util.rng(100 + ft)
    Hk, gqa, nb = 16, 2, 16
    tpf, cap = H * W, 17 * H * W
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, 4096)), n_q_heads=32, n_kv_heads=16)
    if kv_dt == "bf16":
        Kc, Vc = bf16_randn(r, (Hk * cap, 64)), bf16_randn(r, (Hk * 64, cap))
    else:
        Kc, Vc = e4m3_randn(r, (Hk * cap, 64)), e4m3_randn(r, (Hk * 64, cap))
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    got = _attn_run(qb, qkv, Kc, Vc, segs, [n], ft, Hk=Hk, gqa=gqa, H=H, W=W, nb=nb, pd=pd, kv_dt=kv_dt)
    want = ops.owl_attn(qkv, Kc, Vc, segs, [n], ft, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype=kv_dt,
                        q_quant="e4m3" if kv_dt == "e4m3" else None)  # fmt: skip
    _attn_check(got, want, f"attn {H}x{W} pd={pd} ft={ft} {kv_dt}", kv_dt == "e4m3")


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("direction", ["rising", "falling"])
def test_owl_attn_score_scale_drifts_along_the_cache(qb, kv_dt, direction):
    """Key magnitude ramps along the cache rows, so the row maxima jump from tile to tile (rising: the
    running maximum has to be raised again and again; falling: it stays at the first tile's)."""
    r = util.rng(41)
    Hk, gqa, H, W, nb, pd, ft = 2, 2, 16, 16, 8, 1, 20
    tpf, cap = H * W, (nb + 1) * H * W
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, 8 * 64)), n_q_heads=4, n_kv_heads=2)
    ramp = np.linspace(0.25, 14.0, cap, dtype=np.float32)
    if direction == "falling":
        ramp = ramp[::-1]
    Kf = r.standard_normal((Hk, cap, 64), dtype=np.float32) * ramp[None, :, None]
    Vf = r.standard_normal((Hk, 64, cap), dtype=np.float32)
    to = codec.f32_to_bf16 if kv_dt == "bf16" else codec.f32_to_e4m3
    Kc, Vc = to(Kf.reshape(Hk * cap, 64)), to(Vf.reshape(Hk * 64, cap))
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    got = _attn_run(qb, qkv, Kc, Vc, segs, [n], ft, Hk=Hk, gqa=gqa, H=H, W=W, nb=nb, pd=pd, kv_dt=kv_dt)
    # scores reach +-60 here, so one bf16 ulp on a rotated query moves a probability by 20 %: the
    # oracle is fed the rotated query narrowed the way the kernel narrows it for its MMAs (bf16 or
    # e4m3, nearest even), which the reference oracle keeps in f32
    with codec.bf16_rounding("rne"):
        want = ops.owl_attn(qkv, Kc, Vc, segs, [n], ft, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype=kv_dt,
                            q_quant=kv_dt)  # fmt: skip
    _attn_check(got, want, f"attn drifting scale {direction} {kv_dt}", kv_dt == "e4m3")


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("H,W,pd,ft,splits", [(16, 8, 1, 16, 0), (16, 8, 8, 129, 3), (8, 8, 1, 5, 8), (32, 16, 1, 129, 2)])
def test_owl_attn_keys_shared_by_several_ctas(qb, kv_dt, H, W, pd, ft, splits):
    """Key splits (chosen at 360p, where 32 CTAs would leave most SMs idle; forced otherwise, also to more
    shares than there are key tiles): same result as one CTA per (query tile, head) up to the order of the
    sums, the same bytes on every call, and the oracle's result within the usual tolerance."""
    r = util.rng(300 + ft)
    Hk, gqa, nb = 16, 2, 16
    tpf, cap = H * W, 17 * H * W
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, 4096)), n_q_heads=32, n_kv_heads=16)
    if kv_dt == "bf16":
        Kc, Vc = bf16_randn(r, (Hk * cap, 64)), bf16_randn(r, (Hk * 64, cap))
    else:
        Kc, Vc = e4m3_randn(r, (Hk * cap, 64)), e4m3_randn(r, (Hk * 64, cap))
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    args = (T(qb, qkv, "bf16"), T(qb, Kc, kv_dt), T(qb, Vc, kv_dt), T(qb, np.asarray(segs, np.int32)), T(qb, np.array([n], np.int32)), 1, Hk, gqa, H, W, nb, pd)
    kw = dict(compute_dtype="e4m3" if kv_dt == "e4m3" else None, packed_qkv=True, frame_t=T(qb, np.array([ft], np.int32)))
    one = qb.qf.owl_attn(*args, kv_splits=1, **kw).to_numpy()
    got = qb.qf.owl_attn(*args, kv_splits=splits, **kw).to_numpy()
    again = qb.qf.owl_attn(*args, kv_splits=splits, **kw).to_numpy()
    np.testing.assert_array_equal(got, again)
    g, w = f32(got, "bf16"), f32(one, "bf16")
    # e4m3 probabilities are rounded relative to each share's own running maximum (and, by default, every second one
    # comes from the chord of 2^x, whose error depends on that maximum too)
    assert util.cosine(g, w) >= (util.COS_MIN if kv_dt == "e4m3" else 0.99999) and (kv_dt == "e4m3" or util.max_rel(g, w) <= 1e-2)
    if kv_dt == "e4m3":  # with every exponential from the special-function unit the two orders agree more closely
        was = qb._lib.set_attn_exact_exp(True)
        try:
            e1 = qb.qf.owl_attn(*args, kv_splits=1, **kw).to_numpy()
            es = qb.qf.owl_attn(*args, kv_splits=splits, **kw).to_numpy()
        finally:
            qb._lib.set_attn_exact_exp(was)
        assert util.cosine(f32(es, "bf16"), f32(e1, "bf16")) >= 0.9995
    want = ops.owl_attn(qkv, Kc, Vc, segs, [n], ft, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype=kv_dt,
                        q_quant="e4m3" if kv_dt == "e4m3" else None)  # fmt: skip
    _attn_check(got, want, f"attn split {splits} {H}x{W} pd={pd} ft={ft} {kv_dt}", kv_dt == "e4m3")


def test_owl_attn_e4m3_side_output_is_the_narrowed_bf16_output(qb):
    r = util.rng(31)
    Hk, gqa, H, W, nb, pd, ft = 2, 2, 16, 8, 4, 1, 9
    tpf, cap = H * W, (nb + 1) * H * W
    qkv = bf16_randn(r, (tpf, 8 * 64))
    Kc, Vc = e4m3_randn(r, (Hk * cap, 64)), e4m3_randn(r, (Hk * 64, cap))
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    oq = qb.QuarkTensor.empty(tpf, 4 * 64, dtype="e4m3")
    out = qb.qf.owl_attn(T(qb, qkv, "bf16"), T(qb, Kc, "e4m3"), T(qb, Vc, "e4m3"), T(qb, segs), T(qb, np.array([n], np.int32)), 1, Hk, gqa, H, W,
                         nb, pd, compute_dtype="e4m3", packed_qkv=True, frame_t=T(qb, np.array([ft], np.int32)), out_q=oq).to_numpy()  # fmt: skip
    np.testing.assert_array_equal(oq.to_numpy(), codec.f32_to_e4m3(codec.bf16_to_f32(out)))


def test_owl_attn_masked_bucket_is_never_read(qb):
    """NaN-poison the bucket the segment table masks: the output must not change."""
    r = util.rng(77)
    Hk, gqa, H, W, nb, pd, ft = 2, 2, 16, 8, 4, 1, 6  # post-wrap write frame: slot 2 masked
    tpf, cap = H * W, (nb + 1) * H * W
    qkv = bf16_randn(r, (tpf, 8 * 64))
    Kc, Vc = bf16_randn(r, (Hk * cap, 64)), bf16_randn(r, (Hk * 64, cap))
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    assert n == 3
    base = _attn_run(qb, qkv, Kc, Vc, segs, [n], ft, Hk=Hk, gqa=gqa, H=H, W=W, nb=nb, pd=pd, kv_dt="bf16")
    Kp, Vp = Kc.copy().reshape(Hk, cap, 64), Vc.copy().reshape(Hk, 64, cap)
    Kp[:, 2 * tpf : 3 * tpf, :] = 0x7FC0
    Vp[:, :, 2 * tpf : 3 * tpf] = 0x7FC0
    poisoned = _attn_run(qb, qkv, Kp.reshape(Hk * cap, 64), Vp.reshape(Hk * 64, cap), segs, [n], ft, Hk=Hk, gqa=gqa, H=H, W=W, nb=nb, pd=pd, kv_dt="bf16")
    np.testing.assert_array_equal(base, poisoned)


def test_owl_attn_empty_segments_give_zero(qb):
    r = util.rng(78)
    Hk, gqa, H, W, nb = 2, 2, 8, 8, 4
    tpf, cap = 64, 5 * 64
    got = _attn_run(qb, bf16_randn(r, (tpf, 512)), bf16_randn(r, (Hk * cap, 64)), bf16_randn(r, (Hk * 64, cap)), [0, 0, 0, 0, 0, 0], [2], 0,
                    Hk=Hk, gqa=gqa, H=H, W=W, nb=nb, pd=1, kv_dt="bf16")  # fmt: skip
    assert not got.any()


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("nb", [64, 256])
def test_owl_attn_long_histories(qb, kv_dt, nb):
    """The histories of the isolated attention sweep: 64 and 256 buckets of 512 tokens (capacity up to 131 584 rows
    per head, tensor maps of 2.1 M rows), global-bucket geometry (dilation 8), on a write frame after the ring has
    wrapped (three segments, one bucket masked) and on the frame after (two segments).  The kernel runs on all 32
    heads; the oracle (src/quark/kernels/owl_attn/reference.py:47-111) on the four Q heads of the first and the last
    KV head, which it finishes in seconds."""
    H, W, Hk, gqa, pd = 32, 16, 16, 2, 8
    tpf, cap = H * W, (nb + 1) * H * W
    r = util.rng(500 + nb)
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, 4096)), n_q_heads=32, n_kv_heads=16)
    Kf = r.standard_normal((Hk * cap, 64), dtype=np.float32)
    Vf = r.standard_normal((Hk * 64, cap), dtype=np.float32)
    if kv_dt == "bf16":
        Kd, Vd = T(qb, codec.f32_to_bf16(Kf), "bf16"), T(qb, codec.f32_to_bf16(Vf), "bf16")
    else:  # the device narrowing is bit-exact against the oracle's encoder (tested above); the host encodes the compared heads only
        Kd, Vd = qb.qf.quantize_e4m3(T(qb, Kf)), qb.qf.quantize_e4m3(T(qb, Vf))
    heads = [0, Hk - 1]
    to = codec.f32_to_bf16 if kv_dt == "bf16" else codec.f32_to_e4m3
    Ks = to(np.concatenate([Kf[h * cap : (h + 1) * cap] for h in heads]))
    Vs = to(np.concatenate([Vf[h * 64 : (h + 1) * 64] for h in heads]))
    del Kf, Vf
    qcols = np.concatenate([np.arange(2 * h * 64, (2 * h + 2) * 64) for h in heads])
    qkv_sub = np.concatenate([qkv[:, qcols], np.zeros((tpf, 2 * len(heads) * 64), np.uint16)], axis=1)
    for ft in (nb * pd, nb * pd + 1):
        segs, n = ops.compute_segments(ft, nb, tpf, pd)
        assert n == (3 if ft == nb * pd else 2)
        got = qb.qf.owl_attn(T(qb, qkv, "bf16"), Kd, Vd, T(qb, np.asarray(segs, np.int32)), T(qb, np.array([n], np.int32)), 1, Hk, gqa, H, W, nb, pd,
                             compute_dtype="e4m3" if kv_dt == "e4m3" else None, packed_qkv=True, frame_t=T(qb, np.array([ft], np.int32))).to_numpy()  # fmt: skip
        want = ops.owl_attn(qkv_sub, Ks, Vs, segs, [n], ft, n_kv_heads=len(heads), gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype=kv_dt,
                            q_quant="e4m3" if kv_dt == "e4m3" else None)  # fmt: skip
        _attn_check(got[:, qcols], want, f"attn {nb} buckets ft={ft} {kv_dt}", kv_dt == "e4m3")
        assert np.all(np.isfinite(f32(got, "bf16")))


@pytest.mark.parametrize("splits", [1, 3])
def test_owl_attn_per_head_scales(qb, splits):
    """k_scale / v_scale (an extension: the reference's e4m3 is scale free): the caches hold K / k_scale[h] and
    V / v_scale[h] in e4m3 and the kernel computes S = (Q . Kq^T) * k_scale[h] / 8, O = (P . Vq) * v_scale[h].
    Against the oracle run on the de-scaled caches; NULL scales are the scale-free kernel, bit for bit."""
    r = util.rng(61)
    Hk, gqa, H, W, nb, pd, ft = 4, 2, 16, 16, 8, 1, 11
    tpf, cap = H * W, (nb + 1) * H * W
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, (Hk * gqa + 2 * Hk) * 64)), n_q_heads=Hk * gqa, n_kv_heads=Hk)
    ks = np.array([0.5, 0.03125, 1.75, 0.011], np.float32)
    vs = np.array([2.0, 0.0625, 0.4, 0.02], np.float32)
    Kf = r.standard_normal((Hk, cap, 64), dtype=np.float32)
    Vf = r.standard_normal((Hk, 64, cap), dtype=np.float32)
    Kq = codec.f32_to_e4m3(Kf * (np.float32(1) / ks)[:, None, None]).reshape(Hk * cap, 64)
    Vq = codec.f32_to_e4m3(Vf * (np.float32(1) / vs)[:, None, None]).reshape(Hk * 64, cap)
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    args = (T(qb, qkv, "bf16"), T(qb, Kq, "e4m3"), T(qb, Vq, "e4m3"), T(qb, np.asarray(segs, np.int32)), T(qb, np.array([n], np.int32)), 1, Hk, gqa, H, W, nb, pd)
    kw = dict(compute_dtype="e4m3", packed_qkv=True, frame_t=T(qb, np.array([ft], np.int32)), kv_splits=splits)
    got = qb.qf.owl_attn(*args, k_scale=T(qb, ks), v_scale=T(qb, vs), **kw).to_numpy()
    # the oracle on the values the scaled bytes stand for
    Kd = (codec.e4m3_to_f32(Kq).reshape(Hk, cap, 64) * ks[:, None, None]).reshape(Hk * cap, 64)
    Vd = (codec.e4m3_to_f32(Vq).reshape(Hk, 64, cap) * vs[:, None, None]).reshape(Hk * 64, cap)
    want = ops.owl_attn(qkv, Kd, Vd, segs, [n], ft, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype="f32", q_quant="e4m3")
    _attn_check(got, want, f"attn with per-head scales, splits={splits}", True)
    for h in range(Hk * gqa):  # per head, so that a scale applied to the wrong head cannot hide in the average
        _attn_check(got[:, h * 64 : (h + 1) * 64], want[:, h * 64 : (h + 1) * 64], f"scaled attn head {h}", True)
    ones = np.ones(Hk, np.float32)
    a = qb.qf.owl_attn(*args, **kw).to_numpy()
    b = qb.qf.owl_attn(*args, k_scale=T(qb, ones), v_scale=T(qb, ones), **kw).to_numpy()
    np.testing.assert_array_equal(a, b)


def test_gemm_calls_of_different_shapes_share_one_workspace(qb):
    """The tile counters sit in a fixed area at the start of the workspace: a call that leaves an e4m3 copy of A
    (or partial sums) in the workspace must not disturb a later call that sums K slices through it with more
    tiles than the first call had, and a workspace that grows is retired, not freed (a captured CUDA graph may
    still hold its address)."""
    from quark_b200 import functional as qfm

    got1, want1 = _gemm_case(qb, 128, 256, 512, fp8=True, seed=21)  # bf16 A: narrowed into the workspace
    _check_gemm(got1, want1, "fp8 GEMM with a bf16 A", True)
    ws_before = qfm._workspace(0)
    # 512 x 4096 in 64-column tiles = 256 tiles... and 1024 x 4096 = 512 tiles, three K slices through the workspace
    for M in (512, 1024):
        one, want = _gemm_case(qb, M, 4096, 768, fp8=True, split_k=1, tile_n=64, seed=22)
        got, _ = _gemm_case(qb, M, 4096, 768, fp8=True, split_k=3, tile_n=64, slice_mode=1, seed=22)
        _check_gemm(got, want, f"workspace K slices after another shape, M={M}", True)
        again, _ = _gemm_case(qb, M, 4096, 768, fp8=True, split_k=3, tile_n=64, slice_mode=1, seed=22)
        np.testing.assert_array_equal(got.to_numpy(), again.to_numpy())
        assert util.cosine(f32(got.to_numpy(), "bf16"), f32(one.to_numpy(), "bf16")) >= 0.99999
    ws_after = qfm._workspace(0)
    if ws_after is not ws_before:  # it grew: the old buffer must still be owned
        assert any(t is ws_before for t in qfm._RETIRED_WS)


# --------------------------------------------------------------------------- randn


@pytest.mark.parametrize("n", [2048, 1000, 3 * 2048 + 40, 65536])
def test_randn_against_oracle(qb, n):
    """Philox words are integers and exact; the Box-Muller transcendentals differ in the last bits between numpy
    and the device library, so f32 normals are held to 2e-5 (|z| < 5.9) and bf16 ones to one unit in the last place,
    with at least 99.5 % of them bit-equal."""
    ctr = T(qb, np.array([5], np.int32))
    got = qb.qf.randn(shape=(n,), dtype="f32", counter_offset=ctr).to_numpy()
    want = ops.randn(n, 5)
    assert got.shape == (n,) and np.all(np.isfinite(got))
    assert float(np.abs(got - want).max()) <= 2e-5
    gb = qb.qf.randn(shape=(1, n), dtype="bf16", counter_offset=ctr).to_numpy().reshape(-1)
    with codec.bf16_rounding("rne"):
        wb = ops.randn(n, 5, dtype="bf16")
    gf, wf = f32(gb, "bf16"), f32(wb, "bf16")
    assert np.all(np.abs(gf - wf) <= np.abs(wf) * 2.0**-7 + 2e-5)
    assert float((gb == wb).mean()) >= 0.995


def test_randn_is_a_function_of_counter_stride_and_seeds(qb):
    n = 4096
    draw = lambda c, **kw: qb.qf.randn(shape=(n,), dtype="bf16", counter_offset=T(qb, np.array([c], np.int32)), **kw).to_numpy()  # noqa: E731
    a = draw(3)
    np.testing.assert_array_equal(a, draw(3))  # stateless: same counter, same draw
    assert not np.array_equal(a, draw(4))
    np.testing.assert_array_equal(draw(3, counter_stride=256), draw(768))
    np.testing.assert_array_equal(draw(512)[:2048], draw(0)[2048:])  # 512 counters per block of 2048
    assert not np.array_equal(a, draw(3, seed0=1))
    assert not np.array_equal(a, draw(3, seed1=1))
    # writes into a caller's buffer, and only n elements of it
    buf = T(qb, np.full(n + 16, 0x7FC0, np.uint16), "bf16")
    view = qb.QuarkTensor(buf._storage, (n,), "bf16", 0)
    qb.qf.randn(shape=(n,), dtype="bf16", counter_offset=T(qb, np.array([3], np.int32)), out=view)
    back = buf.to_numpy()
    np.testing.assert_array_equal(back[:n], a)
    assert np.all(back[n:] == 0x7FC0)
    with pytest.raises(ValueError):
        qb.qf.randn(shape=(n,), dtype="e4m3", counter_offset=T(qb, np.array([3], np.int32)))
    with pytest.raises(TypeError):
        qb.qf.randn(shape=(n,), counter_offset=T(qb, np.zeros(2, np.int32)))


# --------------------------------------------------------------------------- cache dtype != compute dtype


def test_dequantize_e4m3_is_exact_for_every_code(qb):
    codes = np.tile(np.arange(256, dtype=np.uint8), 5)[:1275]  # ragged length: tail path too
    got = qb.qf.dequantize_e4m3(T(qb, codes, "e4m3")).to_numpy()
    want = codec.f32_to_bf16(codec.e4m3_to_f32(codes))
    nan = np.isnan(codec.e4m3_to_f32(codes))
    np.testing.assert_array_equal(got[~nan], want[~nan])
    assert np.all(np.isnan(f32(got[nan], "bf16"))) and nan.sum() == int(np.isin(codes, [0x7F, 0xFF]).sum()) == 9


@pytest.mark.parametrize("kv_dt,compute", [("e4m3", "bf16"), ("bf16", "e4m3")])
def test_owl_attn_cache_dtype_differs_from_compute_dtype(qb, kv_dt, compute):
    """Cast on load (``src/quark/kernels/owl_attn/kernel.py:342-348``): the result equals attention over a cache
    that already holds the cast values, bit for bit, and the oracle's within the usual bound."""
    r = util.rng(91)
    Hk, gqa, H, W, nb, pd, ft = 2, 2, 16, 8, 4, 1, 6
    tpf, cap = H * W, (nb + 1) * H * W
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, 8 * 64)), n_q_heads=4, n_kv_heads=2)
    if kv_dt == "e4m3":
        Kc, Vc = e4m3_randn(r, (Hk * cap, 64)), e4m3_randn(r, (Hk * 64, cap))
        Kx, Vx = codec.f32_to_bf16(codec.e4m3_to_f32(Kc)), codec.f32_to_bf16(codec.e4m3_to_f32(Vc))
    else:
        Kc, Vc = bf16_randn(r, (Hk * cap, 64)), bf16_randn(r, (Hk * 64, cap))
        Kx, Vx = codec.f32_to_e4m3(codec.bf16_to_f32(Kc)), codec.f32_to_e4m3(codec.bf16_to_f32(Vc))
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    common = (T(qb, np.asarray(segs, np.int32)), T(qb, np.array([n], np.int32)), 1, Hk, gqa, H, W, nb, pd)
    kw = dict(compute_dtype=compute, packed_qkv=True, frame_t=T(qb, np.array([ft], np.int32)))
    got = qb.qf.owl_attn(T(qb, qkv, "bf16"), T(qb, Kc, kv_dt), T(qb, Vc, kv_dt), *common, **kw).to_numpy()
    direct = qb.qf.owl_attn(T(qb, qkv, "bf16"), T(qb, Kx, compute), T(qb, Vx, compute), *common, **kw).to_numpy()
    np.testing.assert_array_equal(got, direct)
    want = ops.owl_attn(qkv, Kx, Vx, segs, [n], ft, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype=compute,
                        q_quant="e4m3" if compute == "e4m3" else None)  # fmt: skip
    _attn_check(got, want, f"attn cache={kv_dt} compute={compute}", compute == "e4m3")


# --------------------------------------------------------------------------- separate Q / K / V (packed_qkv=False)


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
def test_separate_q_k_v_layout_equals_packed(qb, kv_dt):
    """``packed_qkv=False`` (the functional default upstream): Q, K, V and the output are head-major ``[heads * tpf,
    64]`` tensors (``src/quark/kernels/owl_attn/reference.py:62-69, 106-110``; ``kv_cache_update/reference.py:183-186``).
    Same bytes in the caches and, after regrouping, the same output bits as the packed call, which the oracle covers."""
    r = util.rng(57)
    Hq, Hk, H, W, nb, pd, ft = 4, 2, 16, 8, 4, 1, 6
    tpf, cap = H * W, (nb + 1) * H * W
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, (Hq + 2 * Hk) * 64)), n_q_heads=Hq, n_kv_heads=Hk)
    heads = lambda a, n: np.ascontiguousarray(a.reshape(tpf, n, 64).transpose(1, 0, 2)).reshape(n * tpf, 64)  # noqa: E731
    Q, K, V = heads(qkv[:, : Hq * 64], Hq), heads(qkv[:, Hq * 64 : (Hq + Hk) * 64], Hk), heads(qkv[:, (Hq + Hk) * 64 :], Hk)

    def state():
        z = lambda *s: qb.QuarkTensor.zeros(*s, dtype=kv_dt)  # noqa: E731
        return dict(Vt_cache=z(Hk * 64, cap), segments=T(qb, np.array([0, 0, nb * tpf, tpf, 0, 0], np.int32)),
                    n_segments=T(qb, np.array([2], np.int32)), K_cache=z(Hk * cap, 64))  # fmt: skip

    geo = dict(B=1, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd)
    ftt, frz = T(qb, np.array([ft], np.int32)), T(qb, np.array([0], np.int32))
    a, b = state(), state()
    qb.qf.kv_cache_update(T(qb, qkv, "bf16"), None, ftt, frz, **a, packed_qkv=True, n_q_heads=Hq, **geo)
    qb.qf.kv_cache_update(T(qb, K, "bf16"), T(qb, V, "bf16"), ftt, frz, **b, packed_qkv=False, **geo)
    for k in ("K_cache", "Vt_cache", "segments", "n_segments"):
        np.testing.assert_array_equal(a[k].to_numpy(), b[k].to_numpy(), err_msg=k)
    assert a["K_cache"].to_numpy().any()

    cd = "e4m3" if kv_dt == "e4m3" else None
    att = dict(gqa_ratio=Hq // Hk, compute_dtype=cd, frame_t=ftt)
    args = (a["K_cache"], a["Vt_cache"], a["segments"], a["n_segments"], 1, Hk)
    packed = qb.qf.owl_attn(T(qb, qkv, "bf16"), *args, att["gqa_ratio"], H, W, nb, pd, compute_dtype=cd, packed_qkv=True, frame_t=ftt).to_numpy()
    sep = qb.qf.owl_attn(T(qb, Q, "bf16"), *args, att["gqa_ratio"], H, W, nb, pd, compute_dtype=cd, frame_t=ftt)  # packed_qkv defaults to False
    assert tuple(sep.shape) == (Hq * tpf, 64)
    np.testing.assert_array_equal(sep.to_numpy(), heads(packed, Hq))
    with pytest.raises(ValueError):
        qb.qf.owl_attn(T(qb, qkv, "bf16"), *args, att["gqa_ratio"], H, W, nb, pd, compute_dtype=cd, frame_t=ftt)
    with pytest.raises(ValueError):
        qb.qf.kv_cache_update(T(qb, K, "bf16"), None, ftt, frz, **b, packed_qkv=False, **geo)


# --------------------------------------------------------------------------- quilt


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("quilt,qoff,ft", [(2, 1, 3), (4, 2, 9), (2, 0, 6)])
def test_quilted_cache_append_and_attention(qb, kv_dt, quilt, qoff, ft):
    """``quilt_factor > 1``: the cache keeps every quilt-th token of a frame (``kv_cache_update/reference.py:201-207``);
    two appends (one of them a ring write after the wrap) give the oracle's cache bytes and segment table, and
    attention over the quilted cache (all queries, fewer keys) the oracle's output."""
    r = util.rng(300 + quilt)
    Hq, Hk, H, W, nb, pd = 4, 2, 16, 16, 4, 1
    tpf = H * W
    tc = tpf // quilt
    cap = (nb + 1) * tc
    geo = dict(B=1, n_kv_heads=Hk, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd)
    Kd, Vd = qb.QuarkTensor.zeros(Hk * cap, 64, dtype=kv_dt), qb.QuarkTensor.zeros(Hk * 64, cap, dtype=kv_dt)
    segs, nseg = T(qb, np.array([0, 0, nb * tc, tc, 0, 0], np.int32)), T(qb, np.array([2], np.int32))
    Ko = Vo = None
    for f in (ft - 1, ft):
        qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, (Hq + 2 * Hk) * 64)), n_q_heads=Hq, n_kv_heads=Hk)
        qb.qf.kv_cache_update(T(qb, qkv, "bf16"), None, T(qb, np.array([f], np.int32)), T(qb, np.array([0], np.int32)), Vd, segs, nseg, Kd,
                              packed_qkv=True, n_q_heads=Hq, quilt_factor=quilt, quilt_offset=qoff, **geo)  # fmt: skip
        Ko, Vo, so, no = ops.kv_cache_update(qkv, f, 0, n_kv_heads=Hk, n_q_heads=Hq, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd,
                                             kv_dtype=kv_dt, K_cache=Ko, Vt_cache=Vo, quilt_factor=quilt, quilt_offset=qoff)  # fmt: skip
    assert Ko.shape == (Hk * cap, 64)
    np.testing.assert_array_equal(segs.to_numpy(), so)
    np.testing.assert_array_equal(nseg.to_numpy(), no)
    np.testing.assert_array_equal(Vd.to_numpy(), Vo)
    gK, wK = Kd.to_numpy(), Ko
    if kv_dt == "bf16":
        assert float(np.abs(f32(gK, "bf16") - f32(wK, "bf16")).max()) <= 2e-2  # rotation in f32, rounded vs truncated
    else:
        assert float((gK != wK).mean()) <= 2e-3  # an e4m3 rounding boundary now and then (device vs numpy cos / sin)
    np.testing.assert_array_equal(gK.any(axis=1), wK.any(axis=1))  # the same cache rows were written
    cd = "e4m3" if kv_dt == "e4m3" else None
    got = qb.qf.owl_attn(T(qb, qkv, "bf16"), Kd, Vd, segs, nseg, 1, Hk, Hq // Hk, H, W, nb, pd, compute_dtype=cd, packed_qkv=True,
                         quilt_factor=quilt, quilt_offset=qoff, frame_t=T(qb, np.array([ft], np.int32))).to_numpy()  # fmt: skip
    want = ops.owl_attn(qkv, gK, Vd.to_numpy(), so, no, ft, n_kv_heads=Hk, gqa_ratio=Hq // Hk, H_spatial=H, W_spatial=W, kv_dtype=kv_dt,
                        q_quant="e4m3" if kv_dt == "e4m3" else None)  # fmt: skip
    _attn_check(got, want, f"quilt {quilt}/{qoff} {kv_dt}", kv_dt == "e4m3")


# --------------------------------------------------------------------------- the reference's own problem lists

# name, n_kv_heads, H, W, num_buckets, pinned_dilation, kv dtype, quilt_factor, quilt_offset: the thirteen
# configurations of src/quark/kernels/kv_cache_update/problems.py:17-159 (B = 1, head_dim 64)
KV_PROBLEMS = [
    ("smoke_dense", 2, 8, 8, 4, 1, "bf16", 1, 0),
    ("owl_360p_dense", 16, 16, 8, 16, 1, "bf16", 1, 0),
    ("owl_360p_dilated", 16, 16, 8, 16, 8, "bf16", 1, 0),
    ("owl_720p_dense", 16, 32, 16, 16, 1, "bf16", 1, 0),
    ("owl_720p_dilated", 16, 32, 16, 16, 8, "bf16", 1, 0),
    ("owl_360p_dense_fp8", 16, 16, 8, 16, 1, "e4m3", 1, 0),
    ("owl_360p_dilated_fp8", 16, 16, 8, 16, 8, "e4m3", 1, 0),
    ("owl_720p_dense_fp8", 16, 32, 16, 16, 1, "e4m3", 1, 0),
    ("owl_720p_dilated_fp8", 16, 32, 16, 16, 8, "e4m3", 1, 0),
    ("quilt2_off0_360p_dense", 16, 16, 8, 16, 1, "bf16", 2, 0),
    ("quilt2_off1_360p_dense", 16, 16, 8, 16, 1, "bf16", 2, 1),
    ("quilt2_off0_360p_dense_fp8", 16, 16, 8, 16, 1, "e4m3", 2, 0),
    ("quilt4_off2_360p_dense_fp8", 16, 16, 8, 16, 1, "e4m3", 4, 2),
]


@pytest.mark.parametrize("name,Hk,H,W,nb,pd,kv_dt,quilt,qoff", KV_PROBLEMS, ids=[p[0] for p in KV_PROBLEMS])
def test_kv_cache_update_reference_problem_list(qb, name, Hk, H, W, nb, pd, kv_dt, quilt, qoff):
    """Every configuration the reference sweeps this kernel over (its ``make fuzz``), each on a ring-write frame
    after the wrap and on a frozen frame, against the oracle: segment table and V bytes exact, K as in ``_check_kv``."""
    r = util.rng(len(name) * 31 + H)
    Hq = 2 * Hk
    geo = dict(Hq=Hq, Hk=Hk, H=H, W=W, nb=nb, pd=pd, kv_dt=kv_dt, quilt=quilt, qoff=qoff)
    qkv = ops.head_rmsnorm(bf16_randn(r, (H * W, (Hq + 2 * Hk) * 64)), n_q_heads=Hq, n_kv_heads=Hk)
    for ft, frozen in ((pd * (nb + 3), 0), (pd * (nb + 3), 1)):
        K, Vt, segs, nseg = _kv_run(qb, qkv, ft, frozen, **geo)
        _check_kv(K, Vt, segs, nseg, qkv, ft, frozen, **geo)
        assert K.shape[0] == Hk * (nb + 1) * (H * W // quilt)


@pytest.mark.parametrize("kv_dt", ["bf16", "e4m3"])
@pytest.mark.parametrize("quilt,qoff", [(2, 0), (2, 1), (4, 2)])
def test_owl_attn_reference_quilt_problems(qb, kv_dt, quilt, qoff):
    """The three quilted configurations of ``src/quark/kernels/owl_attn/problems.py:26-90`` (360p, 16 buckets, 16 KV
    heads, GQA 2); its dense and dilated 360p / 720p ones are ``test_owl_attn_model_geometry``.  The cache holds
    128 / quilt tokens per frame, so key tiles end inside a tile and segments start off tile boundaries."""
    r = util.rng(500 + quilt + qoff)
    Hk, gqa, H, W, nb, pd, ft = 16, 2, 16, 8, 16, 1, 21
    tpf = H * W
    cap = (nb + 1) * (tpf // quilt)
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, 4096)), n_q_heads=32, n_kv_heads=16)
    if kv_dt == "bf16":
        Kc, Vc = bf16_randn(r, (Hk * cap, 64)), bf16_randn(r, (Hk * 64, cap))
    else:
        Kc, Vc = e4m3_randn(r, (Hk * cap, 64)), e4m3_randn(r, (Hk * 64, cap))
    segs, n = ops.compute_segments(ft, nb, tpf // quilt, pd)
    assert n == 3
    got = qb.qf.owl_attn(T(qb, qkv, "bf16"), T(qb, Kc, kv_dt), T(qb, Vc, kv_dt), T(qb, np.asarray(segs, np.int32)), T(qb, np.array([n], np.int32)),
                         1, Hk, gqa, H, W, nb, pd, compute_dtype="e4m3" if kv_dt == "e4m3" else None, packed_qkv=True, quilt_factor=quilt,
                         quilt_offset=qoff, frame_t=T(qb, np.array([ft], np.int32))).to_numpy()  # fmt: skip
    want = ops.owl_attn(qkv, Kc, Vc, segs, [n], ft, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype=kv_dt,
                        q_quant="e4m3" if kv_dt == "e4m3" else None)  # fmt: skip
    _attn_check(got, want, f"attn quilt {quilt}/{qoff} {kv_dt}", kv_dt == "e4m3")


# --------------------------------------------------------------------------- mixture of experts


def test_moe_route_and_combine(qb):
    r = util.rng(71)
    M, E, D, K = 200, 8, 64, 2
    logits = bf16_randn(r, (M, E))
    logits[5, :] = logits[5, 0]  # all equal: ties go to the lower index
    logits[6, 3] = logits[6, 7] = 0x4100  # a tie for the first place
    w = qb.qf.moe_route(T(qb, logits, "bf16"), top_k=K).to_numpy()
    want = ops.moe_route(logits, K)
    np.testing.assert_array_equal(w != 0, want != 0)
    assert float(np.abs(w - want).max()) <= 1e-6
    assert np.flatnonzero(w[:, 5]).tolist() == [0, 1] and np.flatnonzero(w[:, 6]).tolist() == [3, 7]
    np.testing.assert_allclose(w.sum(axis=0), 1.0, atol=1e-6)
    parts = r.standard_normal((E * M, D)).astype(np.float32)
    parts[(w == 0).reshape(-1)] = np.nan  # what an unused expert computed must never be read
    got = qb.qf.moe_combine(T(qb, parts), T(qb, w)).to_numpy()
    p3 = np.nan_to_num(parts).reshape(E, M, D)
    ref = np.zeros((M, D), np.float32)
    for e in range(E):
        ref = ref + w[e][:, None] * p3[e]
    with codec.bf16_rounding("rne"):
        wantb = codec.f32_to_bf16(ref)
    assert np.all(np.abs(got.astype(np.int32) - wantb.astype(np.int32)) <= 1)
    assert float((got == wantb).mean()) > 0.99


@pytest.mark.parametrize("M,E,K", [(200, 8, 2), (1500, 16, 3), (64, 8, 1)])
def test_moe_slot_tables(qb, M, E, K):
    """The routing as slot tables sorted by expert, every run padded to whole 128-row tiles: the tables are a function of
    the logits alone (slots of an expert in (token, k) order) and say the same as the dense weights
    (``src/quark/kernels/moe_router_correct/reference.py:38-120``)."""
    r = util.rng([72, M])
    logits = bf16_randn(r, (M, E))
    logits[5, :] = logits[5, 0]
    qf = qb.qf
    n = qf.moe_slots(M, E, K)
    assert n % 128 == 0 and n >= M * K
    counts = T(qb, np.full(E, -1, np.int32))
    st, sw, te, ts = qf.moe_route_slots(T(qb, logits, "bf16"), top_k=K, counts=counts)
    st, sw, te, ts, counts = st.to_numpy(), sw.to_numpy(), te.to_numpy(), ts.to_numpy().reshape(M, K), counts.to_numpy()
    dense = ops.moe_route(logits, K)  # [E, M]
    np.testing.assert_array_equal(counts, (dense != 0).sum(axis=1))
    # the oracle's tables (pinned at the reference's row tile of 32 to the reference's own router, tests/test_oracle_golden.py)
    want = ops.moe_route_slots(logits, K, tile=128, total_slots=n)
    np.testing.assert_array_equal(st, want["slot_token"])
    np.testing.assert_array_equal(ts, want["token_slot"])
    np.testing.assert_array_equal(te, want["tile_expert"])
    np.testing.assert_allclose(sw, want["slot_weight"], atol=1e-6)
    used = st >= 0
    assert np.all(sw[~used] == 0)
    exp_of_slot = np.repeat(te, 128)
    np.testing.assert_allclose(sw[used], dense[exp_of_slot[used], st[used]], atol=1e-6)
    # gather: rows in slot order, zeros for padding
    x = bf16_randn(r, (M, 64))
    xs = qf.moe_gather(T(qb, x, "bf16"), T(qb, st)).to_numpy()
    np.testing.assert_array_equal(xs[used], x[st[used]])
    assert not xs[~used].any()
    # reduce: each token's top_k partial rows, weighted, summed in f32
    parts = r.standard_normal((n, 32)).astype(np.float32)
    parts[~used] = np.nan  # padding rows are never read
    got = qf.moe_reduce(T(qb, parts), T(qb, sw), T(qb, ts)).to_numpy()
    ref = np.zeros((M, 32), np.float32)
    tss = np.sort(ts, axis=1)  # in order of increasing slot, i.e. of increasing expert index
    for k in range(K):
        ref = ref + sw[tss[:, k]][:, None] * parts[tss[:, k]]
    with codec.bf16_rounding("rne"):
        wantb = codec.f32_to_bf16(ref)
    assert np.all(util.bf16_ulp_diff(got, wantb) <= 1) and float((got == wantb).mean()) > 0.99


@pytest.mark.parametrize("fp8", [False, True])
def test_gemm_grouped_rows_use_their_experts_weights(qb, fp8):
    """128-row tiles of A against the weight block of the tile's expert; tiles marked -1 are left alone."""
    r = util.rng(73)
    E, N, K = 4, 96, 256
    tiles = np.array([2, 0, -1, 3, 3, -1], np.int32)
    Mrows = 128 * len(tiles)
    dt = "e4m3" if fp8 else "bf16"
    A = e4m3_randn(r, (Mrows, K)) if fp8 else bf16_randn(r, (Mrows, K))
    B = e4m3_randn(r, (E * N, K), 0.05) if fp8 else bf16_randn(r, (E * N, K), 0.05)
    out = T(qb, np.full((Mrows, N), 0x7FC0, np.uint16), "bf16")  # NaN: what a skipped tile must leave behind
    qb.qf.gemm_grouped(T(qb, A, dt), T(qb, B, dt), T(qb, tiles), n_experts=E, activation="silu", out=out, compute_dtype=dt)
    got = out.to_numpy()
    for i, e in enumerate(tiles):
        rows = slice(128 * i, 128 * i + 128)
        if e < 0:
            assert np.all(got[rows] == 0x7FC0)
            continue
        want = ops.gemm(A[rows], B[e * N : (e + 1) * N], a_dtype=dt, b_dtype=dt, activation="silu", return_f32=True)
        _check_gemm(T(qb, got[rows], "bf16"), want, f"tile {i} expert {e} fp8={fp8}", fp8)


@pytest.mark.parametrize("H,W", [(16, 8), (32, 16)])
def test_owl_attn_e4m3_exponentials_fast_and_exact(qb, H, W):
    """e4m3 attention builds every second probability from a chord of 2^x on the FMA pipe unless told otherwise: both
    settings stay inside the tolerance against the oracle, the exact one closer, and the switch changes the result."""
    r = util.rng(310 + H)
    Hk, gqa, nb, pd, ft = 16, 2, 16, 1, 129
    tpf, cap = H * W, 17 * H * W
    qkv = ops.head_rmsnorm(bf16_randn(r, (tpf, 4096)), n_q_heads=32, n_kv_heads=16)
    Kc, Vc = e4m3_randn(r, (Hk * cap, 64)), e4m3_randn(r, (Hk * 64, cap))
    segs, n = ops.compute_segments(ft, nb, tpf, pd)
    want = f32(ops.owl_attn(qkv, Kc, Vc, segs, [n], ft, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype="e4m3", q_quant="e4m3"), "bf16")
    res = {}
    for exact in (False, True):
        was = qb._lib.set_attn_exact_exp(exact)
        try:
            got = _attn_run(qb, qkv, Kc, Vc, segs, n, ft, Hk=Hk, gqa=gqa, H=H, W=W, nb=nb, pd=pd, kv_dt="e4m3")
        finally:
            qb._lib.set_attn_exact_exp(was)
        res[exact] = (got, 1.0 - util.cosine(f32(got, "bf16"), want))
    util.parity_report({"test": "owl_attn_e4m3_exponentials", "grid": [H, W], "fast_1mcos": float(f"{res[False][1]:.4g}"), "exact_1mcos": float(f"{res[True][1]:.4g}")})
    assert res[True][1] <= res[False][1] <= 1.0 - util.COS_MIN
    assert res[False][1] <= 0.7 * (1.0 - util.COS_MIN)  # and not by a hair
    assert np.any(res[False][0] != res[True][0])
