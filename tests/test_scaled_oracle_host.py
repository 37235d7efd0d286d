"""The restated formulas of the scaled-e4m3 mode (``oracle/ops.py``), checked on the host against their definition
and against the scale-free oracle they extend (the reference has no scales: ``src/quark/runtime/cublas.py:151-158``)."""

import numpy as np

from oracle import codec, ops
from tests import util


def test_row_scaled_narrowing_uses_the_whole_range_and_inverts():
    r = util.rng(1)
    x = codec.f32_to_bf16_rne((r.standard_normal((32, 256)) * np.exp2(r.integers(-10, 8, size=(32, 1)))).astype(np.float32))
    x[3] = 0
    q, s = ops.quantize_e4m3_rows(x)
    xf = codec.bf16_to_f32(x)
    assert s[3] == 1.0 and not q[3].any()
    live = np.arange(32) != 3
    np.testing.assert_array_equal(np.max(np.abs(codec.e4m3_to_f32(q[live])), axis=1), 448.0)
    back = codec.e4m3_to_f32(q) * s[:, None]
    big = (np.abs(xf) >= np.max(np.abs(xf), axis=1, keepdims=True) * 2.0**-6) & (xf != 0)  # normal e4m3 codes after scaling
    assert np.max(np.abs(back - xf)[big] / np.abs(xf)[big]) <= 2.0**-4 + 1e-6  # half a unit of 3 mantissa bits


def test_scaled_gemm_and_attention_reduce_to_the_scale_free_oracle_at_scale_one():
    r = util.rng(2)
    A, B = util.bf16_randn(r, (16, 64)), util.e4m3_randn(r, (24, 64))
    plain = ops.gemm(A, B, b_dtype="e4m3", a_quant="e4m3")
    np.testing.assert_array_equal(ops.gemm(A, B, b_dtype="e4m3", a_quant="e4m3", a_scale=np.float32(1), w_scale=np.ones(24, np.float32)), plain)
    w = (0.5 + r.random(24)).astype(np.float32)
    scaled = ops.gemm(A, B, b_dtype="e4m3", a_quant="e4m3", a_scale=np.float32(0.25), w_scale=w, return_f32=True)
    np.testing.assert_allclose(scaled, ops.gemm(A, B, b_dtype="e4m3", a_quant="e4m3", return_f32=True) * 0.25 * w[None], rtol=1e-6)

    H, W, Hk, gqa, nb, ft = 8, 8, 2, 2, 2, 5
    tpf, cap = H * W, (nb + 1) * H * W
    qkv = util.bf16_randn(r, (tpf, (Hk * gqa + 2 * Hk) * 64))
    geo = dict(n_kv_heads=Hk, n_q_heads=Hk * gqa, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=1, kv_dtype="e4m3")
    K0, V0, segs, n = ops.kv_cache_update(qkv, ft, 0, **geo)
    one = np.ones(Hk, np.float32)
    K1, V1, _, _ = ops.kv_cache_update(qkv, ft, 0, k_scale=one, v_scale=one, **geo)
    np.testing.assert_array_equal(K1, K0)
    np.testing.assert_array_equal(V1, V0)
    # power-of-two scales move the exponent only: the de-scaled cache is the scale-free cache wherever neither
    # side left the normal range, and attention over it with the same scales gives the scale-free result
    ks, vs = np.array([0.25, 0.0625], np.float32), np.array([0.5, 0.125], np.float32)
    K2, V2, _, _ = ops.kv_cache_update(qkv, ft, 0, k_scale=ks, v_scale=vs, **geo)
    kf0, kf2 = codec.e4m3_to_f32(K0).reshape(Hk, cap, 64), codec.e4m3_to_f32(K2).reshape(Hk, cap, 64) * ks[:, None, None]
    ok = (np.abs(kf0) >= 2.0**-5) & (np.abs(kf2) < 448 * ks[:, None, None])  # away from the subnormal spacing of either side
    np.testing.assert_array_equal(kf2[ok], kf0[ok])
    att = dict(n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype="e4m3", q_quant="e4m3", return_f32=True)
    a0 = ops.owl_attn(qkv, K0, V0, segs, n, ft, **att)
    a2 = ops.owl_attn(qkv, K2, V2, segs, n, ft, k_scale=ks, v_scale=vs, **att)
    assert util.cosine(a2, a0) >= 0.9995
