"""The AdaRMSNorm that follows out-proj / fc2 as the tail of that GEMM (``qb_gemm_norm``).

What it replaces is the pair ``gemm(+ gate, residual)`` -> ``ada_rmsnorm`` of the block wiring
(``src/quark/models/waypoint_15.py:413-440``).  The GEMM part must not change a bit.  The norm part sums the squares
tile by tile instead of thread by thread, so against the separate launch it may differ where that f32 sum rounds
differently: at most one bf16 ulp (one e4m3 code) on rare elements; against the oracle
(``oracle.ops.ada_rmsnorm``, ``src/quark/kernels/ada_rmsnorm/reference.py:10-29``) it is held to the strict tolerance.
"""

import numpy as np
import pytest

from oracle import codec, ops
from tests import util
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


CASES = [
    # M, N, K, fp8, gate_groups, norm_groups, activation, gated
    (512, 2048, 2048, True, 1, 1, None, True),    # out-proj at 720p
    (512, 2048, 8192, True, 1, 1, None, True),    # fc2 at 720p
    (512, 2048, 2048, False, 1, 1, "silu", True),  # the output norm, bf16
    (128, 2048, 2048, True, 1, 1, None, True),    # one row block
    (256, 512, 256, False, 2, 2, None, True),     # two row groups of one tile each
    (384, 1024, 512, True, 1, 3, None, False),    # no gate / residual; norm rows per 128-row tile
    (200, 256, 128, False, 1, 1, None, True),     # ragged M: rows past the end take no part
]


@pytest.mark.parametrize("M,N,K,fp8,gg,ng,act,gated", CASES)
def test_gemm_norm_against_the_separate_launches_and_the_oracle(qb, M, N, K, fp8, gg, ng, act, gated):
    qf = qb.qf
    r = util.rng([81, M, N, K])
    A = e4m3_randn(r, (M, K)) if fp8 else bf16_randn(r, (M, K))
    W = e4m3_randn(r, (N, K), 0.05) if fp8 else bf16_randn(r, (N, K), 0.05)
    dt = "e4m3" if fp8 else "bf16"
    gate, res = bf16_randn(r, (gg, N)), bf16_randn(r, (M, N))
    ns, nb = bf16_randn(r, (ng, N), 0.5), bf16_randn(r, (ng, N), 0.5)
    tA, tW, tg, tr, tns, tnb = T(qb, A, dt), T(qb, W, dt), T(qb, gate, "bf16"), T(qb, res, "bf16"), T(qb, ns, "bf16"), T(qb, nb, "bf16")
    gkw = dict(gate=tg, residual=tr, gate_groups=gg) if gated else {}
    # the separate launches
    x_ref = qf.gemm(tA, tW, out_dtype="bf16", compute_dtype=dt, tile_n=64 if N % 128 else 0, **gkw)
    h_ref = qb.QuarkTensor.empty(M, N, dtype="bf16")
    hq_ref = qb.QuarkTensor.empty(M, N, dtype="e4m3")
    qf.ada_rmsnorm(x_ref, tns, tnb, activation=act, out=h_ref, out_q=hq_ref)
    # one kernel, three times over (the row blocks' counters must be back at zero after every launch)
    outs = []
    for _ in range(3):
        x, h, hq = qf.gemm_norm(tA, tW, tns, tnb, emit_bf16=True, emit_e4m3=True, activation=act, compute_dtype=dt, **gkw)
        outs.append((x.to_numpy(), h.to_numpy(), hq.to_numpy()))
    qb.runtime.synchronize()
    assert qb._lib.device_status() == 0
    for o in outs[1:]:
        for a, b in zip(o, outs[0]):
            np.testing.assert_array_equal(a, b)
    gx, gh, ghq = outs[0]
    np.testing.assert_array_equal(gx, x_ref.to_numpy())  # the GEMM and its epilogue: not a bit changed
    ulp = util.bf16_ulp_diff(gh, h_ref.to_numpy())
    assert ulp.max() <= 1 and (ulp != 0).mean() <= 2e-3, (int(ulp.max()), float((ulp != 0).mean()))
    dq = np.abs(ghq.astype(np.int16) - hq_ref.to_numpy().astype(np.int16))
    assert dq.max() <= 1 and (dq != 0).mean() <= 2e-3
    # the e4m3 copy is the narrowing of the bf16 result, as a cast of it would give
    np.testing.assert_array_equal(ghq, codec.f32_to_e4m3(f32(gh, "bf16")))
    # the oracle's norm of the device's x
    with codec.bf16_rounding("rne"):
        want = ops.ada_rmsnorm(gx, ns, nb, activation=act)
    g, w = f32(gh, "bf16"), f32(want, "bf16")
    assert util.cosine(g, w) >= util.COS_MIN and util.max_rel(g, w) <= util.BF16_MAX_REL


def test_gemm_norm_rejects_what_the_tail_cannot_take(qb):
    qf = qb.qf
    r = util.rng(82)
    ns = T(qb, bf16_randn(r, (1, 4096)), "bf16")
    A, W = T(qb, bf16_randn(r, (1024, 64)), "bf16"), T(qb, bf16_randn(r, (4096, 64)), "bf16")
    assert not qf.gemm_norm_fits(1024, 4096)
    with pytest.raises(qb.QuarkError, match="fit the device"):  # 8 x 32 tiles of 128 columns: more than one per SM
        qf.gemm_norm(A, W, ns, ns)
    A, W = T(qb, bf16_randn(r, (128, 64)), "bf16"), T(qb, bf16_randn(r, (72, 64)), "bf16")
    ns = T(qb, bf16_randn(r, (1, 72)), "bf16")
    assert not qf.gemm_norm_fits(128, 72)
    with pytest.raises(qb.QuarkError):  # ragged N
        qf.gemm_norm(A, W, ns, ns)
    qb.runtime.synchronize()
    assert qb._lib.device_status() == 0


@pytest.mark.parametrize("quant", ["bf16", "fp8"])
def test_session_with_norm_tails_matches_the_separate_launches_and_replays(qb, quant):
    """A small model with the tails forced on: the frames stay within the strict tolerance of the session that
    launches every norm by itself, graph replay equals eager bit for bit, and of the 2 x layers + 1 norm launches of an
    NFE only the first block's pre-attention norm is left."""
    from tests.test_gpu_model import small_cfg
    from quark_b200.models import Waypoint15Config, make_params

    base = small_cfg(qb, quant)
    params = make_params(base, seed=23, weight_std=0.08)
    r = util.rng(83)
    lat = codec.f32_to_bf16(r.standard_normal((1, base.latent_numel)).astype(np.float32))
    noises = [r.standard_normal((1, base.latent_numel)).astype(np.float32) for _ in range(2)]
    got = {}
    launches = {}
    for name, fuse, graph in (("separate", False, True), ("tail", True, False), ("tail_graph", True, True)):
        cfg = Waypoint15Config(**{**base.__dict__, "fuse_norm": fuse})
        eng = qb.Engine(cfg=cfg, quant=cfg.quant, params=params, use_graph=graph)
        eng.append_frame(lat)
        got[name] = [eng.gen_frame(noise=nz).reshape(-1).copy() for nz in noises]
        launches[name] = eng.launches_per_frame if graph else None
        eng.close()
    for a, b in zip(got["tail"], got["tail_graph"]):
        np.testing.assert_array_equal(a, b)
    assert launches["separate"] - launches["tail_graph"] == 5 * 2 * base.n_layers
    for k, (a, b) in enumerate(zip(got["tail"], got["separate"])):
        g, w = f32(a, "bf16"), f32(b, "bf16")
        c, m = util.cosine(g, w), util.max_rel(g, w)
        assert c >= 0.9999 and m <= util.BF16_MAX_REL, f"frame {k}: cosine={c:.6f} max_rel={m:.3e}"
