"""Generate the golden fixtures in this folder from the reference's own CPU oracles.

Run where the reference tree is available (it is not needed to *use* the fixtures):

    python tests/golden/make_golden.py /path/to/reference

The script imports the reference's numpy references (``src/quark/kernels/*/reference.py``,
``src/quark/runtime/npconv.py``, ``src/quark/models/_waypoint_15_io.py``), runs them on small
seeded inputs and stores inputs and outputs as ``.npz`` files.  ``tests/test_oracle_golden.py``
replays every file against ``oracle/``.  The reference publishes no golden vectors for this
path, so these files are what pins the oracle to it.
"""

from __future__ import annotations

import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def _bf16(a):
    return (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def main(ref_root: str) -> None:
    sys.path.insert(0, str(Path(ref_root) / "src"))
    from quark.kernels.ada_gate_residual.reference import ada_gate_residual_reference_numpy
    from quark.kernels.ada_gate_residual.spec import AdaGateResidualSpec
    from quark.kernels.ada_rmsnorm.reference import ada_rmsnorm_reference_numpy
    from quark.kernels.ada_rmsnorm.spec import AdaRMSNormSpec
    from quark.kernels.gemm.reference import gemm_reference_numpy
    from quark.kernels.gemm.spec import GemmSpec
    from quark.kernels.head_rmsnorm.reference import head_rmsnorm_reference_numpy
    from quark.kernels.head_rmsnorm.spec import HeadRMSNormSpec
    from quark.kernels.kv_cache_update.reference import (
        _compute_segments,
        _make_ortho_rope_freqs,
        kv_cache_update_reference_numpy,
    )
    from quark.kernels.kv_cache_update.spec import KVCacheUpdateSpec
    from quark.kernels.owl_attn.reference import owl_attn_reference_numpy
    from quark.kernels.owl_attn.spec import OwlAttnSpec
    from quark.kernels.patchify.reference import patchify_reference_numpy
    from quark.kernels.patchify.spec import PatchifySpec
    from quark.kernels.silu.reference import silu_reference_numpy
    from quark.kernels.silu.spec import SiLUSpec
    from quark.kernels.unpatchify.reference import unpatchify_reference_numpy
    from quark.kernels.unpatchify.spec import UnpatchifySpec
    from quark.kernels.value_residual_packed.reference import value_residual_packed_reference_numpy
    from quark.kernels.value_residual_packed.spec import ValueResidualPackedSpec
    from quark.models import _waypoint_15_io as wio
    from quark.runtime import npconv

    rng = np.random.default_rng(0x5A1E5EED)

    # ---- codecs: every bf16 bit pattern through the reference e4m3 encoder, and the decode LUT
    all_bf16 = np.arange(65536, dtype=np.uint16)
    as_f32 = npconv.bf16_u16_to_f32(all_bf16)
    extra = np.array(
        [0.0, -0.0, 447.9, 448.0, 464.0, 1e9, -1e9, np.inf, -np.inf, np.nan, 2.0**-9, 2.0**-10, 1.5 * 2.0**-10, 0.0146484375, 0.015624, 0.3, -0.3, 17.0, 18.0, 19.0],
        dtype=np.float32,
    )
    np.savez_compressed(
        HERE / "codec.npz",
        e4m3_of_all_bf16=npconv.f32_to_e4m3_u8(as_f32),
        extra_f32=extra,
        e4m3_of_extra=npconv.f32_to_e4m3_u8(extra),
        e4m3_decode_lut=npconv.e4m3_u8_to_f32(np.arange(256, dtype=np.uint8)),
        bf16_trunc_in=(x := rng.standard_normal(4096).astype(np.float32)),
        bf16_trunc_out=npconv.f32_to_bf16_u16(x),
    )

    # ---- RoPE tables
    rope = {}
    for H, W, ft in [(16, 8, 16), (8, 16, 129), (32, 16, 128), (4, 4, 1000), (8, 8, 0), (8, 8, 3)]:
        c, s = _make_ortho_rope_freqs(H, W, ft + 1, 64)
        tpf = H * W
        rope[f"cos_{H}_{W}_{ft}"] = c[ft * tpf : (ft + 1) * tpf]
        rope[f"sin_{H}_{W}_{ft}"] = s[ft * tpf : (ft + 1) * tpf]
    np.savez_compressed(HERE / "rope.npz", **rope)

    # ---- segment tables
    rows = []
    for nb, tpf, pd in [(16, 128, 1), (16, 128, 8), (16, 512, 8), (4, 64, 1), (4, 64, 2), (2, 512, 8)]:
        for ft in list(range(0, 3 * nb * pd + 3)) + [1000, 1001, 1024]:
            segs, n = _compute_segments(ft, nb, tpf, pd, nb * tpf, 3)
            rows.append([nb, tpf, pd, ft, n, *segs.reshape(-1).tolist()])
    np.savez_compressed(HERE / "segments.npz", table=np.array(rows, dtype=np.int64))

    # ---- kv_cache_update (the reference's smoke geometry: Hk=2, 8x8 grid, 4 buckets)
    kv = {}
    Hq, Hk, H, W, nb = 4, 2, 8, 8, 4
    qkv = _bf16(rng.standard_normal((H * W, (Hq + 2 * Hk) * 64)))
    kv["qkv"] = qkv
    cases = []
    for kv_dt in ("bf16", "e4m3"):
        for pd, ft, frozen in [(1, 0, 0), (1, 3, 0), (1, 4, 0), (1, 9, 1), (2, 8, 0), (2, 9, 0), (2, 16, 1)]:
            spec = KVCacheUpdateSpec(
                B=1, n_kv_heads=Hk, Dh=64, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd,
                in_dtype="bf16", kv_dtype=kv_dt, packed_qkv=True, n_q_heads=Hq,
            )
            out = kv_cache_update_reference_numpy(
                spec, K=qkv, V=qkv, frame_t=np.array([ft], dtype=np.int32), frozen=np.array([frozen], dtype=np.int32)
            )
            tag = f"{kv_dt}_{pd}_{ft}_{frozen}"
            cases.append(tag)
            for k, v in out.items():
                kv[f"{tag}.{k}"] = v
    kv["cases"] = np.array(cases)
    kv["geometry"] = np.array([Hq, Hk, H, W, nb], dtype=np.int64)
    np.savez_compressed(HERE / "kv_cache_update.npz", **kv)

    # ---- owl_attn
    at = {}
    Hk, gqa, H, W, nb = 2, 2, 8, 8, 4
    Hq = Hk * gqa
    tpf = H * W
    cap = nb * tpf + tpf
    qkv = _bf16(rng.standard_normal((tpf, (Hq + 2 * Hk) * 64)))
    at["qkv"] = qkv
    cases = []
    for kv_dt in ("bf16", "e4m3"):
        kf = rng.standard_normal((Hk * cap, 64)).astype(np.float32)
        vf = rng.standard_normal((Hk * 64, cap)).astype(np.float32)
        if kv_dt == "bf16":
            Kc, Vc = _bf16(kf), _bf16(vf)
        else:
            Kc, Vc = npconv.f32_to_e4m3_u8(kf), npconv.f32_to_e4m3_u8(vf)
        at[f"K_{kv_dt}"] = Kc
        at[f"Vt_{kv_dt}"] = Vc
        for pd, ft in [(1, 2), (1, 4), (1, 6), (2, 8), (2, 9), (1, 0)]:
            segs, n = _compute_segments(ft, nb, tpf, pd, nb * tpf, 3)
            spec = OwlAttnSpec(
                B=1, n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, num_buckets=nb, pinned_dilation=pd,
                Dh=64, a_dtype="bf16", kv_dtype=kv_dt, out_dtype="bf16", packed_qkv=True,
            )
            out = owl_attn_reference_numpy(
                spec, Q=qkv, K_cache=Kc, Vt_cache=Vc, segments=segs.reshape(-1).astype(np.int32),
                n_segments=np.array([n], dtype=np.int32), frame_t=np.array([ft], dtype=np.int32),
            )
            tag = f"{kv_dt}_{pd}_{ft}"
            cases.append(tag)
            at[f"{tag}.out"] = out
            at[f"{tag}.segments"] = segs.reshape(-1).astype(np.int32)
            at[f"{tag}.n_segments"] = np.array([n], dtype=np.int32)
    at["cases"] = np.array(cases)
    at["geometry"] = np.array([Hk, gqa, H, W, nb], dtype=np.int64)
    np.savez_compressed(HERE / "owl_attn.npz", **at)

    # ---- GEMM with every epilogue
    gm = {}
    M, N, K = 64, 128, 256
    A = _bf16(rng.standard_normal((M, K)))
    Bw = _bf16(0.02 * rng.standard_normal((N, K)))
    Bq = npconv.f32_to_e4m3_u8(0.5 * rng.standard_normal((N, K)).astype(np.float32))
    bias = _bf16(rng.standard_normal(N))
    gate = _bf16(rng.standard_normal((4, N)))
    resid = _bf16(rng.standard_normal((M, N)))
    gm.update(A=A, B=Bw, Bq=Bq, bias=bias, gate=gate, resid=resid)
    gm["plain"] = gemm_reference_numpy(GemmSpec(M=M, N=N, K=K), A=A, B=Bw)
    gm["bias_silu"] = gemm_reference_numpy(GemmSpec(M=M, N=N, K=K, activation="silu", has_bias=True), A=A, B=Bw, Bias=bias)
    gm["gate1"] = gemm_reference_numpy(GemmSpec(M=M, N=N, K=K, has_gate_residual=True, G=1), A=A, B=Bw, Gate=gate[:1], Residual=resid)
    gm["gate4"] = gemm_reference_numpy(GemmSpec(M=M, N=N, K=K, has_gate_residual=True, G=4), A=A, B=Bw, Gate=gate, Residual=resid)
    gm["fp8w"] = gemm_reference_numpy(GemmSpec(M=M, N=N, K=K, b_dtype="e4m3", compute_dtype="e4m3"), A=A, B=Bq)
    np.savez_compressed(HERE / "gemm.npz", **gm)

    # ---- norm / elementwise glue
    gl = {}
    M, D = 32, 256
    X = _bf16(rng.standard_normal((M, D)))
    Y = _bf16(rng.standard_normal((M, D)))
    sc = _bf16(0.1 * rng.standard_normal((1, D)))
    bi = _bf16(0.1 * rng.standard_normal((1, D)))
    gl.update(X=X, Y=Y, scale=sc, bias=bi)
    gl["ada_rmsnorm"] = ada_rmsnorm_reference_numpy(AdaRMSNormSpec(G=1, M=M, D=D, eps=1e-6), X=X, scale=sc, bias=bi)
    # the SiLU variant of ada_rmsnorm has no numpy reference upstream (the kernel applies
    # SiLU after the affine step, ada_rmsnorm/kernel.py:239-251); it is pinned by composition
    gl["silu"] = silu_reference_numpy(SiLUSpec(N=M * D), X=X.reshape(-1))
    gl["ada_gate_residual"] = ada_gate_residual_reference_numpy(AdaGateResidualSpec(G=1, M=M, D=D), X=X, Y=Y, gate=sc)
    Hq, Hk = 2, 1
    QKV = _bf16(rng.standard_normal((M, (Hq + 2 * Hk) * 64)))
    QKV0 = _bf16(rng.standard_normal((M, (Hq + 2 * Hk) * 64)))
    gl.update(QKV=QKV, QKV0=QKV0)
    gl["head_rmsnorm"] = head_rmsnorm_reference_numpy(
        HeadRMSNormSpec(M=M, D_full=QKV.shape[1], n_q_heads=Hq, n_kv_heads=Hk, Dh=64, eps=1e-6), X=QKV
    )
    gl["value_residual_packed"] = value_residual_packed_reference_numpy(
        ValueResidualPackedSpec(M=M, D_full=QKV.shape[1], v_col_offset=(Hq + Hk) * 64, v_width=Hk * 64),
        QKV_curr=QKV, QKV_first=QKV0, lamb=np.array([0.37], dtype=np.float32),
    )
    C, Hh, Ww, d = 4, 8, 12, 64
    lat = _bf16(rng.standard_normal((1, C * Hh * Ww)))
    Wp_ = _bf16(0.1 * rng.standard_normal((d, C * 4)))
    Wu = _bf16(0.1 * rng.standard_normal((C * 4, d)))
    bu = _bf16(0.1 * rng.standard_normal(C * 4))
    tok = _bf16(rng.standard_normal(((Hh // 2) * (Ww // 2), d)))
    gl.update(lat=lat, Wp=Wp_, Wu=Wu, bu=bu, tok=tok)
    gl["patchify"] = patchify_reference_numpy(PatchifySpec(B=1, C=C, H=Hh, W=Ww, d_model=d), X=lat, W=Wp_)
    gl["unpatchify"] = unpatchify_reference_numpy(UnpatchifySpec(B=1, C=C, H=Hh, W=Ww, d_model=d), X=tok, W=Wu, Bias=bu)
    np.savez_compressed(HERE / "glue.npz", **gl)

    # ---- conditioning tables (host-side numpy upstream too), small d
    d, fd = 64, 16
    sig = (1.0, 0.9, 0.75, 0.3, 0.0)
    w1 = _bf16(0.2 * rng.standard_normal((4 * d, fd)))
    w2 = _bf16(0.2 * rng.standard_normal((d, 4 * d)))
    ab = _bf16(0.2 * rng.standard_normal(d))
    mb = _bf16(0.2 * rng.standard_normal(d))
    pw = [_bf16(0.2 * rng.standard_normal((d, d))) for _ in range(6)]
    onw = _bf16(0.2 * rng.standard_normal((2 * d, d)))
    P = lambda a: types.SimpleNamespace(data=a)  # noqa: E731
    blk = types.SimpleNamespace(
        attn_cond_bias_in=P(ab), mlp_cond_bias_in=P(mb), cond_projs=[types.SimpleNamespace(weight=P(w)) for w in pw]
    )
    model = types.SimpleNamespace(
        noise_fc1=types.SimpleNamespace(weight=P(w1)), noise_fc2=types.SimpleNamespace(weight=P(w2)),
        out_norm_proj=types.SimpleNamespace(weight=P(onw)), blocks=[blk],
    )
    cfg = types.SimpleNamespace(fourier_dim=fd, scheduler_sigmas=sig)
    wio._IS_METAL = True  # keep the tables on the host as tagged numpy carriers
    import quark.runtime.sync as qsync

    qsync.synchronize = lambda: None
    wio.compute_noise_emb_numpy(model, cfg)
    wio.prepare_cond_luts(model, cfg, d)
    cd = dict(w1=w1, w2=w2, attn_bias=ab, mlp_bias=mb, on_w=onw, sigmas=np.array(sig), fourier_dim=np.array(fd))
    for j, w in enumerate(pw):
        cd[f"proj{j}"] = w
    cd["noise_emb"] = np.stack(model._noise_emb_np)
    for si in range(len(sig)):
        for j in range(6):
            cd[f"lut_{si}_{j}"] = np.asarray(blk._cond_lut[si][j]).view(np.uint16)
        cd[f"on_{si}_0"] = np.asarray(model._out_norm_luts[si][0]).view(np.uint16)
        cd[f"on_{si}_1"] = np.asarray(model._out_norm_luts[si][1]).view(np.uint16)
    np.savez_compressed(HERE / "cond.npz", **cd)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
