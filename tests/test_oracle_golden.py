"""The CPU oracle against the fixtures generated from the reference's own numpy oracles.

Every ``.npz`` in ``tests/golden`` holds seeded inputs and the outputs the reference produced
for them (``tests/golden/make_golden.py``).  Byte and index results must be identical; f32
chains whose summation order differs from the reference's are compared on the bf16 carrier
with at most one unit in the last place.
"""

from pathlib import Path

import numpy as np
import pytest

from oracle import codec, model, ops

G = Path(__file__).parent / "golden"


def load(name):
    return np.load(G / name, allow_pickle=False)


def assert_bf16_close(got_u16, want_u16, max_ulp=1, frac_exact=0.98):
    g = got_u16.astype(np.int64).ravel()
    w = want_u16.astype(np.int64).ravel()
    # bf16 carriers are sign-magnitude; compare in value space for a sign flip near zero
    d = np.abs(g - w)
    bad = d > max_ulp
    if bad.any():
        gf, wf = codec.bf16_to_f32(got_u16).ravel(), codec.bf16_to_f32(want_u16).ravel()
        assert np.all(np.abs(gf[bad] - wf[bad]) <= 1e-6), f"{bad.sum()} elements differ by more than {max_ulp} ulp"
    assert np.mean(d == 0) >= frac_exact


def test_e4m3_encoder_matches_reference_on_every_bf16_value():
    z = load("codec.npz")
    x = codec.bf16_to_f32(np.arange(65536, dtype=np.uint16))
    np.testing.assert_array_equal(codec.f32_to_e4m3(x, reference_quirk=True), z["e4m3_of_all_bf16"])
    np.testing.assert_array_equal(codec.f32_to_e4m3(z["extra_f32"], reference_quirk=True), z["e4m3_of_extra"])
    # without the quirk the only difference is the band that should round up to the smallest normal
    mine = codec.f32_to_e4m3(x)
    diff = mine != z["e4m3_of_all_bf16"]
    ax = np.abs(x)
    assert np.array_equal(diff, (ax >= codec.QUIRK_LO) & (ax < codec.QUIRK_HI))
    assert diff.sum() == 32
    assert set(mine[diff] & 0x7F) == {0x08}


def test_e4m3_decode_and_bf16_truncation():
    z = load("codec.npz")
    got = codec.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    np.testing.assert_array_equal(np.isnan(got), np.isnan(z["e4m3_decode_lut"]))
    np.testing.assert_array_equal(got[~np.isnan(got)], z["e4m3_decode_lut"][~np.isnan(got)])
    np.testing.assert_array_equal(codec.f32_to_bf16(z["bf16_trunc_in"]), z["bf16_trunc_out"])
    # encode(decode(b)) == b for every finite byte
    b = np.arange(256, dtype=np.uint8)
    fin = ~np.isnan(got)
    np.testing.assert_array_equal(codec.f32_to_e4m3(got[fin]), b[fin])


def test_rope_tables_bit_exact():
    z = load("rope.npz")
    for key in z.files:
        if not key.startswith("cos_"):
            continue
        H, W, ft = (int(v) for v in key.split("_")[1:])
        c, s = ops.rope_tables(H, W, ft)
        np.testing.assert_array_equal(c, z[key])
        np.testing.assert_array_equal(s, z["sin_" + key[4:]])


def test_segment_tables():
    for nb, tpf, pd, ft, n, *segs in load("segments.npz")["table"].tolist():
        got, gn = ops.compute_segments(ft, nb, tpf, pd)
        assert gn == n and got.tolist() == segs, (nb, tpf, pd, ft)


def test_kv_cache_update_bit_exact():
    z = load("kv_cache_update.npz")
    Hq, Hk, H, W, nb = (int(v) for v in z["geometry"])
    for tag in z["cases"].tolist():
        kv_dt, pd, ft, frozen = tag.split("_")
        K, Vt, segs, n = ops.kv_cache_update(
            z["qkv"], int(ft), int(frozen), n_kv_heads=Hk, n_q_heads=Hq, H_spatial=H, W_spatial=W,
            num_buckets=nb, pinned_dilation=int(pd), kv_dtype=kv_dt, reference_quirk=True,
        )
        np.testing.assert_array_equal(K, z[f"{tag}.K_cache"], err_msg=tag)
        np.testing.assert_array_equal(Vt, z[f"{tag}.Vt_cache"], err_msg=tag)
        np.testing.assert_array_equal(segs, z[f"{tag}.segments"], err_msg=tag)
        np.testing.assert_array_equal(n, z[f"{tag}.n_segments"], err_msg=tag)


def test_kv_cache_update_in_place_keeps_other_rows():
    z = load("kv_cache_update.npz")
    Hq, Hk, H, W, nb = (int(v) for v in z["geometry"])
    tpf, cap = H * W, (nb + 1) * H * W
    K0 = np.full((Hk * cap, 64), 0x1234, dtype=np.uint16)
    V0 = np.full((Hk * 64, cap), 0x4321, dtype=np.uint16)
    K, Vt, _, _ = ops.kv_cache_update(
        z["qkv"], 3, 0, n_kv_heads=Hk, n_q_heads=Hq, H_spatial=H, W_spatial=W, num_buckets=nb,
        pinned_dilation=1, K_cache=K0, Vt_cache=V0,
    )
    fresh = z["bf16_1_3_0.K_cache"].reshape(Hk, cap, 64)
    Kr = K.reshape(Hk, cap, 64)
    written = np.zeros(cap, dtype=bool)
    written[3 * tpf : 4 * tpf] = True
    written[nb * tpf :] = True
    np.testing.assert_array_equal(Kr[:, written], fresh[:, written])
    assert np.all(Kr[:, ~written] == 0x1234)
    assert np.all(Vt.reshape(Hk, 64, cap)[:, :, ~written] == 0x4321)


def test_owl_attn():
    z = load("owl_attn.npz")
    Hk, gqa, H, W, nb = (int(v) for v in z["geometry"])
    for tag in z["cases"].tolist():
        kv_dt, pd, ft = tag.split("_")
        out = ops.owl_attn(
            z["qkv"], z[f"K_{kv_dt}"], z[f"Vt_{kv_dt}"], z[f"{tag}.segments"], z[f"{tag}.n_segments"], int(ft),
            n_kv_heads=Hk, gqa_ratio=gqa, H_spatial=H, W_spatial=W, kv_dtype=kv_dt,
        )
        assert_bf16_close(out, z[f"{tag}.out"])


def test_gemm_epilogues():
    z = load("gemm.npz")
    A, B = z["A"], z["B"]
    assert_bf16_close(ops.gemm(A, B), z["plain"])
    assert_bf16_close(ops.gemm(A, B, bias=z["bias"], activation="silu"), z["bias_silu"])
    assert_bf16_close(ops.gemm(A, B, gate=z["gate"][:1], residual=z["resid"]), z["gate1"])
    assert_bf16_close(ops.gemm(A, B, gate=z["gate"], residual=z["resid"], gate_groups=4), z["gate4"])
    assert_bf16_close(ops.gemm(A, z["Bq"], b_dtype="e4m3"), z["fp8w"])


def test_glue_ops():
    z = load("glue.npz")
    np.testing.assert_array_equal(ops.ada_rmsnorm(z["X"], z["scale"], z["bias"]), z["ada_rmsnorm"])
    np.testing.assert_array_equal(ops.silu(z["X"]).ravel(), z["silu"].ravel())
    np.testing.assert_array_equal(ops.ada_gate_residual(z["X"], z["Y"], z["scale"]), z["ada_gate_residual"])
    np.testing.assert_array_equal(ops.head_rmsnorm(z["QKV"], n_q_heads=2, n_kv_heads=1), z["head_rmsnorm"])
    np.testing.assert_array_equal(
        ops.value_residual_packed(z["QKV"], z["QKV0"], 0.37, v_col_offset=192, v_width=64), z["value_residual_packed"]
    )
    assert_bf16_close(ops.patchify(z["lat"], z["Wp"], C=4, H=8, Wd=12), z["patchify"])
    assert_bf16_close(ops.unpatchify(z["tok"], z["Wu"], z["bu"], C=4, H=8, Wd=12), z["unpatchify"])
    # SiLU variant of ada_rmsnorm == silu applied to the unrounded affine result
    y = ops.ada_rmsnorm(z["X"], z["scale"], z["bias"], return_f32=True)
    np.testing.assert_array_equal(
        ops.ada_rmsnorm(z["X"], z["scale"], z["bias"], activation="silu"), codec.f32_to_bf16(ops.silu_f32(y))
    )


def test_conditioning_tables():
    z = load("cond.npz")
    f = codec.bf16_to_f32
    sig = z["sigmas"].tolist()
    emb = model.noise_embedding(sig, int(z["fourier_dim"]), f(z["w1"]), f(z["w2"]))
    np.testing.assert_allclose(emb, z["noise_emb"], rtol=0, atol=0)
    projs = [f(z[f"proj{j}"]) for j in range(6)]
    for si in range(len(sig)):
        rows = model.cond_rows(emb[si], f(z["attn_bias"]), f(z["mlp_bias"]), projs)
        for j in range(6):
            np.testing.assert_array_equal(rows[j].ravel(), z[f"lut_{si}_{j}"].ravel())
        on = model.out_norm_rows(emb[si], f(z["on_w"]))
        np.testing.assert_array_equal(on[0].ravel(), z[f"on_{si}_0"].ravel())
        np.testing.assert_array_equal(on[1].ravel(), z[f"on_{si}_1"].ravel())


@pytest.mark.parametrize("H,W", [(16, 8), (8, 16)])
def test_rope_orientation_matters(H, W):
    # token -> (h, w) = (idx // W, idx % W): swapping H and W changes the table
    c1, _ = ops.rope_tables(H, W, 5)
    c2, _ = ops.rope_tables(W, H, 5)
    assert not np.array_equal(c1, c2)


def test_controller_conditioning_ops():
    """Plain RMSNorm, elementwise add, MLPFusion and the controller embedding against the reference's numpy
    oracles composed in the order its modules launch them (``tests/golden/make_golden_ctrl.py``)."""
    z = load("ctrl.npz")
    np.testing.assert_array_equal(ops.rmsnorm(z["X"]), z["rmsnorm"])
    np.testing.assert_array_equal(ops.rmsnorm(z["cond"]), z["rmsnorm_row"])
    np.testing.assert_array_equal(ops.add(z["X"], z["Y"]), z["add"])
    assert_bf16_close(ops.mlp_fusion(z["X"], z["cond"], z["Wx"], z["Wc"], z["W2"]), z["mlp_fusion"])
    assert_bf16_close(ops.controller_embedding(z["ctrl_input"], z["We1"], z["We2"]), z["ctrl_emb"])


def test_mixture_of_experts_against_the_reference_oracles():
    """``ops.moe_route`` / ``ops.moe`` (dense form) against the reference's router, in-projection, out-projection and
    reduction references chained as ``nn.MoE`` launches them with routing "correct" (``tests/golden/make_golden_moe.py``):
    the same experts for every token, the same weights, and the same output up to the order of the f32 sums.

    One difference is deliberate.  Where a token's k-th and (k+1)-th logits are equal (bf16 logits: it happens), the
    reference's numpy oracle takes whichever numpy's unstable ``argsort`` puts first, while its kernel inserts with a
    strict ``>`` and so keeps the lower expert index (``src/quark/kernels/_moe_router_dsl.py:32-66``).  The oracle here
    follows the kernel; such tokens are compared for their weights' values only."""
    z = load("moe.npz")
    M, D, H, E, K = (int(v) for v in z["geometry"])
    logits = ops.gemm(z["X"], z["Wr"])
    np.testing.assert_array_equal(logits, z["logits"])
    w = ops.moe_route(z["logits"], K)
    assert w.shape == (E, M)
    srt = -np.sort(-codec.bf16_to_f32(z["logits"]), axis=1)
    tie = srt[:, K - 1] == srt[:, K]
    assert 0 < tie.sum() < M // 8  # the fixture has such tokens, and few
    np.testing.assert_array_equal((w != 0)[:, ~tie], (z["weights"] != 0)[:, ~tie])
    np.testing.assert_allclose(w[:, ~tie], z["weights"][:, ~tie], rtol=0, atol=1e-7)
    np.testing.assert_allclose(np.sort(w[:, tie], axis=0), np.sort(z["weights"][:, tie], axis=0), rtol=0, atol=1e-7)
    for m in np.flatnonzero(tie):  # ties towards the lower index
        mine, theirs = np.flatnonzero(w[:, m]), np.flatnonzero(z["weights"][:, m])
        assert mine.sum() <= theirs.sum()
    got = ops.moe(z["X"], z["Wr"], z["W_in"], z["W_out"], top_k=K)
    assert_bf16_close(got[~tie], z["out"][~tie])


def test_moe_slot_tables_match_the_reference_router():
    """``ops.moe_route_slots`` at the reference's row tile (32) against the slot tables its own numpy router wrote
    (``src/quark/kernels/moe_router_correct/reference.py:51-108``; ``tests/golden/make_golden_moe.py``): counts, offsets,
    the slot of every (token, k), the token and weight in every slot, the expert of every 32-row chunk - all exact.
    The fixture has one token with two equal logits, which the reference's unstable sort gives to the higher expert
    index and this oracle (like the reference's kernel) to the lower: the choice of experts is compared first, tie
    aside, and the layout is then derived from the reference's choice."""
    z = load("moe.npz")
    M, D, H, E, K = (int(v) for v in z["geometry"])
    cap = int(z["capacity"][0])
    ref_order = np.searchsorted(z["slot_offsets"][1:], z["token_slot_table"], side="right")  # expert of every (token, k)
    own = ops.moe_route_slots(z["logits"], K, tile=32, total_slots=E * cap)
    own_order = np.searchsorted(own["offsets"][1:], own["token_slot"], side="right")
    differ = np.flatnonzero((own_order != ref_order).any(axis=1))
    assert len(differ) <= 1
    for m in differ:  # a tie: the same logit value at both experts
        lg = z["logits"][m]
        assert sorted(lg[own_order[m]].tolist()) == sorted(lg[ref_order[m]].tolist())
    r = ops.moe_route_slots(z["logits"], K, tile=32, total_slots=E * cap, order=ref_order)
    np.testing.assert_array_equal(r["counts"], z["counts"])
    np.testing.assert_array_equal(r["offsets"], z["slot_offsets"])
    np.testing.assert_array_equal(r["token_slot"], z["token_slot_table"])
    np.testing.assert_array_equal(r["tile_expert"], z["work_list"][1::2])
    np.testing.assert_array_equal(z["work_list"][0::2], 32 * np.arange(E * cap // 32))
    used = r["slot_token"] >= 0
    np.testing.assert_array_equal(r["slot_token"][used], z["slot_token_ids"][used])
    assert not z["slot_token_ids"][~used].any() and not z["slot_weights"][~used].any()  # the reference pads with zeros
    np.testing.assert_allclose(r["slot_weight"], z["slot_weights"], atol=1e-6)
