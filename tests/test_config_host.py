"""``Waypoint15Config`` / ``QuantConfig`` on the host: what is accepted, what is refused and why."""

import pytest

from quark_b200.models import QuantConfig, Waypoint15Config

SMALL = dict(d_model=128, n_layers=4, n_heads=2, n_kv_heads=1, height=16, width=8, channels=4, local_window=2, global_window=4,
             global_pinned_dilation=2)  # fmt: skip


def test_quant_config_takes_every_mix():
    for lin in ("fp8", "bf16"):
        for kv in ("fp8", "bf16"):
            for attn in ("fp8", "bf16"):
                q = QuantConfig(linear=lin, kv_cache=kv, attn_compute=attn, moe=lin)
                assert (q.linear, q.kv_cache, q.attn_compute) == (lin, kv, attn)
    with pytest.raises(ValueError, match="kv_cache"):
        QuantConfig(kv_cache="fp4")
    assert QuantConfig.all_bf16().moe == "bf16" and QuantConfig.all_fp8().linear == "fp8"


def test_quilt_and_layer_geometry():
    c = Waypoint15Config(**SMALL, quilt_factor=4)
    assert c.tpf == 128 and c.quilt_factor == 4
    for bad in (3, 0, 256):  # not a power of two, not positive, does not divide 128 tokens
        with pytest.raises(ValueError, match="quilt_factor"):
            Waypoint15Config(**SMALL, quilt_factor=bad)
    # layers 3, 7, ... are the global ones (offset -1, period 4): fewer, dilated buckets
    assert [c.is_global(i) for i in range(4)] == [False, False, False, True]
    assert (c.num_buckets(0), c.pinned_dilation(0), c.num_buckets(3), c.pinned_dilation(3)) == (2, 1, 2, 2)


def test_mixture_of_experts_configuration():
    c = Waypoint15Config(**SMALL, moe=True)
    assert (c.moe_n_experts, c.moe_top_k, c.moe_routing, c.mlp_dim // c.moe_top_k) == (8, 2, "correct", 256)
    with pytest.raises(NotImplementedError, match="balanced"):
        Waypoint15Config(**SMALL, moe=True, moe_routing="balanced")
    with pytest.raises(ValueError, match="experts"):
        Waypoint15Config(**SMALL, moe=True, moe_n_experts=4)  # the router GEMM wants a multiple of 8 columns
    with pytest.raises(ValueError, match="experts"):
        Waypoint15Config(**SMALL, moe=True, moe_top_k=9)
    with pytest.raises(NotImplementedError, match="tp_world"):
        Waypoint15Config(**{**SMALL, "n_kv_heads": 2}, moe=True, tp_world=2)
    raw = dict(SMALL, moe=True, moe_n_experts=16, moe_top_k=4, moe_routing="correct", quilt_factor=2, patch=[2, 2], ctrl_conditioning=None)
    c = Waypoint15Config.from_dict(raw)
    assert (c.moe, c.moe_n_experts, c.moe_top_k, c.quilt_factor, c.ctrl_conditioning) == (True, 16, 4, 2, False)


def test_other_refusals():
    with pytest.raises(NotImplementedError, match="head_dim"):
        Waypoint15Config(**{**SMALL, "n_heads": 4})
    with pytest.raises(ValueError, match="tp_rank"):
        Waypoint15Config(**SMALL, tp_world=1, tp_rank=1)
    with pytest.raises(ValueError, match="do not divide"):
        Waypoint15Config(**SMALL, tp_world=2)
