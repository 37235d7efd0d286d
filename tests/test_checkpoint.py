"""Checkpoint ingestion on the host: the safetensors container, the key remap, the conditioning tables.

The expected parameters are computed here a second time, straight from the synthetic upstream tensors with the
arithmetic of the reference's loader (``src/quark/models/_waypoint_15_io.py:70-217`` for the remap and ``:385-478``
for the tables), not through the module under test.
"""

import json
import math
import struct

import numpy as np
import pytest

from quark_b200.models import _cond
from quark_b200.models import checkpoint as ck


def tiny_cfg(**kw):
    from quark_b200.models import Waypoint15Config

    base = dict(d_model=128, n_layers=4, n_heads=2, n_kv_heads=1, height=8, width=8, channels=4, local_window=2, global_window=4,
                global_pinned_dilation=2, fourier_dim=32, ctrl_conditioning=True, n_buttons=20)  # fmt: skip
    base.update(kw)
    return Waypoint15Config(**base)


def synth_upstream(cfg, seed=0, std=0.08):
    """An upstream-format state dict ``{name: (tag, array)}`` that exercises every branch of the remap: 4-D patch
    weights, per-channel bias, a shared cond head (block 1) and separate ones, both MLP prefixes, a 0-d and a 1-d
    ``v_lamb`` and a block without one, both controller layouts, f32 and bf16 storage."""
    r = np.random.default_rng([seed, 99])
    d, C, (ph, pw) = cfg.d_model, cfg.channels, cfg.patch

    def bf(*shape):
        return ("BF16", _cond._bf16(r.standard_normal(shape, dtype=np.float32) * np.float32(std)))

    def f4(*shape):
        return ("F32", r.standard_normal(shape, dtype=np.float32) * np.float32(std))

    sd = {
        "patchify.weight": bf(d, C, ph, pw),
        "unpatchify.weight": bf(d, C, ph, pw),
        "unpatchify.bias": bf(C),
        "denoise_step_emb.mlp.fc1.weight": f4(cfg.mlp_dim, cfg.fourier_dim),  # stored wide: narrowed on load
        "denoise_step_emb.mlp.fc2.weight": bf(d, cfg.mlp_dim),
        "out_norm.fc.weight": bf(2 * d, d),
        "unrelated.prompt_encoder.weight": bf(8, 8),  # keys outside the transformer are ignored
    }
    Dh = cfg.Dh
    for i in range(cfg.n_layers):
        p = f"transformer.blocks.{i}."
        if i == 1:
            sd[p + "cond_head.bias_in"] = bf(d)
            for j in range(6):
                sd[p + f"cond_head.cond_proj.{j}.weight"] = bf(d, d)
        else:
            sd[p + "attn_cond_head.bias_in"] = bf(d)
            sd[p + "mlp_cond_head.bias_in"] = f4(d)
            for j in range(3):
                sd[p + f"attn_cond_head.cond_proj.{j}.weight"] = bf(d, d)
                sd[p + f"mlp_cond_head.cond_proj.{j}.weight"] = bf(d, d)
        sd[p + "attn.q_proj.weight"] = bf(cfg.n_heads * Dh, d)
        sd[p + "attn.k_proj.weight"] = bf(cfg.n_kv_heads * Dh, d)
        sd[p + "attn.v_proj.weight"] = bf(cfg.n_kv_heads * Dh, d)
        sd[p + "attn.out_proj.weight"] = bf(d, cfg.n_heads * Dh)
        pre = "mlp." if i % 2 == 0 else "dit_mlp."
        sd[p + pre + "fc1.weight"] = bf(cfg.mlp_dim, d)
        sd[p + pre + "fc2.weight"] = bf(d, cfg.mlp_dim)
        if i == 0:
            sd[p + "attn.v_lamb"] = ("F32", np.asarray(0.625, np.float32))
        elif i == 1:
            sd[p + "attn.v_lamb"] = ("BF16", _cond._bf16(np.asarray([0.25], np.float32)))
        if cfg.has_ctrl(i):
            if i == 0:
                sd[p + "ctrl_mlpfusion.mlp.fc1.weight"] = bf(d, 2 * d)
                sd[p + "ctrl_mlpfusion.mlp.fc2.weight"] = bf(d, d)
            else:
                for k in ("fc1_x", "fc1_c", "fc2"):
                    sd[p + f"ctrl_mlpfusion.{k}.weight"] = bf(d, d)
    if cfg.ctrl_conditioning:
        sd["ctrl_emb.mlp.fc1.weight"] = bf(cfg.mlp_dim, cfg.n_buttons + 3)
        sd["ctrl_emb.mlp.fc2.weight"] = bf(d, cfg.mlp_dim)
    return sd


def write_model_dir(cfg, path, seed=0, extra_yaml=""):
    """``config.yaml`` + ``model.safetensors`` of a synthetic upstream checkpoint under ``path``; returns the state dict."""
    sd = synth_upstream(cfg, seed)
    ck.write_safetensors(path / "model.safetensors", sd)
    lines = [f"{k}: {getattr(cfg, k)}" for k in ("d_model", "n_layers", "n_heads", "n_kv_heads", "mlp_ratio", "channels", "height", "width",
                                                "local_window", "global_window", "global_pinned_dilation", "global_attn_period",
                                                "global_attn_offset", "fourier_dim", "n_buttons", "ctrl_conditioning_period")]  # fmt: skip
    lines += [f"patch: [{cfg.patch[0]}, {cfg.patch[1]}]", "scheduler_sigmas: [" + ", ".join(str(s) for s in cfg.scheduler_sigmas) + "]",
              "value_residual: true", "base_fps: 60", "ae_uri: some/autoencoder"]  # fmt: skip
    if cfg.ctrl_conditioning:
        lines.append("ctrl_conditioning:\n  kind: mouse_keyboard")
    (path / "config.yaml").write_text("\n".join(lines) + "\n" + extra_yaml)
    return sd


def w32(entry):
    """What the model holds of a stored tensor: its bf16 narrowing (by truncation), widened again."""
    tag, a = entry
    u = a if tag == "BF16" else (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)
    return (u.astype(np.uint32) << 16).view(np.float32), u


def silu(x):
    return x * (1.0 / (1.0 + np.exp(-x)))


def expected_noise_emb(cfg, sd):
    half = cfg.fourier_dim // 2
    freqs = np.array([10000.0 ** (-i / max(half - 1, 1)) for i in range(half)], np.float32)
    feats = np.zeros((len(cfg.scheduler_sigmas), 2 * half), np.float32)
    for i, s in enumerate(cfg.scheduler_sigmas):
        ph = np.array([float(s) * 1000.0 * f for f in freqs], np.float32)
        feats[i, :half], feats[i, half:] = math.sqrt(2.0) * np.sin(ph), math.sqrt(2.0) * np.cos(ph)
    h = feats @ w32(sd["denoise_step_emb.mlp.fc1.weight"])[0].T
    return silu(h) @ w32(sd["denoise_step_emb.mlp.fc2.weight"])[0].T


def trunc_bf16(a):
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def test_container_round_trip_and_independent_writer(tmp_path):
    """Our reader against files written by the ``safetensors`` package, our writer against its reader."""
    st = pytest.importorskip("safetensors.torch")
    import torch

    g = torch.Generator().manual_seed(5)
    tensors = {"a.weight": torch.randn(7, 12, generator=g).to(torch.bfloat16), "b": torch.randn(3, generator=g),
               "scalar": torch.tensor(0.375), "idx": torch.arange(5, dtype=torch.int64)}  # fmt: skip
    st.save_file(tensors, str(tmp_path / "theirs.safetensors"), metadata={"format": "pt"})
    got = ck.read_safetensors(tmp_path / "theirs.safetensors")
    assert sorted(got) == sorted(tensors)
    assert got["a.weight"][0] == "BF16" and got["a.weight"][1].shape == (7, 12)
    np.testing.assert_array_equal(got["a.weight"][1], tensors["a.weight"].view(torch.uint16).numpy())
    np.testing.assert_array_equal(got["b"][1], tensors["b"].numpy())
    assert got["scalar"][1].shape == () and float(got["scalar"][1]) == 0.375
    np.testing.assert_array_equal(got["idx"][1], np.arange(5))

    ck.write_safetensors(tmp_path / "ours.safetensors", got)
    back = st.load_file(str(tmp_path / "ours.safetensors"))
    for k, t in tensors.items():
        assert back[k].dtype == t.dtype and torch.equal(back[k], t), k


def test_container_rejects_damaged_files(tmp_path):
    (tmp_path / "short").write_bytes(b"\x01\x02")
    with pytest.raises(ValueError, match="not a safetensors"):
        ck.read_safetensors(tmp_path / "short")
    (tmp_path / "long_header").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ValueError, match="does not fit"):
        ck.read_safetensors(tmp_path / "long_header")
    h = json.dumps({"x": {"dtype": "F8_E5M2", "shape": [1], "data_offsets": [0, 1]}}).encode()
    (tmp_path / "odd_dtype").write_bytes(struct.pack("<Q", len(h)) + h + b"\0")
    with pytest.raises(NotImplementedError, match="F8_E5M2"):
        ck.read_safetensors(tmp_path / "odd_dtype")


def test_remap_matches_a_second_derivation(tmp_path):
    cfg = tiny_cfg()
    sd = write_model_dir(cfg, tmp_path)
    params = ck.load_checkpoint(tmp_path, cfg)
    d, C, (ph, pw) = cfg.d_model, cfg.channels, cfg.patch
    kp = C * ph * pw

    np.testing.assert_array_equal(params["patchify.weight"], sd["patchify.weight"][1].reshape(d, kp))
    # unpatchify: out[c, y, x, :] = w[:, c, y, x]
    uw = sd["unpatchify.weight"][1]
    want = np.empty((kp, d), np.uint16)
    for c in range(C):
        for y in range(ph):
            for x in range(pw):
                want[(c * ph + y) * pw + x] = uw[:, c, y, x]
    np.testing.assert_array_equal(params["unpatchify.weight"], want)
    ub = sd["unpatchify.bias"][1]
    np.testing.assert_array_equal(params["unpatchify.bias"], np.array([ub[c] for c in range(C) for _ in range(ph * pw)], np.uint16))

    emb = expected_noise_emb(cfg, sd)
    on = w32(sd["out_norm.fc.weight"])[0]
    for si in range(len(cfg.scheduler_sigmas)):
        ab = silu(emb[si]) @ on.T
        np.testing.assert_array_equal(params["out_norm.lut"][si][0], trunc_bf16(ab[:d]).reshape(1, d))
        np.testing.assert_array_equal(params["out_norm.lut"][si][1], trunc_bf16(ab[d:]).reshape(1, d))

    assert len(params["blocks"]) == cfg.n_layers
    for i, blk in enumerate(params["blocks"]):
        p = f"transformer.blocks.{i}."
        q, k, v = (sd[p + f"attn.{n}_proj.weight"][1] for n in "qkv")
        assert blk["qkv.weight"].shape == (cfg.qkv_dim, d)
        np.testing.assert_array_equal(blk["qkv.weight"][: q.shape[0]], q)
        np.testing.assert_array_equal(blk["qkv.weight"][q.shape[0] : q.shape[0] + k.shape[0]], k)
        np.testing.assert_array_equal(blk["qkv.weight"][q.shape[0] + k.shape[0] :], v)
        np.testing.assert_array_equal(blk["out.weight"], sd[p + "attn.out_proj.weight"][1])
        pre = "mlp." if i % 2 == 0 else "dit_mlp."
        np.testing.assert_array_equal(blk["fc1.weight"], sd[p + pre + "fc1.weight"][1])
        np.testing.assert_array_equal(blk["fc2.weight"], sd[p + pre + "fc2.weight"][1])
        assert blk["lamb"] == {0: 0.625, 1: 0.25}.get(i, 0.5)
        if i == 1:
            ab_ = mb_ = w32(sd[p + "cond_head.bias_in"])[0]
            pw_ = [w32(sd[p + f"cond_head.cond_proj.{j}.weight"])[0] for j in range(6)]
        else:
            ab_, mb_ = w32(sd[p + "attn_cond_head.bias_in"])[0], w32(sd[p + "mlp_cond_head.bias_in"])[0]
            pw_ = [w32(sd[p + f"attn_cond_head.cond_proj.{j}.weight"])[0] for j in range(3)]
            pw_ += [w32(sd[p + f"mlp_cond_head.cond_proj.{j}.weight"])[0] for j in range(3)]
        for si in range(len(cfg.scheduler_sigmas)):
            ha, hm = silu(emb[si] + ab_), silu(emb[si] + mb_)
            for j in range(6):
                row = (ha if j < 3 else hm) @ pw_[j].T
                np.testing.assert_array_equal(blk["lut"][si][j], trunc_bf16(row).reshape(1, d), err_msg=f"block {i} sigma {si} row {j}")
        assert ("ctrl.fc2.weight" in blk) == cfg.has_ctrl(i)
    b0, b3 = params["blocks"][0], params["blocks"][3]
    cat = sd["transformer.blocks.0.ctrl_mlpfusion.mlp.fc1.weight"][1]
    np.testing.assert_array_equal(b0["ctrl.fc1_x.weight"], cat[:, :d])
    np.testing.assert_array_equal(b0["ctrl.fc1_c.weight"], cat[:, d:])
    assert b0["ctrl.fc1_x.weight"].flags.c_contiguous and b0["ctrl.fc1_c.weight"].flags.c_contiguous
    np.testing.assert_array_equal(b0["ctrl.fc2.weight"], sd["transformer.blocks.0.ctrl_mlpfusion.mlp.fc2.weight"][1])
    for k in ("fc1_x", "fc1_c", "fc2"):
        np.testing.assert_array_equal(b3[f"ctrl.{k}.weight"], sd[f"transformer.blocks.3.ctrl_mlpfusion.{k}.weight"][1])
    w1 = sd["ctrl_emb.mlp.fc1.weight"][1]
    assert w1.shape[1] == 23 and params["ctrl_emb.fc1.weight"].shape == (cfg.mlp_dim, 32)
    np.testing.assert_array_equal(params["ctrl_emb.fc1.weight"][:, :23], w1)
    assert not params["ctrl_emb.fc1.weight"][:, 23:].any()
    np.testing.assert_array_equal(params["ctrl_emb.fc2.weight"], sd["ctrl_emb.mlp.fc2.weight"][1])


def test_loaded_params_have_the_layout_of_random_init(tmp_path):
    """Same keys, shapes and dtypes as ``make_params``, so the model's upload path is the one the GPU tests cover."""
    from quark_b200.models import make_params

    cfg = tiny_cfg()
    write_model_dir(cfg, tmp_path)
    got, ref = ck.load_checkpoint(tmp_path / "model.safetensors", cfg), make_params(cfg, seed=1)

    def same(a, b, where):
        if isinstance(b, dict):
            assert sorted(a) == sorted(b), where
            for k in b:
                same(a[k], b[k], f"{where}.{k}")
        elif isinstance(b, (list, tuple)):
            assert len(a) == len(b), where
            for n, (x, y) in enumerate(zip(a, b)):
                same(x, y, f"{where}[{n}]")
        elif isinstance(b, np.ndarray):
            assert a.shape == b.shape and a.dtype == b.dtype, f"{where}: {a.shape} {a.dtype} vs {b.shape} {b.dtype}"
        else:
            assert type(a) is type(b), where

    same(got, ref, "params")


def test_config_yaml_defaults_references_and_overrides(tmp_path):
    from quark_b200.models import Waypoint15Config

    cfg = tiny_cfg()
    write_model_dir(cfg, tmp_path)
    got = Waypoint15Config.from_yaml(tmp_path)
    for k in ("d_model", "n_layers", "n_heads", "n_kv_heads", "patch", "scheduler_sigmas", "n_buttons", "fourier_dim", "global_window"):
        assert getattr(got, k) == getattr(cfg, k), k
    assert got.ctrl_conditioning and got.value_residual
    raw = ck.load_yaml_config(tmp_path / "config.yaml")
    assert raw["inference_fps"] == 60 and raw["ae_uri"] == "some/autoencoder"  # ${base_fps} resolved; extras kept
    assert Waypoint15Config.from_yaml(tmp_path, n_layers=2).n_layers == 2

    # the training defaults: no n_kv_heads -> as many as n_heads; no ctrl_conditioning key -> the class default;
    # an explicit null -> off
    (tmp_path / "min.yaml").write_text("d_model: 256\nn_heads: 4\nn_layers: 2\npatch: [2, 2]\nctrl_conditioning: null\n")
    m = Waypoint15Config.from_yaml(tmp_path / "min.yaml")
    assert (m.n_kv_heads, m.n_heads, m.ctrl_conditioning, m.value_residual) == (4, 4, False, False)
    (tmp_path / "list.yaml").write_text("- 1\n- 2\n")
    with pytest.raises(ValueError, match="mapping"):
        Waypoint15Config.from_yaml(tmp_path / "list.yaml")
    with pytest.raises(FileNotFoundError, match="hub"):
        Waypoint15Config.from_yaml("Overworld/some-model")


def test_bad_checkpoints_fail_loudly(tmp_path):
    cfg = tiny_cfg()
    sd = synth_upstream(cfg)
    missing = {k: v for k, v in sd.items() if k != "transformer.blocks.2.attn.k_proj.weight"}
    with pytest.raises(KeyError, match="blocks.2.attn.k_proj"):
        ck.params_from_state_dict(missing, cfg)
    moe = dict(sd)
    moe["transformer.blocks.1.dit_mlp.router.weight"] = ("BF16", np.zeros((8, cfg.d_model), np.uint16))
    with pytest.raises(ValueError, match="mixture of experts"):  # expert weights under a dense configuration
        ck.params_from_state_dict(moe, cfg)
    with pytest.raises(ValueError, match="dense"):  # and dense weights under a MoE configuration
        ck.params_from_state_dict(sd, tiny_cfg(moe=True))
    with pytest.raises(ValueError, match="merged QKV"):
        ck.params_from_state_dict(sd, tiny_cfg(n_kv_heads=2))
    wide = dict(sd)
    wide["ctrl_emb.mlp.fc1.weight"] = ("BF16", np.zeros((cfg.mlp_dim, 40), np.uint16))
    with pytest.raises(ValueError, match="ctrl_emb fc1"):
        ck.params_from_state_dict(wide, cfg)
    with pytest.raises(FileNotFoundError):
        ck.load_checkpoint(tmp_path / "nowhere", cfg)


def test_moe_blocks_are_remapped(tmp_path):
    """Expert weights stored 3-D (``[E, H, D]``, ``[E, D, H]``) come out flattened, the router as it is
    (``_waypoint_15_io.py:139-163``); the dense keys of those blocks are absent."""
    cfg = tiny_cfg(moe=True, moe_n_experts=8, moe_top_k=2, ctrl_conditioning=False)
    sd = synth_upstream(cfg)
    r = np.random.default_rng(3)
    E, H, d = 8, cfg.mlp_dim // 2, cfg.d_model
    for i in range(cfg.n_layers):
        p = f"transformer.blocks.{i}."
        pre = "mlp." if i % 2 == 0 else "dit_mlp."
        del sd[p + pre + "fc1.weight"], sd[p + pre + "fc2.weight"]
        sd[p + pre + "router.weight"] = ("BF16", _cond._bf16(r.standard_normal((E, d), dtype=np.float32)))
        sd[p + pre + "expert_in"] = ("BF16", _cond._bf16(r.standard_normal((E, H, d), dtype=np.float32)))
        sd[p + pre + "expert_out"] = ("F32", r.standard_normal((E, d, H), dtype=np.float32))
    params = ck.params_from_state_dict(sd, cfg)
    for i, blk in enumerate(params["blocks"]):
        p = f"transformer.blocks.{i}." + ("mlp." if i % 2 == 0 else "dit_mlp.")
        assert "fc1.weight" not in blk and blk["moe.expert_in"].shape == (E * H, d) and blk["moe.expert_out"].shape == (E * d, H)
        np.testing.assert_array_equal(blk["moe.router.weight"], sd[p + "router.weight"][1])
        np.testing.assert_array_equal(blk["moe.expert_in"].reshape(E, H, d)[3], sd[p + "expert_in"][1][3])
        np.testing.assert_array_equal(blk["moe.expert_out"].reshape(E, d, H)[5], trunc_bf16(sd[p + "expert_out"][1][5]))
