"""Real-weights ingestion: a ``.safetensors`` file in the upstream training layout -> the host parameter dict
``Waypoint15.load_params`` takes (the layout of ``make_params``).

Follows ``remap_state_dict`` of the reference (``src/quark/models/_waypoint_15_io.py:70-217``): Q / K / V
projections merged into the packed ``qkv`` weight, shared or separate conditioning heads, 4-D patch weights
flattened, the per-channel unpatchify bias tiled over the patch, the fused controller ``fc1`` split into its x and
cond halves, the controller embedding's ``fc1`` padded to a multiple of 16 columns.  The conditioning heads are
then folded into per-sigma rows on the host exactly as for random-init parameters (``_cond.py``), so nothing of
the conditioning network runs on the device.

The safetensors container (8-byte little-endian header length, JSON header, raw little-endian tensor bytes) is
read and written here directly; tensors come back as numpy arrays, bf16 as its ``uint16`` carrier.
"""

from __future__ import annotations

import json
import re
import struct
from pathlib import Path

import numpy as np

from . import _cond

_NP = {"BF16": np.uint16, "F16": np.float16, "F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64, "U8": np.uint8}


def read_safetensors(path) -> dict:
    """``{name: (dtype_tag, array)}``; ``dtype_tag`` is the container's (``"BF16"`` arrays are ``uint16`` carriers)."""
    raw = Path(path).read_bytes()
    if len(raw) < 8:
        raise ValueError(f"{path}: not a safetensors file")
    (hlen,) = struct.unpack("<Q", raw[:8])
    if hlen <= 0 or 8 + hlen > len(raw):
        raise ValueError(f"{path}: header length {hlen} does not fit the file")
    header = json.loads(raw[8 : 8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        tag = meta["dtype"]
        if tag not in _NP:
            raise NotImplementedError(f"{path}: tensor {name!r} has dtype {tag}")
        b, e = meta["data_offsets"]
        arr = np.frombuffer(raw, dtype=_NP[tag], count=(e - b) // np.dtype(_NP[tag]).itemsize, offset=base + b)
        out[name] = (tag, arr.reshape(meta["shape"]))
    return out


def write_safetensors(path, tensors: dict) -> None:
    """``tensors``: ``{name: (dtype_tag, array)}``; the inverse of ``read_safetensors`` (used by tests and tools)."""
    header, blobs, off = {}, [], 0
    for name, (tag, arr) in tensors.items():
        shape = list(np.shape(arr))  # taken first: ascontiguousarray turns a 0-d array into a 1-d one
        a = np.ascontiguousarray(arr, dtype=_NP[tag])
        header[name] = {"dtype": tag, "shape": shape, "data_offsets": [off, off + a.nbytes]}
        blobs.append(a.tobytes())
        off += a.nbytes
    h = json.dumps(header, separators=(",", ":")).encode("utf-8")
    h += b" " * (-len(h) % 8)
    Path(path).write_bytes(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def _as_bf16(entry) -> np.ndarray:
    """Any float tensor as a bf16 carrier (narrowed by truncation, like every upload of the reference)."""
    tag, a = entry
    if tag == "BF16":
        return np.asarray(a, np.uint16)
    return _cond._bf16(np.asarray(a, np.float32))


def _as_f32(entry) -> np.ndarray:
    """The f32 value of the bf16 weight the model holds: the host tables are computed from the loaded bf16
    parameters (``_waypoint_15_io.py:385-393``), so a wider checkpoint is narrowed first."""
    return _cond.bf16_to_f32(_as_bf16(entry))


def params_from_state_dict(raw: dict, cfg) -> dict:
    """Upstream-format state dict (``read_safetensors`` output) -> ``make_params``-layout host parameters."""
    d, ns = cfg.d_model, len(cfg.scheduler_sigmas)
    ph, pw = cfg.patch
    C = cfg.channels
    kpatch = C * ph * pw

    def need(key):
        if key not in raw:
            raise KeyError(f"checkpoint has no tensor {key!r}")
        return raw[key]

    w = _as_bf16(need("patchify.weight"))
    params = {"patchify.weight": w.reshape(d, kpatch)}  # [d, C, ph, pw] flattens to [d, C*ph*pw]
    w = _as_bf16(need("unpatchify.weight"))
    if w.ndim == 4:  # [d, C, ph, pw] -> [C*ph*pw, d]
        w = np.ascontiguousarray(w.transpose(1, 2, 3, 0)).reshape(kpatch, d)
    params["unpatchify.weight"] = w
    b = _as_bf16(need("unpatchify.bias")).reshape(-1)
    if b.size == C:  # one bias per channel: repeat it over the ph * pw positions of the patch
        b = np.repeat(b, ph * pw)
    if b.size != kpatch:
        raise ValueError(f"unpatchify.bias has {b.size} elements, expected {C} or {kpatch}")
    params["unpatchify.bias"] = b

    emb = _cond.noise_embedding(cfg.scheduler_sigmas, cfg.fourier_dim, _as_f32(need("denoise_step_emb.mlp.fc1.weight")),
                                _as_f32(need("denoise_step_emb.mlp.fc2.weight")))  # fmt: skip
    on_w = _as_f32(need("out_norm.fc.weight"))
    params["out_norm.lut"] = [_cond.out_norm_rows(emb[si], on_w) for si in range(ns)]

    blocks = []
    for i in range(cfg.n_layers):
        p = f"transformer.blocks.{i}."
        if p + "cond_head.bias_in" in raw:  # one head shared by the attention and the MLP path
            ab = mb = _as_f32(raw[p + "cond_head.bias_in"])
            projs = [_as_f32(need(p + f"cond_head.cond_proj.{j}.weight")) for j in range(6)]
        else:
            ab = _as_f32(need(p + "attn_cond_head.bias_in"))
            mb = _as_f32(need(p + "mlp_cond_head.bias_in"))
            projs = [_as_f32(need(p + f"attn_cond_head.cond_proj.{j}.weight")) for j in range(3)]
            projs += [_as_f32(need(p + f"mlp_cond_head.cond_proj.{j}.weight")) for j in range(3)]
        # the checkpoint, not the configuration, says whether a block's MLP is dense or a mixture of experts, so that
        # dense weights under a MoE configuration (or the reverse) fail here (_waypoint_15_io.py:135-168)
        moe_pre = next((pre for pre in ("mlp.", "dit_mlp.") if p + pre + "router.weight" in raw), None)
        if (moe_pre is not None) != bool(cfg.moe):
            raise ValueError(f"block {i}: the checkpoint's MLP is {'a mixture of experts' if moe_pre else 'dense'}, the configuration says moe={cfg.moe}")
        pre = "mlp." if p + "mlp.fc1.weight" in raw else "dit_mlp."
        mlp = {}
        if moe_pre is None:
            mlp = {"fc1.weight": _as_bf16(need(p + pre + "fc1.weight")), "fc2.weight": _as_bf16(need(p + pre + "fc2.weight"))}
        else:  # [E, H, D] and [E, D, H] flatten to [E * H, D] and [E * D, H]: the same memory
            E, Hm = cfg.moe_n_experts, cfg.mlp_dim // cfg.moe_top_k
            mlp = {"moe.router.weight": _as_bf16(raw[p + moe_pre + "router.weight"]),
                   "moe.expert_in": _as_bf16(need(p + moe_pre + "expert_in")).reshape(E * Hm, d),
                   "moe.expert_out": _as_bf16(need(p + moe_pre + "expert_out")).reshape(E * d, Hm)}  # fmt: skip
            if mlp["moe.router.weight"].shape != (E, d):
                raise ValueError(f"block {i}: router weight is {mlp['moe.router.weight'].shape}, expected {(E, d)}")
        blk = {
            "qkv.weight": np.concatenate([_as_bf16(need(p + f"attn.{n}_proj.weight")) for n in ("q", "k", "v")], axis=0),
            "out.weight": _as_bf16(need(p + "attn.out_proj.weight")),
            **mlp,
            "lamb": float(_as_f32(raw[p + "attn.v_lamb"]).reshape(-1)[0]) if cfg.value_residual and p + "attn.v_lamb" in raw else 0.5,
            "lut": [_cond.block_rows(emb[si], ab.reshape(-1), mb.reshape(-1), projs) for si in range(ns)],
        }
        if blk["qkv.weight"].shape != (cfg.qkv_dim, d):
            raise ValueError(f"block {i}: merged QKV weight is {blk['qkv.weight'].shape}, expected {(cfg.qkv_dim, d)}")
        if cfg.has_ctrl(i):
            if p + "ctrl_mlpfusion.fc1_x.weight" in raw:
                blk["ctrl.fc1_x.weight"] = _as_bf16(raw[p + "ctrl_mlpfusion.fc1_x.weight"])
                blk["ctrl.fc1_c.weight"] = _as_bf16(need(p + "ctrl_mlpfusion.fc1_c.weight"))
                blk["ctrl.fc2.weight"] = _as_bf16(need(p + "ctrl_mlpfusion.fc2.weight"))
            else:  # one fc1 over cat([x, cond]): its column halves are the two projections
                cat = _as_bf16(need(p + "ctrl_mlpfusion.mlp.fc1.weight"))
                half = cat.shape[1] // 2
                blk["ctrl.fc1_x.weight"] = np.ascontiguousarray(cat[:, :half])
                blk["ctrl.fc1_c.weight"] = np.ascontiguousarray(cat[:, half:])
                blk["ctrl.fc2.weight"] = _as_bf16(need(p + "ctrl_mlpfusion.mlp.fc2.weight"))
        blocks.append(blk)
    params["blocks"] = blocks

    if cfg.ctrl_conditioning:
        w1 = _as_bf16(need("ctrl_emb.mlp.fc1.weight"))  # [d_mid, n_buttons + 3]: columns padded with zeros to 16 k
        if w1.shape[1] > cfg.ctrl_input_width:
            raise ValueError(f"ctrl_emb fc1 has {w1.shape[1]} inputs, the configuration allows {cfg.ctrl_input_width}")
        padded = np.zeros((w1.shape[0], cfg.ctrl_input_width), np.uint16)
        padded[:, : w1.shape[1]] = w1
        params["ctrl_emb.fc1.weight"] = padded
        params["ctrl_emb.fc2.weight"] = _as_bf16(need("ctrl_emb.mlp.fc2.weight"))
    return params


def _local(model_uri, filename: str) -> Path:
    """The file itself, or ``filename`` inside a directory (``src/quark/models/config.py:77-89``); a hub
    repository id would need a download client and a network, neither of which this package has."""
    p = Path(model_uri)
    if p.is_file():
        return p
    if p.is_dir() and (p / filename).is_file():
        return p / filename
    raise FileNotFoundError(f"{model_uri!r}: no local {filename} (download from a hub is not implemented)")


# Defaults of the training repository that change the transformer (``src/quark/models/config.py:25-39``); a
# string of the form ``${name}`` stands for the value of another top-level key.
_CONFIG_DEFAULTS = {"n_kv_heads": "${n_heads}", "patch": [1, 1], "value_residual": False, "inference_fps": "${base_fps}"}
_VAR = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)\}")


def load_yaml_config(model_uri) -> dict:
    """``config.yaml`` (a path, or a directory holding it) merged over the defaults, top-level ``${name}``
    references resolved (``src/quark/models/config.py:45-64, 92-102``)."""
    import yaml

    path = _local(model_uri, "config.yaml")
    raw = yaml.safe_load(path.read_text())
    if not isinstance(raw, dict):
        raise ValueError(f"{path}: the top level of a model config is a mapping")
    out = {**_CONFIG_DEFAULTS, **raw}
    for _ in range(4):  # chains of references are short
        changed = False
        for k, v in list(out.items()):
            m = _VAR.fullmatch(v.strip()) if isinstance(v, str) else None
            if m and m.group(1) in out:
                out[k], changed = out[m.group(1)], True
        if not changed:
            break
    return out


def load_checkpoint(model_uri, cfg) -> dict:
    """``model_uri``: a ``.safetensors`` file, or a directory holding ``model.safetensors``."""
    return params_from_state_dict(read_safetensors(_local(model_uri, "model.safetensors")), cfg)
