"""Tensor parallelism by KV-head group, host side (no GPU): the weight partition, the rank-local block
restated through the numpy oracle, and the sum over ranks on two gloo processes.

The GPU model shards with ``shard_block_params`` and runs the same kernels on fewer heads, so what can
go wrong on the host is the partition itself; these tests pin it against the unsharded oracle block.
"""

import os
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import codec
from oracle import model as om
from tests import util

ROOT = Path(__file__).resolve().parent.parent


def _cfg(world=1, rank=0):
    from quark_b200.models import QuantConfig, Waypoint15Config

    return Waypoint15Config(d_model=1024, n_layers=1, n_heads=16, n_kv_heads=8, height=4, width=4, local_window=2, global_window=16,
                            quant=QuantConfig.all_bf16(), tp_world=world, tp_rank=rank)  # fmt: skip


def _local_state(cfg, world):
    from quark_b200.models import Waypoint15Config

    sub = Waypoint15Config(**{**cfg.__dict__, "n_heads": cfg.n_heads, "n_kv_heads": cfg.n_kv_heads})
    st = om.new_state(sub, om.Quant(linear="bf16", kv_cache="bf16", attn_compute="bf16"))[0]
    Hk_l = cfg.n_kv_heads // world
    cap = st["K_cache"].shape[0] // cfg.n_kv_heads
    st["K_cache"] = st["K_cache"][: Hk_l * cap].copy()
    st["Vt_cache"] = st["Vt_cache"][: Hk_l * 64].copy()
    return st


def _inputs(cfg):
    from quark_b200.models import make_params

    params = make_params(cfg, seed=3, weight_std=0.08, threads=1)
    r = util.rng(21)
    x = codec.f32_to_bf16(r.standard_normal((cfg.tpf, cfg.d_model)).astype(np.float32))
    return params["blocks"][0], x


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shards_partition_every_weight(world):
    from quark_b200.models.waypoint_15 import shard_block_params

    full, _ = _inputs(_cfg())
    shards = [shard_block_params(_cfg(world, r), full) for r in range(world)]
    c = _cfg()
    Dh, nq, nk = 64, c.n_heads // world * 64, c.n_kv_heads // world * 64
    q = np.concatenate([s["qkv.weight"][:nq] for s in shards])
    k = np.concatenate([s["qkv.weight"][nq : nq + nk] for s in shards])
    v = np.concatenate([s["qkv.weight"][nq + nk :] for s in shards])
    np.testing.assert_array_equal(np.concatenate([q, k, v]), full["qkv.weight"])
    np.testing.assert_array_equal(np.concatenate([s["out.weight"] for s in shards], axis=1), full["out.weight"])
    np.testing.assert_array_equal(np.concatenate([s["fc1.weight"] for s in shards], axis=0), full["fc1.weight"])
    np.testing.assert_array_equal(np.concatenate([s["fc2.weight"] for s in shards], axis=1), full["fc2.weight"])
    for s in shards:  # conditioning rows and the scalar are replicated
        assert s["lamb"] == full["lamb"] and s["lut"] is full["lut"]
        assert s["qkv.weight"].shape == (nq + 2 * nk, c.d_model) and s["qkv.weight"].flags.c_contiguous
    assert Dh == c.Dh


def _sum_bf16(parts):
    """What a bf16 sum all-reduce returns: the f32 sum of the bf16 partials, rounded to bf16 (nearest even)."""
    acc = np.zeros(codec.bf16_to_f32(parts[0]).shape, np.float32)
    for p in parts:
        acc += codec.bf16_to_f32(p)
    return codec.f32_to_bf16_rne(acc)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_rank_local_blocks_sum_to_the_unsharded_block(world):
    """All ranks emulated in one process, in lock step: the reduce hook hands every rank the same sum."""
    from quark_b200.models.waypoint_15 import shard_block_params

    cfg = _cfg()
    full, x = _inputs(cfg)
    q = om.Quant(linear="bf16", kv_cache="bf16", attn_compute="bf16")
    ft = 3
    want, want_qkv = om.block_forward(cfg, 0, full, om.new_state(cfg, q)[0], x, 0, ft, qkv_first=None, frozen=False, quant=q)

    # run the ranks as coroutines so that each reduce sees the partials of all of them
    import threading

    barrier = threading.Barrier(world)
    slots, outs = [None] * world, [None] * world

    def rank_fn(r):
        def reduce(part):
            slots[r] = part
            barrier.wait()
            tot = _sum_bf16(slots)
            barrier.wait()
            return tot

        st = _local_state(cfg, world)
        outs[r] = om.block_forward(cfg, 0, shard_block_params(_cfg(world, r), full), st, x, 0, ft, qkv_first=None, frozen=False,
                                   quant=q, tp_world=world, reduce=reduce) + (st,)  # fmt: skip

    ts = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    full_state = om.new_state(cfg, q)[0]
    om.block_forward(cfg, 0, full, full_state, x, 0, ft, qkv_first=None, frozen=False, quant=q)
    cap = full_state["K_cache"].shape[0] // cfg.n_kv_heads
    Hk_l, nq, nk = cfg.n_kv_heads // world, cfg.n_heads // world * 64, cfg.n_kv_heads // world * 64
    for r in range(world):
        xr, qkv_r, st = outs[r]
        # every rank ends with the same residual stream, equal to the unsharded one up to the order of the sums
        g, w = codec.bf16_to_f32(xr), codec.bf16_to_f32(want)
        assert util.max_rel(g, w) <= util.BF16_MAX_REL and util.cosine(g, w) >= util.COS_MIN
        np.testing.assert_array_equal(xr, outs[0][0])
        # the rank's qkv columns and cache rows are exactly the unsharded ones for its heads
        np.testing.assert_array_equal(qkv_r[:, :nq], want_qkv[:, r * nq : (r + 1) * nq])
        np.testing.assert_array_equal(qkv_r[:, nq : nq + nk], want_qkv[:, cfg.n_heads * 64 + r * nk : cfg.n_heads * 64 + (r + 1) * nk])
        np.testing.assert_array_equal(st["K_cache"], full_state["K_cache"][r * Hk_l * cap : (r + 1) * Hk_l * cap])
        np.testing.assert_array_equal(st["Vt_cache"], full_state["Vt_cache"][r * Hk_l * 64 : (r + 1) * Hk_l * 64])


_CHILD = r"""
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from oracle import codec, model as om
from tests import test_tp_host as T
from quark_b200.models.waypoint_15 import shard_block_params
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
cfg = T._cfg()
full, x = T._inputs(cfg)
q = om.Quant(linear="bf16", kv_cache="bf16", attn_compute="bf16")
def reduce(part):
    t = torch.from_numpy(codec.bf16_to_f32(part).copy())
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return codec.f32_to_bf16_rne(t.numpy())
st = T._local_state(cfg, world)
xr, _ = om.block_forward(cfg, 0, shard_block_params(T._cfg(world, rank), full), st, x, 0, 3, qkv_first=None, frozen=False, quant=q,
                         tp_world=world, reduce=reduce)
if rank == 0:
    want, _ = om.block_forward(cfg, 0, full, om.new_state(cfg, q)[0], x, 0, 3, qkv_first=None, frozen=False, quant=q)
    g, w = codec.bf16_to_f32(xr), codec.bf16_to_f32(want)
    from tests import util
    assert util.max_rel(g, w) <= util.BF16_MAX_REL and util.cosine(g, w) >= util.COS_MIN, (util.max_rel(g, w), util.cosine(g, w))
    print("TP_GLOO_OK")
dist.destroy_process_group()
"""


def test_two_gloo_ranks_reproduce_the_unsharded_block(tmp_path):
    import subprocess

    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    port = 29500 + (os.getpid() % 400)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script), str(ROOT)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0])
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "TP_GLOO_OK" in outs[0]


def test_nccl_binding_loads_and_rejects_bad_ranks():
    from quark_b200.runtime import nccl

    lib = nccl.load()
    for name in ("ncclGetUniqueId", "ncclCommInitRank", "ncclAllReduce", "ncclCommDestroy", "ncclCommAbort"):
        assert hasattr(lib, name)
    with pytest.raises(ValueError):
        nccl.NcclComm(2, 2, "/nonexistent")
    c = nccl.LocalComm()
    assert c.world == 1 and c.all_reduce_sum("x") == "x"


def test_nccl_unique_id_survives_the_file_with_its_zero_bytes(tmp_path):
    import ctypes as C

    from quark_b200.runtime import nccl

    raw = bytes([7, 0, 0, 9]) + bytes(range(124))
    uid = nccl._UniqueId()
    C.memmove(C.byref(uid), raw, 128)
    path = str(tmp_path / "id")
    nccl._write_id(path, uid)
    back = nccl._read_id(path, 1.0, 1)
    assert C.string_at(C.byref(back), 128) == raw
    with pytest.raises(nccl.NcclError):
        nccl._read_id(str(tmp_path / "missing"), 0.05, 1)
