"""Host-side logic of the multi-GPU bench on CPU: two `gloo` ranks, no GPU.

`bench.py --gpus N` runs one independent session per rank (the path has no exchange step), takes the
maximum of the per-rank times and reports the sum of the ranks' frames over that time.  This test
runs that reduction with world_size 2 and checks the session-sharding rules that need no device.
"""

import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench

    # rank r "measured" (10 + r) ms on the device and (20 - r) ms end to end
    dev_ms, e2e_ms = bench.max_over_ranks([10.0 + rank, 20.0 - rank], dist, "cpu")
    dist.barrier()
    q.put((rank, dev_ms, e2e_ms, bench.aggregate_fps(world, 5, dev_ms)))
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_slowest_time():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, dev_ms, e2e_ms, fps in res:
        assert dev_ms == 11.0 and e2e_ms == 20.0  # max over ranks, identical on every rank
        assert fps == pytest.approx(2 * 5 * 1000.0 / 11.0)


def test_single_process_is_the_identity():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.max_over_ranks([3.0, 4.0], None) == [3.0, 4.0]
    assert bench.aggregate_fps(1, 10, 500.0) == pytest.approx(20.0)


def test_sessions_are_seeded_per_rank():
    """Each rank owns a whole session: its own seed gives its own weights; nothing is shared or split."""
    sys.path.insert(0, str(ROOT))
    import numpy as np

    from quark_b200.models import Waypoint15Config, make_params

    cfg = Waypoint15Config(d_model=128, n_layers=1, n_heads=2, n_kv_heads=1, height=8, width=8, channels=4)
    a, b = make_params(cfg, seed=0), make_params(cfg, seed=1)
    assert not np.array_equal(a["blocks"][0]["qkv.weight"], b["blocks"][0]["qkv.weight"])
    assert np.array_equal(a["blocks"][0]["qkv.weight"], make_params(cfg, seed=0)["blocks"][0]["qkv.weight"])
