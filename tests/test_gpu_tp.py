"""Tensor-parallel session on two GPUs against the single-GPU session (needs two B200s; skipped otherwise).

Each rank is a child process that sees only its own GPU.  The ranks meet on a file barrier after their
engines are built and before the first collective is launched, so a rank that failed during set-up
never leaves its peer waiting inside an NCCL kernel.
"""

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import codec
from tests import util

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

_CHILD = r"""
import os, sys, time
import numpy as np
rank, world, tmp, quant, fused = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[6] == "1"
os.environ["NCCL_NVLS_ENABLE"] = "0"  # every GPU stays visible: the fused reduction maps the peers' buffers (CUDA IPC)
sys.path.insert(0, sys.argv[5])
import quark_b200 as qb
from quark_b200.models import QuantConfig, Waypoint15Config, make_params
from quark_b200.runtime.nccl import NcclComm
from tests.test_gpu_model import small_cfg

def barrier(tag):
    open(os.path.join(tmp, f"{tag}.{rank}"), "w").close()
    t0 = time.monotonic()
    while not all(os.path.exists(os.path.join(tmp, f"{tag}.{r}")) for r in range(world)):
        if time.monotonic() - t0 > 120:
            raise SystemExit(f"rank {rank}: peer never reached {tag}")
        time.sleep(0.01)

base = small_cfg(qb, quant, d_model=256, n_heads=4, n_kv_heads=2)
cfg = Waypoint15Config(**{**base.__dict__, "tp_world": world, "tp_rank": rank})
params = make_params(base, seed=8, weight_std=0.08)
r = np.random.default_rng(44)
lats = [r.standard_normal((1, base.latent_numel)).astype(np.float32) for _ in range(4)]
qb._lib.require_device(rank)
qb._lib.check(qb._lib.load().qb_set_device(rank))
barrier("loaded")                      # both ranks have a working library and a GPU
comm = NcclComm(rank, world, os.path.join(tmp, "nccl.id"), fused=fused)
eng = qb.Engine(cfg=cfg, quant=cfg.quant, params=params, comm=comm, use_graph=True, device=rank)
barrier("built")
eng.append_frame(lats[0])
blk0 = eng.model.blocks[0].kv_cache
k0, v0 = blk0.K_cache.to_numpy(), blk0.Vt_cache.to_numpy()
outs = [eng.gen_frame(noise=lats[1 + k]) for k in range(3)]
qb.runtime.synchronize()
status = qb._lib.device_status()
barrier("ran")
eng.close()                            # the frame graph holds the communicator's collectives
assert comm.destroy(), "ncclCommDestroy did not return"
res = dict(status=status, k0=k0, v0=v0, **{f"out{k}": o for k, o in enumerate(outs)})
if rank == 0:                          # the single-GPU session with the same weights and inputs
    ref = qb.Engine(cfg=base, quant=base.quant, params=params, use_graph=True, device=rank)
    ref.append_frame(lats[0])
    b0 = ref.model.blocks[0].kv_cache
    res.update(ref_k0=b0.K_cache.to_numpy(), ref_v0=b0.Vt_cache.to_numpy())
    for k in range(3):
        res[f"ref{k}"] = ref.gen_frame(noise=lats[1 + k])
np.savez(os.path.join(tmp, f"rank{rank}.npz"), **res)
print("TP_CHILD_OK", rank)
"""


@pytest.mark.parametrize("fused", [False, True], ids=["nccl", "fused"])
@pytest.mark.parametrize("quant", ["bf16", "fp8"])
def test_two_rank_session_matches_the_single_gpu_session(tmp_path, quant, fused):
    """`fused`: the sum over the ranks, gate + residual and the following AdaRMSNorm as one kernel over peer-mapped
    buffers (`qb_tp_reduce`); otherwise ncclAllReduce followed by the gate and norm kernels."""
    import quark_b200 as qb

    if qb._lib.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), str(tmp_path), quant, str(ROOT), "1" if fused else "0"], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]  # fmt: skip
    # wait for both; as soon as one rank fails the other is stopped (it would wait for its peer otherwise)
    import time

    deadline = time.monotonic() + 300
    while any(p.poll() is None for p in procs):
        if time.monotonic() > deadline or any(p.poll() not in (None, 0) for p in procs):
            for p in procs:
                if p.poll() is None:
                    p.kill()
            break
        time.sleep(0.2)
    outs = [p.communicate()[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(o[-3000:] for o in outs)
    z = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    assert all(int(zz["status"]) == 0 for zz in z)
    # layer 0's cache rows depend on nothing that was summed over ranks: the rank's heads, byte for byte
    nk = z[0]["ref_k0"].shape[0] // world
    nv = z[0]["ref_v0"].shape[0] // world
    for r in range(world):
        np.testing.assert_array_equal(z[r]["k0"], z[0]["ref_k0"][r * nk : (r + 1) * nk])
        np.testing.assert_array_equal(z[r]["v0"], z[0]["ref_v0"][r * nv : (r + 1) * nv])
    for k in range(3):
        np.testing.assert_array_equal(z[0][f"out{k}"], z[1][f"out{k}"])  # both ranks hold the same latent
        g, w = codec.bf16_to_f32(z[0][f"out{k}"]).ravel(), codec.bf16_to_f32(z[0][f"ref{k}"]).ravel()
        cs, mr = util.cosine(g, w), util.max_rel(g, w)
        # three chained frames (15 NFE of 4 layers): the two sessions sum the row-parallel GEMMs in different orders, and
        # that last-bit difference is amplified along the chain like the oracle's two roundings are, so the largest single
        # deviation is held to the chained bound of tests/test_gpu_model.py, the cosine to the per-tensor bound
        assert cs >= util.COS_MIN and (quant == "fp8" or mr <= 5e-2), f"frame {k}: cosine={cs:.6f} max_rel={mr:.3e}"
