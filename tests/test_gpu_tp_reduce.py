"""The fused cross-GPU reduction (``qb_tp_reduce``) on ONE GPU.

Kernels that wait on one another must never be separate launches on one GPU, so the protocol is exercised through
``qb_tp_reduce_emulated``: all ranks run as one cooperative launch over arenas that all live on this GPU, with the same
flags, epochs, peer loads and peer stores as the multi-GPU kernel (the peers' arenas are simply local pointers).
Checked: every rank's arena ends up with the bytes of the unfused chain (sum in rank order rounded to bf16, then
``qf.ada_gate_residual``, then ``qf.ada_rmsnorm`` with its bf16 and e4m3 outputs), over consecutive calls that reuse
the buffers the way a block does.  The bounded wait is checked with a peer that never shows up: the kernel must come
back on its own, with bit 3 of the device status word raised, and the context must stay usable.  The multi-process path
is covered by ``tests/test_gpu_tp.py`` (needs two GPUs).  The reference is single-GPU and has no counterpart.
"""

import ctypes as C

import numpy as np
import pytest

from oracle import codec
from tests import util
from tests.util import bf16_randn

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


class Arenas:
    def __init__(self, qb, world, rows, D):
        lib = qb._lib.load()
        self.qb, self.world, self.rows, self.D = qb, world, rows, D
        n = int(lib.qb_tp_arena_bytes(rows, D))
        assert n == 4096 + rows * D * 11
        self.bufs = [qb.QuarkTensor.zeros(n, dtype="e4m3") for _ in range(world)]
        off = (C.c_size_t * 6)()
        qb._lib.check(lib.qb_tp_arena_offsets(rows, D, off))
        self.off = [int(o) for o in off]

    def view(self, r, i, dt="bf16"):
        return self.qb.QuarkTensor.borrow(self.bufs[r].data_ptr() + self.off[i], (self.rows, self.D), dt, keepalive=self.bufs[r])

    def params(self, **kw):
        p = self.qb._lib.TpParams(world=self.world, rank=0, rows=self.rows, D=self.D, gate_groups=1, norm_groups=1, eps=1e-6, **kw)
        for r in range(self.world):
            p.arena[r] = self.bufs[r].data_ptr()
        return p


def rank_order_sum_bf16(parts):
    acc = np.zeros(parts[0].shape, np.float32)
    for y in parts:
        acc = (acc + codec.bf16_to_f32(y)).astype(np.float32)
    return codec.f32_to_bf16_rne(acc)


@pytest.mark.parametrize("schedule", [1, 2], ids=["one-shot", "two-shot"])
@pytest.mark.parametrize("world,rows,D", [(2, 64, 256), (4, 512, 2048), (8, 128, 2048)])
def test_emulated_ranks_reproduce_the_unfused_chain(qb, world, rows, D, schedule):
    """Both schedules (every rank reduces every row for itself / every rank reduces its share and sends it to all),
    four consecutive calls that alternate the y and x slots the way a block does, each call's residual being the
    x of the call before."""
    r = util.rng(900 + world)
    lib = qb._lib.load()
    ar = Arenas(qb, world, rows, D)
    gate, ns, nb = (T(qb, bf16_randn(r, (1, D)), "bf16") for _ in range(3))
    x_host = bf16_randn(r, (rows, D))
    residuals = [T(qb, x_host, "bf16") for _ in range(world)]  # x is replicated on the ranks
    ptr = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    s = C.c_void_p(qb.runtime.active_stream())
    for call, (slot, act, emit_q) in enumerate([(0, None, True), (1, None, False), (0, "silu", False), (1, None, True)]):
        parts = [bf16_randn(r, (rows, D), 0.5) for _ in range(world)]
        for rk in range(world):
            ar.view(rk, slot).copy_from_numpy(parts[rk])  # y slot = x slot
        p = ar.params(x_slot=slot, norm_activation=1 if act else 0, emit_h=0 if emit_q else 1, emit_hq=1 if emit_q else 0, schedule=schedule)
        res = (C.c_void_p * world)(*[t.data_ptr() for t in residuals])
        qb._lib.check(lib.qb_tp_reduce_emulated(res, ptr(gate), ptr(ns), ptr(nb), C.byref(p), s))
        qb.runtime.synchronize()
        assert qb._lib.device_status() == 0
        # the unfused chain on the same inputs
        summed = T(qb, rank_order_sum_bf16(parts), "bf16")
        want_x = qb.qf.ada_gate_residual(residuals[0], summed, gate)
        want_q = qb.QuarkTensor.empty(rows, D, dtype="e4m3")
        want_h = qb.qf.ada_rmsnorm(want_x, ns, nb, activation=act, out_q=want_q)
        for rk in range(world):
            np.testing.assert_array_equal(ar.view(rk, 2 + slot).to_numpy(), want_x.to_numpy(), err_msg=f"call {call} rank {rk}: x")
            if emit_q:
                np.testing.assert_array_equal(ar.view(rk, 5, "e4m3").to_numpy(), want_q.to_numpy(), err_msg=f"call {call} rank {rk}: hq")
            else:
                np.testing.assert_array_equal(ar.view(rk, 4).to_numpy(), want_h.to_numpy(), err_msg=f"call {call} rank {rk}: h")
        residuals = [ar.view(rk, 2 + slot) for rk in range(world)]  # the next call's residual is this call's x, as in a block


@pytest.mark.parametrize("schedule", [1, 2], ids=["one-shot", "two-shot"])
def test_reduction_without_a_norm_and_with_gate_groups(qb, schedule):
    r = util.rng(950)
    lib = qb._lib.load()
    world, rows, D, G = 2, 64, 512, 4
    ar = Arenas(qb, world, rows, D)
    gate = T(qb, bf16_randn(r, (G, D)), "bf16")
    x_host = bf16_randn(r, (rows, D))
    residuals = [T(qb, x_host, "bf16") for _ in range(world)]
    parts = [bf16_randn(r, (rows, D)) for _ in range(world)]
    for rk in range(world):
        ar.view(rk, 0).copy_from_numpy(parts[rk])
    p = ar.params(x_slot=0, schedule=schedule)
    p.gate_groups = G
    res = (C.c_void_p * world)(*[t.data_ptr() for t in residuals])
    qb._lib.check(lib.qb_tp_reduce_emulated(res, C.c_void_p(gate.data_ptr()), None, None, C.byref(p), C.c_void_p(qb.runtime.active_stream())))
    want = qb.qf.ada_gate_residual(residuals[0], T(qb, rank_order_sum_bf16(parts), "bf16"), gate)
    for rk in range(world):
        np.testing.assert_array_equal(ar.view(rk, 2).to_numpy(), want.to_numpy())


class _RankView:
    """What qf.gemm_tp needs of an arena set, from the point of view of one emulated rank."""

    def __init__(self, ar, rank):
        self.ar, self.rank, self.rows, self.D = ar, rank, ar.rows, ar.D

    def params(self, **kw):
        p = self.ar.params(**kw)
        p.rank = self.rank
        return p


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fp8", [False, True])
def test_partials_pushed_by_the_gemm_then_reduced(qb, world, fp8):
    """The pushed schedule end to end on one GPU: every emulated rank's row-parallel GEMM (qb_gemm_tp) stores the rows of
    its partial into the staging areas of their owners, then the reduction (schedule 3) sums each owner's local blocks.
    Same bytes as plain GEMMs, a rank-order sum rounded to bf16, qf.ada_gate_residual and qf.ada_rmsnorm."""
    r = util.rng(930 + world)
    lib = qb._lib.load()
    rows, D, K = 512, 2048, 256
    ar = Arenas(qb, world, rows, D)
    gate, ns, nb = (T(qb, bf16_randn(r, (1, D)), "bf16") for _ in range(3))
    x = [T(qb, bf16_randn(r, (rows, D)), "bf16") for _ in range(1)] * world
    parts = []
    for rk in range(world):
        if fp8:
            A, B = T(qb, util.e4m3_randn(r, (rows, K)), "e4m3"), T(qb, util.e4m3_randn(r, (D, K), 0.25), "e4m3")
        else:
            A, B = T(qb, bf16_randn(r, (rows, K)), "bf16"), T(qb, bf16_randn(r, (D, K), 0.1), "bf16")
        qb.qf.gemm_tp(A, B, _RankView(ar, rk), compute_dtype="e4m3" if fp8 else None)
        parts.append(qb.qf.gemm(A, B, out_dtype="bf16", compute_dtype="e4m3" if fp8 else None, split_k=1).to_numpy())
    # the staging area of owner o holds, per source rank, the owner's rows of that rank's partial
    rpo = rows // world
    for o in range(world):
        got = ar.view(o, 0).to_numpy().reshape(world, rpo, D)
        for src in range(world):
            np.testing.assert_array_equal(got[src], parts[src][o * rpo : (o + 1) * rpo], err_msg=f"owner {o}, source {src}")
    p = ar.params(x_slot=1, emit_hq=1, schedule=3)
    res = (C.c_void_p * world)(*[t.data_ptr() for t in x])
    qb._lib.check(lib.qb_tp_reduce_emulated(res, C.c_void_p(gate.data_ptr()), C.c_void_p(ns.data_ptr()), C.c_void_p(nb.data_ptr()), C.byref(p),
                                            C.c_void_p(qb.runtime.active_stream())))
    qb.runtime.synchronize()
    assert qb._lib.device_status() == 0
    want_x = qb.qf.ada_gate_residual(x[0], T(qb, rank_order_sum_bf16(parts), "bf16"), gate)
    want_q = qb.QuarkTensor.empty(rows, D, dtype="e4m3")
    qb.qf.ada_rmsnorm(want_x, ns, nb, out_q=want_q)
    for rk in range(world):
        np.testing.assert_array_equal(ar.view(rk, 3).to_numpy(), want_x.to_numpy(), err_msg=f"rank {rk}: x")
        np.testing.assert_array_equal(ar.view(rk, 5, "e4m3").to_numpy(), want_q.to_numpy(), err_msg=f"rank {rk}: hq")


def test_emulated_reduction_time(qb, capsys):
    """Not a parity check: the time of one emulated call at the benchmark's shape, printed for the record (the flag
    exchange here crosses only this GPU's L2, so this is the kernel's own cost without the NVLink latencies)."""
    r = util.rng(970)
    lib = qb._lib.load()
    rows, D = 512, 2048
    out = {}
    for world in (2, 4, 8):
        for schedule in (1, 2):
            ar = Arenas(qb, world, rows, D)
            gate, ns, nb = (T(qb, bf16_randn(r, (1, D)), "bf16") for _ in range(3))
            x = [T(qb, bf16_randn(r, (rows, D)), "bf16") for _ in range(world)]
            res = (C.c_void_p * world)(*[t.data_ptr() for t in x])
            s = C.c_void_p(qb.runtime.active_stream())
            call = lambda i: qb._lib.check(lib.qb_tp_reduce_emulated(res, C.c_void_p(gate.data_ptr()), C.c_void_p(ns.data_ptr()), C.c_void_p(nb.data_ptr()),
                                                                     C.byref(ar.params(x_slot=i & 1, emit_hq=1, schedule=schedule)), s))  # noqa: E731
            for i in range(4):
                call(i)
            e0, e1 = qb.runtime.Event(), qb.runtime.Event()
            e0.record()
            for i in range(40):
                call(i)
            e1.record()
            e1.synchronize()
            out[f"world{world}_{'one' if schedule == 1 else 'two'}_shot_us"] = round(e0.elapsed_ms(e1) * 1e3 / 40, 2)
    assert qb._lib.device_status() == 0
    with capsys.disabled():
        print("\nemulated tp_reduce [512, 2048]:", out)


def test_a_peer_that_never_arrives_ends_the_wait_with_a_status_bit(qb):
    """Rank 0 of a world of two, launched alone through the multi-GPU entry point: nothing ever sets rank 1's flags.
    The wait is given 2 ms; the kernel must return by itself, report bit 3, and leave the GPU usable."""
    r = util.rng(960)
    lib = qb._lib.load()
    rows, D = 64, 256
    ar = Arenas(qb, 2, rows, D)
    gate = T(qb, bf16_randn(r, (1, D)), "bf16")
    x = T(qb, bf16_randn(r, (rows, D)), "bf16")
    ar.view(0, 0).copy_from_numpy(bf16_randn(r, (rows, D)))
    p = ar.params(x_slot=0, wait_limit_us=2000, schedule=2)
    qb._lib.check(lib.qb_tp_reduce(C.c_void_p(x.data_ptr()), C.c_void_p(gate.data_ptr()), None, None, C.byref(p), C.c_void_p(qb.runtime.active_stream())))
    qb.runtime.synchronize()
    assert qb._lib.device_status() == 8  # bit 3: the cross-GPU reduction's wait ran out (reading clears it)
    assert qb._lib.device_status() == 0
    # the context is alive: an ordinary kernel runs and is right
    y = T(qb, bf16_randn(r, (rows, D)), "bf16")
    got = qb.qf.ada_gate_residual(x, y, gate).to_numpy()
    assert np.all(np.isfinite(codec.bf16_to_f32(got)))
    # bad arguments are refused on the host
    p.rows = 63
    assert lib.qb_tp_reduce(C.c_void_p(x.data_ptr()), C.c_void_p(gate.data_ptr()), None, None, C.byref(p), None) == -1


class _AloneComm:
    """Stands in for the communicator of one rank of a sharded session whose peers are not there: the partial sums stay
    partial, so the numbers mean nothing, but every kernel runs with the shapes that rank would see."""

    fused = False
    reduction_name = "none (a rank alone)"

    def __init__(self, rank, world):
        self.rank, self.world = rank, world

    def all_reduce_sum(self, t):
        return t

    def abort(self):
        pass

    def destroy(self):
        return True


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("quant", ["bf16", "fp8"])
def test_a_rank_of_the_bench_geometry_runs_at_wide_sharding(qb, world, quant):
    """The shapes one rank of the 720p model sees when 16 KV heads are spread over 4 or 8 GPUs (2 KV heads, 4 Q heads,
    512-column QKV, 256-wide out-proj K, 1024-wide MLP slices at 8): every kernel accepts them, the key-split attention
    included, the frame is finite and no bounded wait runs out.  Parity of the sharded arithmetic is checked where all
    ranks exist (``test_gpu_tp.py``, ``test_tp_host.py``)."""
    from quark_b200.models import QuantConfig, Waypoint15Config, make_params

    q = QuantConfig.all_fp8() if quant == "fp8" else QuantConfig.all_bf16()
    base = Waypoint15Config(height=32, width=16, n_layers=2, quant=q)
    params = make_params(base, seed=3)
    for rank in (0, world - 1):
        cfg = Waypoint15Config(**{**base.__dict__, "tp_world": world, "tp_rank": rank})
        eng = qb.Engine(cfg=cfg, quant=q, params=params, comm=_AloneComm(rank, world), use_graph=True)
        blk = eng.model.blocks[0]
        assert int(blk.qkv_proj.weight.data.shape[0]) == (32 + 2 * 16) * 64 // world
        r = util.rng(5)
        eng.append_frame(r.standard_normal((1, base.latent_numel)).astype(np.float32))
        out = eng.gen_frame(noise=r.standard_normal((1, base.latent_numel)).astype(np.float32))
        qb.runtime.synchronize()
        assert np.all(np.isfinite(util.f32(out, "bf16")))
        assert qb._lib.device_status() == 0
        eng.close()
