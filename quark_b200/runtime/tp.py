"""Peer-mapped arenas and the fused cross-GPU reduction of the tensor-parallel mode (``qb_tp_reduce``).

One process per GPU.  Every rank allocates an arena (flags, its partial ``y``, two ``x`` slots, ``h`` in bf16 and
e4m3), exports it with CUDA IPC, and maps its peers' arenas; the kernel then sums the ranks' partials with plain
peer loads and stores its share of the result rows into every rank's arena.  The reference is single-GPU
(``src/quark/models/waypoint_15.py:318``) and has no counterpart.
"""

from __future__ import annotations

import ctypes as C

from .. import _lib
from . import stream as _stream
from .tensor import QuarkTensor


class TpArena:
    """``TpArena(rank, world, rows, D, exchange)``: ``exchange(handle: bytes) -> list[bytes]`` hands every rank's
    64-byte IPC handle to every rank (rank order).  All GPUs of the job must be visible to the process."""

    def __init__(self, rank: int, world: int, rows: int, D: int, exchange):
        lib = _lib.load()
        self.rank, self.world, self.rows, self.D = int(rank), int(world), int(rows), int(D)
        nbytes = int(lib.qb_tp_arena_bytes(rows, D))
        if nbytes == 0 or rows % world:
            raise ValueError(f"TpArena: [{rows}, {D}] over {world} ranks")
        self.buf = QuarkTensor.zeros(nbytes, dtype="e4m3")  # flags start at zero: epoch 0
        _stream.synchronize()
        off = (C.c_size_t * 6)()
        _lib.check(lib.qb_tp_arena_offsets(rows, D, off))
        base = self.buf.data_ptr()
        view = lambda i, dt: QuarkTensor.borrow(base + int(off[i]), (rows, D), dt, keepalive=self.buf)  # noqa: E731
        self.y = (view(0, "bf16"), view(1, "bf16"))  # this rank's row-parallel GEMM writes its partial into y[x_slot]
        self.x = (view(2, "bf16"), view(3, "bf16"))
        self.h, self.hq = view(4, "bf16"), view(5, "e4m3")
        handle = (C.c_uint8 * 64)()
        _lib.check(lib.qb_ipc_export(C.c_void_p(base), handle))
        handles = exchange(bytes(handle))
        if len(handles) != world or handles[rank] != bytes(handle):
            raise RuntimeError("TpArena: the handle exchange did not return this rank's own handle in its place")
        self._opened = []
        self.ptrs = []
        for r in range(world):
            if r == rank:
                self.ptrs.append(base)
                continue
            p = C.c_void_p()
            raw = (C.c_uint8 * 64).from_buffer_copy(handles[r])
            _lib.check(lib.qb_ipc_open(raw, C.byref(p)))
            self._opened.append(int(p.value))
            self.ptrs.append(int(p.value))

    def params(self, **kw):
        p = _lib.TpParams(world=self.world, rank=self.rank, rows=self.rows, D=self.D, **kw)
        for r in range(self.world):
            p.arena[r] = self.ptrs[r]
        return p

    def reduce(self, residual, gate, norm_scale=None, norm_bias=None, *, activation=None, x_slot: int, emit_e4m3: bool = False, eps: float = 1e-6,
               wait_limit_us: int = 0, schedule: int = 0):  # fmt: skip
        """``x_new = residual + gate * sum over ranks of y[x_slot]`` and, with ``norm_scale`` / ``norm_bias``, ``h = ada_rmsnorm(x_new)``.
        Returns ``(x_new, h)``: views into this rank's arena (``h`` is the e4m3 buffer when ``emit_e4m3``; None without a norm)."""
        if activation not in (None, "silu"):
            raise ValueError(f"TpArena.reduce: activation {activation!r}")
        G = gate.numel // self.D
        Gn = norm_scale.numel // self.D if norm_scale is not None else 1
        p = _lib.TpParams(world=self.world, rank=self.rank, rows=self.rows, D=self.D, gate_groups=G, norm_groups=Gn,
                          norm_activation=1 if activation == "silu" else 0, x_slot=int(x_slot), emit_h=0 if emit_e4m3 else 1,
                          emit_hq=1 if emit_e4m3 else 0, wait_limit_us=int(wait_limit_us), eps=float(eps), schedule=int(schedule))  # fmt: skip
        for r in range(self.world):
            p.arena[r] = self.ptrs[r]
        ptr = lambda t: C.c_void_p(t.data_ptr() if t is not None else None)  # noqa: E731
        _lib.check(_lib.load().qb_tp_reduce(ptr(residual), ptr(gate), ptr(norm_scale), ptr(norm_bias), C.byref(p), C.c_void_p(_stream.active_stream())))
        h = None if norm_scale is None else (self.hq if emit_e4m3 else self.h)
        return self.x[x_slot], h

    def close(self) -> None:
        """Unmaps the peers' arenas.  Call only when no rank can still launch a reduction (after a barrier)."""
        lib = _lib.load()
        for p in self._opened:
            lib.qb_ipc_close(C.c_void_p(p))
        self._opened = []
