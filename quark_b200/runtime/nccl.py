"""Sum all-reduce across the GPUs of one node for the tensor-parallel mode, through ``libnccl.so.2`` with ctypes.

The reference is single-GPU; its sharding by KV-head group needs one exchange step per row-parallel
GEMM: the ``[tpf, d_model]`` bf16 partial outputs are summed over the ranks.  NCCL does that here
(ring / NVLS over NVLink, chosen by NCCL).  The call goes to the active stream, so it is captured into
the frame's CUDA graph like any kernel.

One process per GPU.  The ranks of one node agree on the communicator through a file: rank 0 writes
the 128-byte unique id, the others wait for it (bounded).
"""

from __future__ import annotations

import ctypes as C
import importlib.util
import os
import time

from . import stream as _stream

_NCCL_BF16, _NCCL_F32, _NCCL_S32, _NCCL_SUM, _NCCL_MAX = 9, 7, 2, 0, 2
_DT = {"bf16": _NCCL_BF16, "f32": _NCCL_F32, "s32": _NCCL_S32}


class NcclError(RuntimeError):
    pass


class _UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 128)]


def _find_library() -> str:
    env = os.environ.get("QB_NCCL_PATH")
    if env:
        return env
    spec = importlib.util.find_spec("nvidia.nccl")  # the wheel torch depends on; found without importing torch
    if spec is not None and spec.submodule_search_locations:
        for base in spec.submodule_search_locations:
            cand = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                return cand
    return "libnccl.so.2"


def _write_id(path: str, uid: "_UniqueId") -> None:
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "wb") as f:
        f.write(C.string_at(C.byref(uid), 128))  # all 128 bytes (a c_char array would stop at the first NUL)
    os.replace(tmp, path)  # atomic: a reader never sees a partial id


def _read_id(path: str, timeout_s: float, rank: int) -> "_UniqueId":
    t0 = time.monotonic()
    while not os.path.exists(path):
        if time.monotonic() - t0 > timeout_s:
            raise NcclError(f"NcclComm: rank {rank} waited {timeout_s:.0f} s for {path}")
        time.sleep(0.01)
    with open(path, "rb") as f:
        raw = f.read()
    if len(raw) != 128:
        raise NcclError(f"NcclComm: {path} holds {len(raw)} bytes, expected 128")
    uid = _UniqueId()
    C.memmove(C.byref(uid), raw, 128)
    return uid


_lib = None


def load():
    global _lib
    if _lib is None:
        path = _find_library()
        try:
            lib = C.CDLL(path)
        except OSError as e:
            raise NcclError(f"cannot load NCCL ({path}): {e}; set QB_NCCL_PATH") from e
        lib.ncclGetErrorString.restype = C.c_char_p
        lib.ncclGetErrorString.argtypes = [C.c_int]
        lib.ncclGetUniqueId.argtypes = [C.POINTER(_UniqueId)]
        lib.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, _UniqueId, C.c_int]
        lib.ncclAllReduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        lib.ncclCommDestroy.argtypes = [C.c_void_p]
        lib.ncclCommAbort.argtypes = [C.c_void_p]
        _lib = lib
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise NcclError(f"{what}: {load().ncclGetErrorString(rc).decode()} ({rc})")


class Watchdog:
    """Host-side guard around work that contains collectives: when a guarded region does not finish within
    ``timeout_s`` (a peer died, or never joined), ``comm.abort()`` is called from a timer thread, which makes the
    communicator's kernels on this GPU return instead of waiting for the missing rank for ever; the blocked host
    call then raises.  ``fired`` tells whether that happened.  The reference is single-GPU and has no counterpart.

        wd = Watchdog(comm, timeout_s=5 * median_frame_seconds)
        with wd.guard():
            engine.gen_frame()
    """

    def __init__(self, comm, timeout_s: float):
        if timeout_s <= 0:
            raise ValueError("Watchdog: timeout_s must be positive")
        self.comm, self.timeout_s, self.fired = comm, float(timeout_s), False

    class _Guard:
        def __init__(self, wd):
            import threading

            self.wd, self.done = wd, threading.Event()
            self.thread = threading.Thread(target=self._run, daemon=True)

        def _run(self):
            if not self.done.wait(self.wd.timeout_s):
                self.wd.fired = True
                try:
                    self.wd.comm.abort()
                except Exception:
                    pass

        def __enter__(self):
            self.thread.start()
            return self

        def __exit__(self, exc_type, exc, tb):
            self.done.set()
            self.thread.join()
            if self.wd.fired and exc_type is None:
                raise NcclError(f"Watchdog: the guarded region took longer than {self.wd.timeout_s:.1f} s; the communicator was aborted")
            return False

    def guard(self):
        return Watchdog._Guard(self)


class LocalComm:
    """World of one: nothing to exchange."""

    rank, world = 0, 1
    reduction_name = "none (one rank)"

    def abort(self):
        pass

    def all_reduce_sum(self, t):
        return t

    def all_reduce_max(self, t):
        return t

    def destroy(self):
        pass


class NcclComm:
    """``NcclComm(rank, world, id_path)``: the calling process must already have selected its GPU."""

    reduction_name = "ncclAllReduce (bf16 sum) + gate / residual kernel"

    def __init__(self, rank: int, world: int, id_path: str, *, timeout_s: float = 120.0, fused: bool = False):
        if not (0 <= rank < world):
            raise ValueError(f"NcclComm: rank {rank} of {world}")
        self.rank, self.world = int(rank), int(world)
        self.fused = bool(fused)
        lib = load()
        uid = _UniqueId()
        if rank == 0:
            _check(lib.ncclGetUniqueId(C.byref(uid)), "ncclGetUniqueId")
            _write_id(id_path, uid)
        else:
            uid = _read_id(id_path, timeout_s, rank)
        comm = C.c_void_p()
        _check(lib.ncclCommInitRank(C.byref(comm), self.world, uid, self.rank), "ncclCommInitRank")
        self._comm = comm
        self._arenas = {}
        # Schedule of the fused reduction (qb_tp_reduce): one-shot (1): every rank reads all rows of its peers' partials and
        # reduces for itself; one exchange of flags.  Measured per [512, 2048] reduction with the norm, inside the 720p frame:
        # two B200s 12.0 us (90.0 frames/s); four 25.5 us (81.3 frames/s) against 65.7 / 66.9 frames/s for the two-shot and
        # the pushed two-shot schedules, whose second exchange makes every rank's kernel wait for the slowest peer; eight
        # 54.0 us (53.7 frames/s) against 47.2 us (52.5 frames/s) for the pushed schedule.
        # QB_TP_SCHEDULE overrides (0 = let the kernel choose, 1 one-shot, 2 two-shot, 3 pushed two-shot).
        self.tp_schedule = int(os.environ.get("QB_TP_SCHEDULE", "1"))
        if self.fused:
            self.reduction_name = "one kernel per rank over peer-mapped buffers: sum + gate / residual + the next AdaRMSNorm (qb_tp_reduce)"

    def all_gather_bytes(self, mine: bytes) -> list:
        """Every rank's byte string (all of one length, a multiple of 4), in rank order; synchronises the stream."""
        import numpy as np

        from .tensor import QuarkTensor

        n = len(mine) // 4
        host = np.zeros((self.world, n), dtype=np.int32)
        host[self.rank] = np.frombuffer(mine, dtype=np.int32)
        t = QuarkTensor.from_numpy(host)
        self._all_reduce(t, _NCCL_SUM)  # every slot is zero on all ranks but its owner
        out = t.to_numpy()
        return [out[r].tobytes() for r in range(self.world)]

    def arena(self, rows: int, D: int):
        """The peer-mapped arena for partial outputs of shape [rows, D] (made on first use: call once eagerly on every
        rank before a CUDA graph is captured)."""
        key = (int(rows), int(D))
        a = self._arenas.get(key)
        if a is None:
            from .tp import TpArena

            a = TpArena(self.rank, self.world, rows, D, self.all_gather_bytes)
            self._arenas[key] = a
        return a

    def _all_reduce(self, t, op):
        if t.dtype not in _DT:
            raise TypeError(f"all_reduce: dtype {t.dtype}")
        p = C.c_void_p(t.data_ptr())
        _check(load().ncclAllReduce(p, p, t.numel, _DT[t.dtype], op, self._comm, C.c_void_p(_stream.active_stream())), "ncclAllReduce")
        return t

    def all_reduce_sum(self, t):
        """In-place sum of a bf16 or f32 device tensor over all ranks, on the active stream."""
        return self._all_reduce(t, _NCCL_SUM)

    def all_reduce_max(self, t):
        return self._all_reduce(t, _NCCL_MAX)

    def abort(self):
        if self._comm is not None:
            load().ncclCommAbort(self._comm)
            self._comm = None

    def destroy(self, timeout_s: float = 10.0) -> bool:
        """Releases the communicator.  NCCL keeps a communicator alive while a CUDA graph that captured one
        of its collectives exists, and ``ncclCommDestroy`` then blocks: destroy such graphs first
        (``Engine.close()``).  The call runs in a helper thread and is given ``timeout_s``; if it has not
        returned by then the communicator is left to process exit and False is returned."""
        if self._comm is None:
            return True
        import threading

        for a in self._arenas.values():  # every kernel of this rank has finished (the caller synchronised): unmap the peers
            a.close()
        self._arenas = {}

        comm, self._comm = self._comm, None
        th = threading.Thread(target=lambda: load().ncclCommDestroy(comm), daemon=True)
        th.start()
        th.join(timeout_s)
        return not th.is_alive()
