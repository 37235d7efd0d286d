"""The stream every call of the package runs on, and CUDA-graph capture of it.

The reference routes all work to one "active stream" that a capture context swaps
(``src/quark/graph.py:47-49``, ``:105-173``).  Here a single non-blocking stream is created on
first use and used for every launch and copy, so capture needs no stream switch: entering
``capture_graph()`` starts capturing that stream, leaving it instantiates the graph.
"""

from __future__ import annotations

import ctypes as C

from .. import _lib

_stream: int | None = None


def active_stream() -> int:
    global _stream
    if _stream is None:
        p = C.c_void_p()
        _lib.check(_lib.load().qb_stream_create(C.byref(p)))
        _stream = int(p.value)
    return _stream


def set_stream(handle: int) -> None:
    """Run on a caller-owned ``cudaStream_t`` instead (must not be the legacy default stream when graphs are captured)."""
    global _stream
    _stream = int(handle)


def synchronize() -> None:
    _lib.check(_lib.load().qb_stream_sync(C.c_void_p(active_stream())))


class Event:
    def __init__(self):
        p = C.c_void_p()
        _lib.check(_lib.load().qb_event_create(C.byref(p)))
        self.handle = int(p.value)

    def record(self) -> "Event":
        _lib.check(_lib.load().qb_event_record(C.c_void_p(self.handle), C.c_void_p(active_stream())))
        return self

    def synchronize(self) -> None:
        _lib.check(_lib.load().qb_event_sync(C.c_void_p(self.handle)))

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float(0)
        _lib.check(_lib.load().qb_event_elapsed_ms(C.c_void_p(self.handle), C.c_void_p(later.handle), C.byref(ms)))
        return float(ms.value)

    def __del__(self):
        try:
            _lib.load().qb_event_destroy(C.c_void_p(self.handle))
        except Exception:
            pass


class Graph:
    """An instantiated CUDA graph; ``launch()`` replays it on the active stream."""

    def __init__(self, handle: int):
        self.handle = handle

    def launch(self) -> None:
        _lib.check(_lib.load().qb_graph_launch(C.c_void_p(self.handle), C.c_void_p(active_stream())))

    def __del__(self):
        try:
            _lib.load().qb_graph_destroy(C.c_void_p(self.handle))
        except Exception:
            pass


class capture_graph:
    """``with capture_graph() as cap: ...`` then ``cap.graph.launch()``.

    Nothing inside the block may allocate or synchronise; run the same calls once eagerly
    first so that every cached buffer exists (the reference has the same rule,
    ``src/quark/models/waypoint_15.py:729-753``).
    """

    def __init__(self):
        self.graph: Graph | None = None

    def __enter__(self):
        synchronize()
        _lib.check(_lib.load().qb_graph_begin(C.c_void_p(active_stream())))
        return self

    def __exit__(self, exc_type, exc, tb):
        p = C.c_void_p()
        rc = _lib.load().qb_graph_end(C.c_void_p(active_stream()), C.byref(p))
        if exc_type is None:
            _lib.check(rc)
            self.graph = Graph(int(p.value))
        return False
