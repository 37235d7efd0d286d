"""Host logic of the shared scratch buffers of ``qf.*`` (no GPU: the device tensor class is replaced by a stand-in)."""

import ctypes as C


class _FakeTensor:
    _next = 0x1000

    def __init__(self, nbytes):
        self.nbytes = nbytes
        self.addr = _FakeTensor._next
        _FakeTensor._next += 0x100000

    @classmethod
    def zeros(cls, n, dtype="e4m3"):
        return cls(int(n))

    def data_ptr(self):
        return self.addr


def test_a_workspace_that_grows_is_retired_not_freed(monkeypatch):
    """A CUDA graph captured while a smaller workspace was current holds that buffer's address; dropping the
    last reference would free it under the graph.  The replaced buffer must stay owned by the module."""
    from quark_b200 import functional as qfm

    monkeypatch.setattr(qfm, "QuarkTensor", _FakeTensor)
    monkeypatch.setattr(qfm, "_WS", None)
    monkeypatch.setattr(qfm, "_ATTN_WS", None)
    monkeypatch.setattr(qfm, "_RETIRED_WS", [])
    first = qfm._workspace(4096)
    assert first.nbytes >= 1 << 20 and qfm._workspace(8192) is first and qfm._workspace(0) is first
    captured_address = first.data_ptr()
    second = qfm._workspace(64 << 20)
    assert second is not first and second.nbytes >= 64 << 20
    assert any(t is first for t in qfm._RETIRED_WS) and first.data_ptr() == captured_address
    a1 = qfm._attn_workspace(1 << 16)
    a2 = qfm._attn_workspace(1 << 24)
    assert a2 is not a1 and any(t is a1 for t in qfm._RETIRED_WS) and qfm._attn_workspace(0) is None


def test_counter_and_ticket_areas_do_not_depend_on_the_shape():
    """Calls of different shapes share one workspace, so the area that must stay zero between calls (tile
    counters of the GEMM, tickets of the attention key splits) has to end at the same offset for all of them."""
    from quark_b200 import _lib

    lib = _lib.load()

    def gemm_ws(M, N, K, split_k, a_dtype=1):
        p = _lib.GemmParams(M=M, N=N, K=K, a_dtype=a_dtype, b_dtype=1, c_dtype=0, compute_dtype=1, gate_groups=1, split_k=split_k, tile_n=64,
                            reserved=1)  # fmt: skip
        return int(lib.qb_gemm_workspace_bytes(C.byref(p)))

    counters = 64 << 10
    assert gemm_ws(128, 256, 512, 1) == 0  # e4m3 A, one slice: no scratch memory at all
    assert gemm_ws(128, 256, 512, 1, a_dtype=0) == counters + 128 * 512  # the e4m3 copy of a bf16 A follows the counters
    assert gemm_ws(512, 4096, 768, 3) == counters + 3 * 512 * 4096 * 4  # 256 tiles
    assert gemm_ws(1024, 4096, 768, 3) == counters + 3 * 1024 * 4096 * 4  # 512 tiles: same counter area
