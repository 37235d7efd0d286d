"""The GEMM entry point that runs on the library's built-in scratch memory (collected last on purpose).

``qb_gemm_static_scratch`` exists for hosts that may not allocate device memory at the point where
they need a GEMM (a latency-bound frame loop, an embedded plugin with a fixed memory budget, a
process whose device memory is owned by someone else's allocator).  It must give exactly what
``qb_gemm`` gives with a caller-provided workspace: same kernels, same K-slice order.  The shapes
below are chosen so that scratch is really used (bf16 activations narrowed to e4m3 into the scratch,
K split over several CTAs with partial tiles and tile counters in the scratch), and the call is
made twice in a row because the scratch keeps the previous call's contents.
"""

import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run(qb, entry, A, B, gate, res, p, ws=None):
    lib = qb._lib.load()
    M, N = p.M, p.N
    out = qb.QuarkTensor.from_numpy(np.full((M, N), 0x7FC0, dtype=np.uint16), dtype="bf16")  # NaN-filled: every element must be written
    ptr = lambda t: C.c_void_p(t.data_ptr() if t is not None else None)  # noqa: E731
    s = C.c_void_p(qb.runtime.active_stream())
    if entry == "static":
        rc = lib.qb_gemm_static_scratch(ptr(A), ptr(B), ptr(out), None, ptr(gate), ptr(res), C.byref(p), s)
    else:
        rc = lib.qb_gemm(ptr(A), ptr(B), ptr(out), None, ptr(gate), ptr(res), C.byref(p), ptr(ws), ws.nbytes, s)
    qb._lib.check(rc)
    return out.to_numpy()


@pytest.mark.parametrize("M,N,K,split_k,tile_n,fp8", [(128, 2048, 8192, 4, 64, True), (512, 512, 2048, 2, 128, True), (256, 256, 1024, 4, 128, False)])
def test_static_scratch_gemm_equals_workspace_gemm_twice_in_a_row(M, N, K, split_k, tile_n, fp8):
    import quark_b200 as qb

    qb._lib.require_device(0)
    lib = qb._lib.load()
    r = np.random.default_rng(M + N + K)
    A = qb.QuarkTensor.from_numpy(r.standard_normal((M, K)).astype(np.float32), dtype="bf16")
    Bf = qb.QuarkTensor.from_numpy((0.5 * r.standard_normal((N, K))).astype(np.float32), dtype="bf16")
    B = qb.qf.quantize_e4m3(Bf) if fp8 else Bf
    gate = qb.QuarkTensor.from_numpy(r.standard_normal((1, N)).astype(np.float32), dtype="bf16")
    res = qb.QuarkTensor.from_numpy(r.standard_normal((M, N)).astype(np.float32), dtype="bf16")
    code = qb._lib.DTYPE_CODE
    p = qb._lib.GemmParams(M=M, N=N, K=K, a_dtype=code["bf16"], b_dtype=code["e4m3" if fp8 else "bf16"], c_dtype=code["bf16"],
                           compute_dtype=code["e4m3" if fp8 else "bf16"], activation=0, gate_groups=1, split_k=split_k, tile_n=tile_n,
                           reserved=1)  # slice mode 1: partial tiles and tile counters go through the scratch  # fmt: skip
    need = int(lib.qb_gemm_workspace_bytes(C.byref(p)))
    assert 0 < need <= int(lib.qb_gemm_static_scratch_capacity()), "the case must use scratch and fit the built-in array"
    ws = qb.QuarkTensor.zeros(need, dtype="e4m3")
    want = _run(qb, "workspace", A, B, gate, res, p, ws)
    assert not np.any(want == 0x7FC0)
    first = _run(qb, "static", A, B, gate, res, p)
    second = _run(qb, "static", A, B, gate, res, p)
    np.testing.assert_array_equal(first, want)   # same kernels, same slice order: bit-identical
    np.testing.assert_array_equal(second, want)  # the scratch left by the first call does not leak into the second
    qb.runtime.synchronize()
    assert qb._lib.device_status() == 0


def test_static_scratch_rejects_oversized_requests():
    import quark_b200 as qb

    qb._lib.require_device(0)
    lib = qb._lib.load()
    code = qb._lib.DTYPE_CODE
    # 8 K-slices of a 2048 x 4096 f32 tile set: far beyond 8 MiB
    p = qb._lib.GemmParams(M=2048, N=4096, K=8192, a_dtype=code["bf16"], b_dtype=code["bf16"], c_dtype=code["bf16"],
                           compute_dtype=code["bf16"], gate_groups=1, split_k=8, tile_n=128, reserved=1)  # fmt: skip
    assert int(lib.qb_gemm_workspace_bytes(C.byref(p))) > int(lib.qb_gemm_static_scratch_capacity())
    one = C.c_void_p(256)
    rc = lib.qb_gemm_static_scratch(one, one, one, None, None, None, C.byref(p), None)
    assert rc == -6
    msg = lib.qb_last_error_string().decode()
    assert "built-in scratch holds" in msg and str(int(lib.qb_gemm_static_scratch_capacity())) in msg
