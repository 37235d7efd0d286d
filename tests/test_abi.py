"""The shared library loads without a GPU and exports every symbol the header declares."""

import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "quark_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    from quark_b200 import _lib

    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    from quark_b200 import _lib

    lib = _lib.load()
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.qb_version() >= 100
    assert lib.qb_device_count() >= 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from quark_b200 import _lib

    monkeypatch.setenv("QUARK_B200_LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.load()


def test_argument_validation_needs_no_gpu():
    """Entry points reject bad arguments on the host, before touching the device."""
    import ctypes as C

    from quark_b200 import _lib

    lib = _lib.load()
    p = _lib.GemmParams(M=128, N=100, K=64, a_dtype=0, b_dtype=0, c_dtype=0, compute_dtype=0, gate_groups=1)
    assert lib.qb_gemm(None, None, None, None, None, None, C.byref(p), None, 0, None) == -3  # N % 8
    assert b"multiple of 8" in lib.qb_last_error_string()
    p.N = 128
    assert lib.qb_gemm(None, None, None, None, None, None, C.byref(p), None, 0, None) == -1  # NULL operands
    p.compute_dtype = 1
    assert lib.qb_gemm(None, None, None, None, None, None, C.byref(p), None, 0, None) == -1  # e4m3 compute needs e4m3 B
    assert lib.qb_gemm_workspace_bytes(C.byref(p)) == 0
    # every case below fails a check on the host: nothing may reach a launch with these made-up pointers
    kp = _lib.KvParams(n_q_heads=4, n_kv_heads=2, H_spatial=8, W_spatial=8, num_buckets=4, pinned_dilation=1, kv_dtype=0,
                       max_segments=3, quilt_factor=3, packed_qkv=1)  # fmt: skip
    one = C.c_void_p(16)
    assert lib.qb_kv_cache_update(one, one, one, one, one, one, one, one, C.byref(kp), None) == -1  # 64 tokens do not split in 3
    kp.quilt_factor = 8
    assert lib.qb_kv_cache_update(one, one, one, one, one, one, one, one, C.byref(kp), None) == -2  # 8 cached tokens: less than one 16-byte vector of V^T
    kp.quilt_factor, kp.quilt_offset = 2, 2
    assert lib.qb_kv_cache_update(one, one, one, one, one, one, one, one, C.byref(kp), None) == -1  # offset outside [0, quilt_factor)
    kp.quilt_offset, kp.packed_qkv = 0, 0
    assert lib.qb_kv_cache_update(one, one, one, one, one, one, one, one, C.byref(kp), None) == -1  # separate K, V have an entry of their own
    ap = _lib.AttnParams(n_kv_heads=2, gqa_ratio=2, H_spatial=8, W_spatial=8, num_buckets=4, pinned_dilation=1, kv_dtype=0,
                         compute_dtype=1, max_segments=3, packed_qkv=1, quilt_factor=1)  # fmt: skip
    assert lib.qb_owl_attn(one, one, one, one, one, one, one, None, one, C.byref(ap), None, 0, None) == -2  # mixed dtypes
    assert lib.qb_rope_table_build(one, 0, 8, None) == -1
    assert lib.qb_device_check(9999) == -5


def test_attention_key_split_choice_and_workspace_size_need_no_gpu():
    """How many CTAs share the keys of one (query tile, head) follows from the geometry alone: none at 720p
    (4 x 32 items fill the GPU), four at 360p (32 items), eight for a tensor-parallel rank with two KV heads;
    the workspace is a fixed 16 KiB ticket area (the same for every geometry, so that calls can share a
    workspace) plus 66 x 128 floats per item and share."""
    import ctypes as C

    from quark_b200 import _lib

    lib = _lib.load()

    def ws(H, W, Hk, splits=0):
        ap = _lib.AttnParams(n_kv_heads=Hk, gqa_ratio=2, H_spatial=H, W_spatial=W, num_buckets=16, pinned_dilation=1, kv_dtype=1,
                             compute_dtype=1, max_segments=3, packed_qkv=1, quilt_factor=1, kv_splits=splits)  # fmt: skip
        return int(lib.qb_owl_attn_workspace_bytes(C.byref(ap)))

    per = 66 * 128 * 4
    assert ws(32, 16, 16) == 0
    assert ws(16, 8, 16) == 16384 + 32 * 4 * per
    assert ws(32, 16, 2) == 16384 + 16 * 8 * per
    assert ws(32, 16, 16, splits=1) == 0
    assert ws(32, 16, 16, splits=2) == 16384 + 128 * 2 * per
