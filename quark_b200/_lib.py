"""ctypes binding of ``libquark_b200.so`` (declared in ``include/quark_b200.h``).

The library is the only compute path: there is no Python, numpy or torch fallback.  If the
shared object is missing, ``load()`` raises with the build command instead of degrading.
The reference binds ``libcuda`` / ``libcublasLt`` the same way
(``src/quark/runtime/cuda.py:81-110``, ``src/quark/runtime/cublas.py:94-118``).
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

QB_BF16, QB_E4M3, QB_F32, QB_S32 = 0, 1, 2, 3
DTYPE_CODE = {"bf16": QB_BF16, "e4m3": QB_E4M3, "f32": QB_F32, "s32": QB_S32}

_STATUS_NAMES = {
    0: "QB_OK",
    -1: "QB_ERR_INVALID_ARG",
    -2: "QB_ERR_UNSUPPORTED",
    -3: "QB_ERR_ALIGN",
    -4: "QB_ERR_LAUNCH",
    -5: "QB_ERR_DEVICE",
    -6: "QB_ERR_WORKSPACE",
    -7: "QB_ERR_CUDA",
}


class QbError(RuntimeError):
    """A C-ABI call returned a negative status (the reference's counterpart is ``CudaError``,
    ``src/quark/runtime/cuda.py:71-78``)."""

    def __init__(self, code: int, message: str):
        self.code = code
        self.name = _STATUS_NAMES.get(code, f"QB_ERR_{code}")
        self.message = message
        super().__init__(f"{self.name} ({code}): {message}")


class GemmParams(C.Structure):
    _fields_ = [
        ("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("a_dtype", C.c_int32), ("b_dtype", C.c_int32), ("c_dtype", C.c_int32),
        ("compute_dtype", C.c_int32), ("activation", C.c_int32), ("gate_groups", C.c_int32),
        ("split_k", C.c_int32), ("tile_n", C.c_int32), ("reserved", C.c_int32),
        ("a_scale", C.c_void_p), ("w_scale", C.c_void_p),
    ]  # fmt: skip


class KvParams(C.Structure):
    _fields_ = [
        ("n_q_heads", C.c_int32), ("n_kv_heads", C.c_int32),
        ("H_spatial", C.c_int32), ("W_spatial", C.c_int32),
        ("num_buckets", C.c_int32), ("pinned_dilation", C.c_int32),
        ("kv_dtype", C.c_int32), ("max_segments", C.c_int32),
        ("quilt_factor", C.c_int32), ("packed_qkv", C.c_int32), ("quilt_offset", C.c_int32),
        ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
    ]  # fmt: skip


class AttnParams(C.Structure):
    _fields_ = [
        ("n_kv_heads", C.c_int32), ("gqa_ratio", C.c_int32),
        ("H_spatial", C.c_int32), ("W_spatial", C.c_int32),
        ("num_buckets", C.c_int32), ("pinned_dilation", C.c_int32),
        ("kv_dtype", C.c_int32), ("compute_dtype", C.c_int32),
        ("max_segments", C.c_int32), ("packed_qkv", C.c_int32),
        ("quilt_factor", C.c_int32), ("kv_splits", C.c_int32),
        ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
    ]  # fmt: skip


class TpParams(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("rows", C.c_int32), ("D", C.c_int32),
        ("gate_groups", C.c_int32), ("norm_groups", C.c_int32), ("norm_activation", C.c_int32), ("x_slot", C.c_int32),
        ("emit_h", C.c_int32), ("emit_hq", C.c_int32), ("wait_limit_us", C.c_int32), ("eps", C.c_float),
        ("schedule", C.c_int32), ("reserved", C.c_int32),
        ("arena", C.c_void_p * 8),
    ]  # fmt: skip


_P, _I, _Z, _F, _U = C.c_void_p, C.c_int32, C.c_size_t, C.c_float, C.c_uint32

# name -> (restype, argtypes); every symbol include/quark_b200.h declares
SIGNATURES = {
    "qb_version": (_I, []),
    "qb_last_error_string": (C.c_char_p, []),
    "qb_device_count": (_I, []),
    "qb_device_check": (_I, [_I]),
    "qb_set_device": (_I, [_I]),
    "qb_device_status": (_I, [C.POINTER(_U)]),
    "qb_kernel_launch_count": (C.c_uint64, []),
    "qb_set_dependent_launch": (C.c_int32, [C.c_int32]),
    "qb_malloc": (_I, [C.POINTER(_P), _Z]),
    "qb_free": (_I, [_P]),
    "qb_host_alloc": (_I, [C.POINTER(_P), _Z]),
    "qb_host_free": (_I, [_P]),
    "qb_memcpy_async": (_I, [_P, _P, _Z, _I, _P]),
    "qb_memset_async": (_I, [_P, _I, _Z, _P]),
    "qb_memset32_async": (_I, [_P, _U, _Z, _P]),
    "qb_stream_create": (_I, [C.POINTER(_P)]),
    "qb_stream_destroy": (_I, [_P]),
    "qb_stream_sync": (_I, [_P]),
    "qb_device_sync": (_I, []),
    "qb_event_create": (_I, [C.POINTER(_P)]),
    "qb_event_destroy": (_I, [_P]),
    "qb_event_record": (_I, [_P, _P]),
    "qb_event_sync": (_I, [_P]),
    "qb_event_elapsed_ms": (_I, [_P, _P, C.POINTER(_F)]),
    "qb_graph_begin": (_I, [_P]),
    "qb_graph_end": (_I, [_P, C.POINTER(_P)]),
    "qb_graph_launch": (_I, [_P, _P]),
    "qb_graph_destroy": (_I, [_P]),
    "qb_gemm_workspace_bytes": (_Z, [C.POINTER(GemmParams)]),
    "qb_gemm": (_I, [_P, _P, _P, _P, _P, _P, C.POINTER(GemmParams), _P, _Z, _P]),
    "qb_gemm_static_scratch_capacity": (_Z, []),
    "qb_gemm_static_scratch": (_I, [_P, _P, _P, _P, _P, _P, C.POINTER(GemmParams), _P]),
    "qb_quantize_e4m3": (_I, [_P, _P, _Z, _I, _P]),
    "qb_quantize_e4m3_rows": (_I, [_P, _P, _P, _I, _I, _P]),
    "qb_dequantize_e4m3": (_I, [_P, _P, _Z, _P]),
    "qb_kv_cache_update": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, C.POINTER(KvParams), _P]),
    "qb_kv_cache_update_kv": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, C.POINTER(KvParams), _P]),
    "qb_qkv_post": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, C.POINTER(KvParams), _F, _P]),
    "qb_gemm_qkv_post": (_I, [_P] * 12 + [C.POINTER(GemmParams), C.POINTER(KvParams), _F, _P, _Z, _P]),
    "qb_rope_table_build": (_I, [_P, _I, _I, _P]),
    "qb_owl_attn_workspace_bytes": (_Z, [C.POINTER(AttnParams)]),
    "qb_owl_attn": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, C.POINTER(AttnParams), _P, _Z, _P]),
    "qb_ada_rmsnorm": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _P]),
    "qb_rmsnorm": (_I, [_P, _P, _I, _I, _F, _P]),
    "qb_add": (_I, [_P, _P, _P, _Z, _P]),
    "qb_head_rmsnorm": (_I, [_P, _P, _I, _I, _I, _I, _F, _P]),
    "qb_value_residual_packed": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "qb_ada_gate_residual": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "qb_silu": (_I, [_P, _P, _P, _Z, _P]),
    "qb_euler_step": (_I, [_P, _P, _P, _P, _Z, _P]),
    "qb_randn": (_I, [_P, _P, _Z, _I, _U, _U, _U, _P]),
    "qb_moe_route": (_I, [_P, _P, _I, _I, _I, _P]),
    "qb_moe_combine": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "qb_increment": (_I, [_P, _P]),
    "qb_patchify": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "qb_unpatchify": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "qb_patch_gather": (_I, [_P, _P, _I, _I, _I, _I, _I, _P]),
    "qb_patch_scatter": (_I, [_P, _P, _I, _I, _I, _I, _I, _P]),
    "qb_gemm_tp": (_I, [_P, _P, C.POINTER(GemmParams), C.POINTER(TpParams), _P, _Z, _P]),
    "qb_set_attn_exact_exp": (_I, [_I]),
    "qb_kv_cast_appended": (_I, [_P, _P, _P, _P, _P, _P, C.POINTER(KvParams), _P]),
    "qb_moe_slots": (_Z, [_I, _I, _I]),
    "qb_moe_route_slots": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "qb_moe_gather": (_I, [_P, _P, _P, _I, _I, _P]),
    "qb_gemm_grouped_workspace_bytes": (_Z, [C.POINTER(GemmParams)]),
    "qb_gemm_grouped": (_I, [_P, _P, _P, _P, _I, C.POINTER(GemmParams), _P, _Z, _P]),
    "qb_moe_reduce": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "qb_tp_arena_bytes": (_Z, [_I, _I]),
    "qb_tp_arena_offsets": (_I, [_I, _I, C.POINTER(_Z)]),
    "qb_tp_reduce": (_I, [_P, _P, _P, _P, C.POINTER(TpParams), _P]),
    "qb_tp_reduce_emulated": (_I, [C.POINTER(_P), _P, _P, _P, C.POINTER(TpParams), _P]),
    "qb_ipc_export": (_I, [_P, _P]),
    "qb_ipc_open": (_I, [_P, C.POINTER(_P)]),
    "qb_ipc_close": (_I, [_P]),
}

_lib = None


def library_path() -> Path:
    env = os.environ.get("QUARK_B200_LIB_PATH")
    return Path(env) if env else Path(__file__).resolve().parent / "libquark_b200.so"


def load():
    """Load the shared library once; fail loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise ImportError(
            f"{path} is missing: the CUDA kernel library has not been built. "
            f"Run `bash quark_b200/csrc/build.sh` (needs nvcc with sm_100a support); there is no CPU fallback."
        )
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        msg = load().qb_last_error_string()
        raise QbError(int(rc), msg.decode("utf-8", "replace") if msg else "")


def device_count() -> int:
    return int(load().qb_device_count())


def require_device(device: int = 0) -> None:
    """Raise unless ``device`` is a compute-capability 10.0 GPU."""
    check(load().qb_device_check(device))


def kernel_launch_count() -> int:
    return int(load().qb_kernel_launch_count())


def set_dependent_launch(enabled: bool) -> bool:
    """Turns the overlap of a kernel's set-up with its predecessor's tail on or off; returns the old setting."""
    return bool(load().qb_set_dependent_launch(1 if enabled else 0))


def set_attn_exact_exp(enabled: bool) -> bool:
    """e4m3 attention: ``True`` computes every probability with ``ex2.approx``; ``False`` (the default) builds every second one
    on the FMA pipe from a centred chord of ``2^x`` (see ``qb_set_attn_exact_exp``).  Returns the old setting."""
    return bool(load().qb_set_attn_exact_exp(1 if enabled else 0))


def device_status() -> int:
    v = _U(0)
    check(load().qb_device_status(C.byref(v)))
    return int(v.value)
