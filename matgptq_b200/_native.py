"""ctypes binding of ``libmatgptq_b200.so`` (the C ABI in ``include/matgptq_b200.h``).

There is no fallback: if the library is missing or a symbol is absent, importing the
operators raises.  Build it with ``python -m matgptq_b200.build``.
"""
from __future__ import annotations

import ctypes
import os

# MATGPTQ_B200_LIBRARY points at another build of the same library (for A/B measurements)
_LIB_PATH = os.environ.get("MATGPTQ_B200_LIBRARY") or os.path.join(
    os.path.dirname(os.path.abspath(__file__)), "libmatgptq_b200.so")

OK = 0
ERR_CUDA = 2  # MATGPTQ_B200_ERR_CUDA: a CUDA runtime call or a kernel launch failed
FLAG_ASYNC = 1
FLAG_BF16 = 2
FLAG_PDL = 4
FLAG_SCRATCH_REDUCE = 8

_c_i64 = ctypes.c_int64
_c_int = ctypes.c_int
_c_u32 = ctypes.c_uint32
_c_ptr = ctypes.c_void_p

class Segment(ctypes.Structure):
    """``matgptq_b200_segment`` of the C header: one weight matrix of a grouped product."""
    _fields_ = [("w", ctypes.c_void_p), ("s", ctypes.c_void_p), ("n_out", ctypes.c_int64), ("bitwidth", ctypes.c_int64)]


class Comm(ctypes.Structure):
    """``matgptq_b200_comm`` of the C header: peer buffers of the fused row-parallel product + all-reduce."""
    _fields_ = [("data", ctypes.c_void_p * 8), ("ctrl", ctypes.c_void_p),
                ("slot_elems", ctypes.c_int64), ("rank", ctypes.c_int), ("nranks", ctypes.c_int), ("push_only", ctypes.c_int)]


# symbol -> (restype, argtypes); must list every function declared in include/matgptq_b200.h
SIGNATURES = {
    "matgptq_b200_version": (_c_int, []),
    "matgptq_b200_strerror": (ctypes.c_char_p, [_c_int]),
    "matgptq_b200_matmul": (_c_int, [_c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_u32]),
    "matgptq_b200_matmul_zp": (_c_int, [_c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_u32]),
    "matgptq_b200_matmul_tuned": (_c_int, [_c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_u32, _c_int, _c_int]),
    "matgptq_b200_matmul_ws": (_c_int, [_c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_u32, _c_ptr, _c_i64, _c_int, _c_int]),
    "matgptq_b200_matmul_grouped": (_c_int, [ctypes.POINTER(Segment), _c_int, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_u32, _c_ptr, _c_i64]),
    "matgptq_b200_matmul_allreduce": (_c_int, [_c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_u32, ctypes.POINTER(Comm)]),
    "matgptq_b200_allreduce_finish": (_c_int, [ctypes.POINTER(Comm), _c_ptr, _c_i64, _c_i64, _c_ptr, _c_u32]),
    "matgptq_b200_matmul_workspace_bytes": (_c_i64, [_c_i64, _c_i64, _c_i64]),
    "matgptq_b200_matmul_static_scratch": (_c_int, [_c_i64, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_u32]),
    "matgptq_b200_add_rmsnorm": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, ctypes.c_float, _c_u32, _c_ptr]),
    "matgptq_b200_rope_kv": (_c_int, [_c_ptr] * 7 + [_c_i64] * 6 + [_c_u32, _c_ptr]),
    "matgptq_b200_argmax": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_u32, _c_ptr]),
    "matgptq_b200_silu_mul": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_u32, _c_ptr]),
    "matgptq_b200_slice": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_int, _c_int, _c_ptr]),
    "matgptq_b200_pack_qweights": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_int, _c_ptr]),
    "matgptq_b200_pack_qweights_host": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_int]),
    "matgptq_b200_unpack_qweights_host": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_int]),
    "matgptq_b200_reorder_scales": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr]),
    "matgptq_b200_reorder_scales_host": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64]),
    "matgptq_b200_device_status": (_c_int, [ctypes.POINTER(ctypes.c_int), _c_int]),
    "matgptq_b200_selftest_wait_timeout": (_c_int, [_c_int, _c_ptr, _c_ptr]),
    "matgptq_b200_dequantize": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_i64, _c_u32, _c_ptr]),
}

_lib = None


def lib_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library once and declare every signature. Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} not found: the CUDA library of matgptq_b200 is not built. "
            "Run `python -m matgptq_b200.build` (needs nvcc); there is no CPU fallback."
        )
    lib = ctypes.CDLL(_LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def device_status(reset: bool = True) -> int:
    """First failure code recorded by a kernel on the current device (0 = none); synchronises."""
    out = ctypes.c_int(0)
    check(load().matgptq_b200_device_status(ctypes.byref(out), 1 if reset else 0), "device_status")
    return out.value


def check(status: int, what: str) -> None:
    """Turn a non-zero status into the RuntimeError the reference's TORCH_CHECKs raise."""
    if status != OK:
        msg = load().matgptq_b200_strerror(status).decode()
        raise RuntimeError(f"{what}: {msg} (status {status})")
