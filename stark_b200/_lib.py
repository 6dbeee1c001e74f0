"""ctypes binding of ``libstark_b200.so`` (the C ABI in ``include/stark_b200.h``).

The library is the product: there is no Python or CPU fallback.  If it has not been built, or a
call returns a non-zero status, this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libstark_b200.so"

ABI_VERSION = 1
HOST, DEVICE = 0, 1
BF16, F32 = 0, 1
PLANE_F32, PLANE_F16, PLANE_BF16 = 0, 1, 30
GGUF_Q8_0, GGUF_Q4_K = 8, 12

STATUS_NAMES = ["ok", "invalid_argument", "abi_mismatch", "context_limit", "cancelled", "unsupported",
                "out_of_memory", "io_failure", "device_failure", "reload_required", "busy", "invalid_state"]


class StarkB200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else "unknown"
        super().__init__(f"{where}: {name} ({status})")


class AffineDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "struct_size", "abi_version", "rows", "columns", "bits", "group", "plane_kind", "scale_layout",
        "plane_pitch", "location", "pair_halves", "reserved")]


_lib = None


def load() -> C.CDLL:
    """Load the shared library; raises if it is missing (build it with ``python -m stark_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(run `python -m stark_b200.build`); there is no fallback path")
    lib = C.CDLL(str(LIB_PATH))
    vp, u32, u64, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t
    sig = {
        "stark_b200_abi_version": (u32, []),
        "stark_b200_status_name": (C.c_char_p, [u32]),
        "stark_b200_device_count": (u32, [C.POINTER(C.c_int32)]),
        "stark_b200_set_device": (u32, [C.c_int32]),
        "stark_b200_device_malloc": (u32, [C.POINTER(vp), sz]),
        "stark_b200_device_free": (u32, [vp]),
        "stark_b200_memcpy_h2d": (u32, [vp, vp, sz, vp]),
        "stark_b200_memcpy_d2h": (u32, [vp, vp, sz, vp]),
        "stark_b200_stream_synchronize": (u32, [vp]),
        "stark_b200_take_device_error": (u32, [C.POINTER(u32)]),
        "stark_b200_qmatrix_create_affine": (u32, [vp, vp, vp, C.POINTER(AffineDesc), C.POINTER(vp)]),
        "stark_b200_qmatrix_create_gguf": (u32, [vp, u32, u32, u32, u32, C.POINTER(vp)]),
        "stark_b200_qmatrix_destroy": (u32, [C.POINTER(vp)]),
        "stark_b200_qmatrix_device_bytes": (u32, [vp, C.POINTER(u64)]),
        "stark_b200_qmatrix_unpack_codes": (u32, [vp, vp, sz]),
        "stark_b200_op_qmv": (u32, [vp, vp, vp, u32, u32, u32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.stark_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libstark_b200.so ABI version mismatch")
    _lib = lib
    return lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise StarkB200Error(status, where)
