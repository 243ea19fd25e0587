"""ctypes binding of libtq_sm100.so (see include/tq_b200.h for the contract of every symbol).

There is deliberately no fallback: if the library is missing or a call fails, an exception is
raised.  The arithmetic of this package runs in the CUDA kernels or not at all.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libtq_sm100.so"

TQ_OK = 0
TQ_PATH_AUTO, TQ_PATH_EXACT, TQ_PATH_TENSOR = 0, 1, 2

# name -> (restype, argtypes); mirrors include/tq_b200.h one to one
SIGNATURES = {
    "tq_version": (c_int, []),
    "tq_last_error": (c_char_p, []),
    "tq_device_count": (c_int, []),
    "tq_kernel_launches": (c_int64, []),
    "tq_plan_create": (c_int, [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p)]),
    "tq_plan_destroy": (None, [c_void_p]),
    "tq_plan_set_path": (c_int, [c_void_p, c_int]),
    "tq_plan_has_tensor_path": (c_int, [c_void_p]),
    "tq_code_row_bytes": (c_int64, [c_void_p]),
    "tq_sign_row_bytes": (c_int64, [c_void_p]),
    "tq_quantize_scratch_bytes": (c_int64, [c_void_p, c_int64]),
    "tq_topk_scratch_bytes": (c_int64, [c_void_p, c_int, c_int, c_int64, c_int]),
    "tq_mse_quantize": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "tq_mse_quantize_noalloc": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "tq_mse_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "tq_prod_quantize": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_size_t, c_void_p]),
    "tq_prod_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "tq_score_broadcast": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                   c_void_p, c_void_p]),
    "tq_score_pairwise": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                  c_void_p, c_void_p]),
    "tq_score_batched": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_size_t,
                                 c_void_p]),
    "tq_score_cache": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_size_t,
                               c_void_p]),
    "tq_mse_append": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int,
                              c_void_p]),
    "tq_prod_append": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                               c_void_p, c_int, c_void_p]),
    "tq_decode_attention_scratch_bytes": (c_int64, [c_void_p, c_int, c_int, c_int64]),
    "tq_decode_attention": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_float, c_void_p, c_void_p, c_size_t,
                                    c_void_p]),
    "tq_topk_merge": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "tq_topk_merge_gathered": (c_int, [c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "tq_unpack_codes": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "tq_pack_codes": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "tq_unpack_signs": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "tq_pack_signs": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "tq_plan_last_recheck_rows": (c_int, [c_void_p, c_void_p, POINTER(c_int64)]),
    "tq_plan_set_wait_limit": (c_int, [c_void_p, c_int64]),
    "tq_plan_time_kernels": (c_int, [c_void_p, c_int]),
    "tq_plan_kernel_ms": (c_int, [c_void_p, c_int, c_void_p, c_int]),
    "tq_plan_status": (c_int, [c_void_p, c_void_p, POINTER(c_int64)]),
}

_lib = None


class TurboQuantNativeError(RuntimeError):
    """A call into libtq_sm100.so failed (the message comes from tq_last_error)."""


def library_path() -> str:
    return os.environ.get("TQ_LIB") or os.path.join(_PKG_DIR, LIB_NAME)


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise TurboQuantNativeError(
            f"{path} not found: build it with `python -m project_tensor_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.tq_version() != 100:
        raise TurboQuantNativeError(f"{path}: unexpected ABI version {lib.tq_version()}")
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != TQ_OK:
        msg = load().tq_last_error()
        raise TurboQuantNativeError(f"libtq_sm100 error {status}: {msg.decode() if msg else '?'}")
