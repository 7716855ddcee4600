"""ctypes binding of libnf4_b200.so (the C ABI declared in include/nf4_b200.h).

The library is the only compute path: there is no CPU or PyTorch fallback.  If the shared
object is missing or a call returns a non-zero status, a RuntimeError is raised.
"""

from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnf4_b200.so")

NF4_F32, NF4_F16, NF4_BF16 = 0, 1, 2
PATH_GEMV, PATH_GEMM, PATH_GEMV_SLABS, PATH_GENERIC = 1, 2, 3, 4
HAS_SWIGLU_HALVES = True   # epilogue 2 of nf4_b200_gemv_decode

_c_i64 = ctypes.c_int64
_c_int = ctypes.c_int
_c_ptr = ctypes.c_void_p

# name -> (restype, argtypes); must list every symbol include/nf4_b200.h declares
SIGNATURES = {
    "nf4_b200_version": (_c_int, []),
    "nf4_b200_last_error": (_c_int, [ctypes.c_char_p, _c_int]),
    "nf4_b200_last_linear_path": (_c_int, []),
    "nf4_b200_quantize": (_c_int, [_c_ptr, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "nf4_b200_dequantize": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_ptr, _c_int, _c_ptr]),
    "nf4_b200_linear": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_ptr, _c_ptr,
                                 _c_int, _c_ptr, _c_i64, _c_ptr]),
    "nf4_b200_linear_workspace_bytes": (_c_i64, [_c_i64, _c_i64, _c_i64, _c_int]),
    "nf4_b200_gemv": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_int, _c_ptr]),
    "nf4_b200_gemm": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_int,
                               _c_ptr, _c_i64, _c_ptr]),
    "nf4_b200_gemv_decode_next_weight": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64]),
    "nf4_b200_gemm_workspace_bytes": (_c_i64, [_c_i64, _c_i64, _c_i64]),
    "nf4_b200_gemm_decode": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_int,
                                      _c_ptr, _c_i64, _c_int, _c_ptr]),
    "nf4_b200_linear_generic": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_ptr,
                                         _c_ptr, _c_int, _c_ptr]),
    "nf4_b200_device_error": (_c_int, [_c_ptr]),
    "nf4_b200_device_error_clear": (_c_int, []),
    "nf4_b200_dq_quantize": (_c_int, [_c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "nf4_b200_dq_dequantize": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr]),
    "nf4_b200_linear_dq_workspace_bytes": (_c_i64, [_c_i64, _c_i64]),
    "nf4_b200_linear_dq": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr,
                                    _c_ptr, _c_int, _c_ptr, _c_i64, _c_ptr]),
    "nf4_b200_gemv_fused": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr,
                                     _c_int, _c_ptr]),
    "nf4_b200_gemv_decode": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_int, _c_ptr,
                                      ctypes.c_float, _c_int, _c_int, _c_ptr]),
    "nf4_b200_gemv_decode_fits": (_c_int, [_c_i64, _c_i64, _c_i64, _c_int]),
    "nf4_b200_rmsnorm": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, ctypes.c_float, _c_ptr]),
    "nf4_b200_rope_append": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_int, _c_int, _c_i64,
                                      ctypes.c_float, _c_ptr]),
    "nf4_b200_rope_prefill": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_int, _c_int, _c_i64,
                              ctypes.c_float, _c_ptr]),
    "nf4_b200_attn_decode_workspace_bytes": (_c_i64, [_c_i64, _c_int, _c_int]),
    "nf4_b200_attn_decode": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_int, _c_int,
                                      _c_i64, _c_int, _c_ptr]),
    "nf4_b200_attn_decode_fused": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_int,
                                            _c_int, _c_i64, _c_int, ctypes.c_float, _c_int, _c_ptr]),
    "nf4_b200_attn_decode_static": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_int, _c_int,
                                             _c_i64, _c_int, _c_ptr]),
    "nf4_b200_attn_decode_static_max_bytes": (_c_i64, []),
    "nf4_b200_silu_mul": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_ptr]),
    "nf4_b200_add": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr]),
    "nf4_b200_embed": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr]),
    "nf4_b200_argmax": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_ptr]),
    "nf4_b200_tp_allreduce_buffer_bytes": (_c_i64, [_c_i64]),
    "nf4_b200_tp_allreduce": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_i64, _c_int, _c_int, _c_int, _c_ptr]),
    "nf4_b200_tp_allreduce_emulated": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_i64, _c_int, _c_ptr]),
}

_lib = None


class NF4LibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NF4LibraryError(
                f"{LIB_PATH} is missing: build it with lightning-thunder_b200/csrc/build.sh "
                "(there is no fallback path for the NF4 kernels)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    load().nf4_b200_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def device_error():
    """(code, block, stage, count) of the first in-kernel wait that ran out; synchronises."""
    out = (ctypes.c_uint * 4)()
    check(load().nf4_b200_device_error(out), "nf4_b200_device_error")
    return tuple(out)


def device_error_clear() -> None:
    """Sets the (sticky) status words back to "no error"; synchronises."""
    check(load().nf4_b200_device_error_clear(), "nf4_b200_device_error_clear")


def check(status: int, what: str) -> None:
    if status != 0:
        raise NF4LibraryError(f"{what} failed with status {status}: {last_error()}")
