"""The shared library loads without a GPU and exports every symbol include/*.h declares."""

import ctypes
import glob
import os
import re

from conftest import ROOT


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(nf4_b200_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    from nf4_b200 import _lib

    lib = _lib.load()
    decl = declared_symbols()
    assert decl, "no declarations found in include/*.h"
    for name in decl:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    # and the ctypes table covers the header exactly
    assert set(_lib.SIGNATURES) == decl


def test_argument_validation_needs_no_gpu():
    """Host-side checks run before any CUDA call: bad arguments give status codes + messages."""
    from nf4_b200 import _lib

    lib = _lib.load()
    assert lib.nf4_b200_version() >= 100
    rc = lib.nf4_b200_quantize(None, -1, 2, 64, None, None, None, None)
    assert rc == 1 and "numel" in _lib.last_error()
    rc = lib.nf4_b200_quantize(None, 128, 2, 48, None, None, None, None)
    assert rc == 1 and "blocksize" in _lib.last_error()
    rc = lib.nf4_b200_quantize(None, 128, 2, 64, None, None, None, None)
    assert rc == 1 and "null" in _lib.last_error()
    assert lib.nf4_b200_quantize(None, 0, 2, 64, None, None, None, None) == 0   # empty tensor is a no-op
    rc = lib.nf4_b200_gemv(ctypes.c_void_p(256), 17, 64, ctypes.c_void_p(256), ctypes.c_void_p(256),
                           ctypes.c_void_p(256), 8, None, ctypes.c_void_p(256), 2, None)
    assert rc == 1 and "M=17" in _lib.last_error()
    rc = lib.nf4_b200_gemv(ctypes.c_void_p(256), 1, 100, ctypes.c_void_p(256), ctypes.c_void_p(256),
                           ctypes.c_void_p(256), 8, None, ctypes.c_void_p(256), 2, None)
    assert rc == 1 and "multiple of 64" in _lib.last_error()
    rc = lib.nf4_b200_linear(ctypes.c_void_p(256), 1, 64, ctypes.c_void_p(256), ctypes.c_void_p(256),
                             ctypes.c_void_p(256), 8, 64, None, ctypes.c_void_p(256), 7, None, 0, None)
    assert rc == 1 and "dtype" in _lib.last_error()
    assert lib.nf4_b200_linear_workspace_bytes(16, 4096, 4096, 2) >= 0


def test_functional_refuses_cpu_tensors():
    import pytest
    import torch

    import nf4_b200

    with pytest.raises(RuntimeError, match="CUDA"):
        nf4_b200.quantize_4bit(torch.zeros(64, dtype=torch.bfloat16))


def test_tensor_core_entry_points_validate_arguments_without_a_gpu():
    """Argument checks come before any device call, so they can be exercised on a CPU-only machine."""
    import ctypes

    from nf4_b200 import _lib

    lib = _lib.load()
    p = ctypes.c_void_p(256)
    rc = lib.nf4_b200_gemm_decode(p, 16, 128, p, p, p, 7, None, p, 1, None, 0, 0, None)
    assert rc == 1 and "epilogue" in _lib.last_error()           # SwiGLU needs an even N
    rc = lib.nf4_b200_gemm_decode(p, 16, 128, p, p, p, 8, p, p, 1, None, 0, 0, None)
    assert rc == 1 and "epilogue" in _lib.last_error()           # ... and no residual
    rc = lib.nf4_b200_gemm_decode(p, 16, 100, p, p, p, 8, None, p, 0, None, 0, 0, None)
    assert rc == 1 and "multiple of 64" in _lib.last_error()
    assert lib.nf4_b200_gemv_decode_next_weight(p, p, 8, 100) == 1
    assert lib.nf4_b200_gemv_decode_next_weight(p, p, 4096, 4096) == 0
    assert lib.nf4_b200_gemv_decode_next_weight(None, None, 0, 0) == 0      # clears the pending hint
    # K-split planning: decode shapes with few 128-row tiles split; tall tiles only with long K ranges
    assert lib.nf4_b200_gemm_workspace_bytes(16, 4096, 4096) > 0
    assert lib.nf4_b200_gemm_workspace_bytes(16, 128256, 4096) == 0
    assert lib.nf4_b200_gemm_workspace_bytes(256, 4096, 4096) == 0
    assert lib.nf4_b200_gemm_workspace_bytes(256, 4096, 14336) > 0
    assert lib.nf4_b200_gemm_workspace_bytes(2048, 14336, 4096) == 0
