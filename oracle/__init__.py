"""CPU oracle for the NF4 quantized-linear path -- TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import this
package; the product (the CUDA library and its host code) never does.

Two independent restatements of the same published algorithm live here:

* ``nf4_oracle.c`` compiled to ``oracle/_ref/libnf4_oracle.so`` (OpenMP; also the timed CPU
  baseline) and wrapped below with numpy arrays;
* ``numpy_*`` functions, a vectorised numpy restatement used to cross-check the C one.

Tensor contract followed (thunder/transforms/quantization.py:29-39, 53-63, 86-101): codes are
uint8 ``[ceil(numel/2), 1]``, absmax is fp32 ``[ceil(numel/blocksize)]``, the 16-entry fp32
table is an input.  PARITY UNPINNED: the reference pins no bytes for this path and
bitsandbytes (the library it calls) is not available; see the header of ``nf4_oracle.c`` for
the decisions this restatement fixes.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libnf4_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile nf4_oracle.c with the committed Makefile (needs gcc)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(os.path.join(_HERE, "nf4_oracle.c")):
        subprocess.check_call(["make", "-C", _HERE, "-B", "_ref/libnf4_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16); finite inputs."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------------------- C oracle wrappers


def quantize(w: np.ndarray, code16: np.ndarray, blocksize: int = 64):
    """w: fp32 array, or uint16 array of bf16 bit patterns.  Returns (packed [nbytes,1] u8, absmax f32)."""
    code16 = np.ascontiguousarray(code16, dtype=np.float32)
    flat = np.ascontiguousarray(w).reshape(-1)
    numel = flat.size
    packed = np.zeros(((numel + 1) // 2, 1), dtype=np.uint8)
    absmax = np.zeros(((numel + blocksize - 1) // blocksize,), dtype=np.float32)
    if numel == 0:
        return packed, absmax
    if flat.dtype == np.uint16:
        fn = lib().nf4_oracle_quantize_bf16
    elif flat.dtype == np.float32:
        fn = lib().nf4_oracle_quantize_f32
    else:
        raise TypeError(f"oracle.quantize takes fp32 or bf16-bits(uint16), got {flat.dtype}")
    fn(_p(flat), ctypes.c_int64(numel), ctypes.c_int(blocksize), _p(code16), _p(packed), _p(absmax))
    return packed, absmax


def dequantize(packed: np.ndarray, absmax: np.ndarray, code16: np.ndarray, numel: int, blocksize: int = 64,
               out: str = "bf16") -> np.ndarray:
    """Returns uint16 bf16 bit patterns (out="bf16") or fp32 values (out="f32"), flat [numel]."""
    code16 = np.ascontiguousarray(code16, dtype=np.float32)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    absmax = np.ascontiguousarray(absmax, dtype=np.float32)
    if out == "bf16":
        res = np.zeros((numel,), dtype=np.uint16)
        fn = lib().nf4_oracle_dequantize_bf16
    else:
        res = np.zeros((numel,), dtype=np.float32)
        fn = lib().nf4_oracle_dequantize_f32
    if numel:
        fn(_p(packed), _p(absmax), _p(code16), ctypes.c_int64(numel), ctypes.c_int(blocksize), _p(res))
    return res


REF_DEQUANT_MATMUL_MODE, GEMV_MODE, GEMM_MODE = 0, 1, 2


def linear_mode_for(M: int) -> int:
    """The regime the library takes for M bf16 activation rows (fused GEMV up to 16 rows, tensor-core
    GEMM above)."""
    return GEMV_MODE if M <= 16 else GEMM_MODE


def linear_bf16(x_bits: np.ndarray, packed, absmax, code16, N: int, K: int, blocksize: int = 64, bias_bits=None,
                mode=None):
    """x_bits: uint16 [M,K] bf16 bit patterns.  Returns uint16 [M,N] bf16 bit patterns.
    mode: REF_DEQUANT_MATMUL_MODE (weight = bf16(level * absmax)), GEMV_MODE (levels rounded to bf16,
    block sums scaled in fp32), GEMM_MODE (weight = bf16(bf16(level) * absmax)); default = the
    regime the library takes for this M."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16).reshape(-1, K)
    M = x_bits.shape[0]
    code16 = np.ascontiguousarray(code16, dtype=np.float32)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    absmax = np.ascontiguousarray(absmax, dtype=np.float32)
    y = np.zeros((M, N), dtype=np.uint16)
    b = None if bias_bits is None else np.ascontiguousarray(bias_bits, dtype=np.uint16)
    lib().nf4_oracle_linear_bf16(_p(x_bits), ctypes.c_int64(M), ctypes.c_int64(K), _p(packed), _p(absmax),
                                 _p(code16), ctypes.c_int64(N), ctypes.c_int(blocksize),
                                 _p(b) if b is not None else None, _p(y),
                                 ctypes.c_int(linear_mode_for(M) if mode is None else mode))
    return y


def linear_f32(x: np.ndarray, packed, absmax, code16, N: int, K: int, blocksize: int = 64, bias=None):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, K)
    M = x.shape[0]
    code16 = np.ascontiguousarray(code16, dtype=np.float32)
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    absmax = np.ascontiguousarray(absmax, dtype=np.float32)
    y = np.zeros((M, N), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().nf4_oracle_linear_f32(_p(x), ctypes.c_int64(M), ctypes.c_int64(K), _p(packed), _p(absmax), _p(code16),
                                ctypes.c_int64(N), ctypes.c_int(blocksize), _p(b) if b is not None else None, _p(y))
    return y


def dq_quantize(absmax: np.ndarray, code256: np.ndarray, blocksize2: int = 256):
    """Double quantization of absmax.  Returns (u8 [nblocks], scale2 f32 [ceil(nblocks/256)], offset f32 scalar)."""
    absmax = np.ascontiguousarray(absmax, dtype=np.float32)
    code256 = np.ascontiguousarray(code256, dtype=np.float32)
    n = absmax.size
    u8 = np.zeros((n,), dtype=np.uint8)
    scale2 = np.zeros(((n + blocksize2 - 1) // blocksize2,), dtype=np.float32)
    offset = np.zeros((1,), dtype=np.float32)
    lib().nf4_oracle_dq_quantize(_p(absmax), ctypes.c_int64(n), ctypes.c_int(blocksize2), _p(code256), _p(u8),
                                 _p(scale2), _p(offset))
    return u8, scale2, offset[0]


def dq_dequantize(u8: np.ndarray, scale2: np.ndarray, offset, code256: np.ndarray, blocksize2: int = 256):
    u8 = np.ascontiguousarray(u8, dtype=np.uint8)
    scale2 = np.ascontiguousarray(scale2, dtype=np.float32)
    code256 = np.ascontiguousarray(code256, dtype=np.float32)
    out = np.zeros((u8.size,), dtype=np.float32)
    lib().nf4_oracle_dq_dequantize(_p(u8), _p(scale2), ctypes.c_float(float(offset)), _p(code256),
                                   ctypes.c_int64(u8.size), ctypes.c_int(blocksize2), _p(out))
    return out


# ------------------------------------------------------------------------- numpy restatement


def numpy_quantize(w_f32: np.ndarray, code16: np.ndarray, blocksize: int = 64):
    """Same algorithm, vectorised: absmax per block, fp32 division, argmin over the 16 levels
    (numpy's argmin returns the first minimum = the lower index on a tie), high nibble first."""
    code16 = np.asarray(code16, dtype=np.float32)
    flat = np.ascontiguousarray(w_f32, dtype=np.float32).reshape(-1)
    numel = flat.size
    nblocks = (numel + blocksize - 1) // blocksize
    pad = nblocks * blocksize - numel
    blocks = np.concatenate([flat, np.zeros(pad, np.float32)]).reshape(nblocks, blocksize)
    absmax = np.abs(blocks).max(axis=1).astype(np.float32) if nblocks else np.zeros(0, np.float32)
    zidx = int(np.where(code16 == 0.0)[0][0])
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (blocks / absmax[:, None]).astype(np.float32)
    idx = np.abs(v[..., None] - code16[None, None, :]).astype(np.float32).argmin(axis=-1).astype(np.uint8)
    idx[absmax == 0.0, :] = zidx
    idx = idx.reshape(-1)[:numel]
    if numel & 1:
        idx = np.concatenate([idx, np.zeros(1, np.uint8)])
    packed = ((idx[0::2] << 4) | idx[1::2]).astype(np.uint8).reshape(-1, 1)
    return packed, absmax


def numpy_dequantize(packed, absmax, code16, numel: int, blocksize: int = 64) -> np.ndarray:
    code16 = np.asarray(code16, dtype=np.float32)
    b = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    idx = np.stack([b >> 4, b & 15], axis=1).reshape(-1)[:numel]
    scale = np.repeat(np.asarray(absmax, dtype=np.float32), blocksize)[:numel]
    return (code16[idx] * scale).astype(np.float32)
