"""Host-side mirror of the three bitsandbytes entry points the reference's NF4 path calls
(thunder/transforms/quantization.py:35-39, 63), backed by the sm_100a kernels:

    quantize_4bit(w, quant_type="nf4")            -> (packed uint8 [ceil(numel/2), 1], QuantState)
    QuantState(absmax, shape=, blocksize=, code=, quant_type="nf4", dtype=)
    matmul_4bit(x, qweight.t(), bias=, quant_state=)   -> x @ dequant(W).T + bias
    dequantize_4bit(packed, quant_state)          -> W in quant_state.dtype

Names, argument meaning and error behaviour follow those calls so that the reference's
transform can drive these functions unchanged.  Tensors must live on a CUDA device; there is
no CPU path.
"""

from __future__ import annotations

import ctypes
from collections.abc import Sequence

import torch

from . import _lib
from .codebook import NF4_LEVELS

_DTYPE_CODE = {torch.float32: _lib.NF4_F32, torch.float16: _lib.NF4_F16, torch.bfloat16: _lib.NF4_BF16}

_code_cache: dict = {}


def nf4_code(device) -> torch.Tensor:
    """The 16 NF4 levels as an fp32 tensor on `device` (one cached copy per device)."""
    device = torch.device(device)
    key = (device.type, device.index)
    t = _code_cache.get(key)
    if t is None:
        t = torch.tensor(NF4_LEVELS, dtype=torch.float32, device=device)
        _code_cache[key] = t
    return t


class QuantState:
    """Metadata of one NF4-quantized tensor; same fields the reference reads
    (thunder/transforms/quantization.py:90-101): absmax, shape, blocksize, code, dtype."""

    def __init__(self, absmax, shape=None, code=None, blocksize=64, quant_type="nf4", dtype=None):
        if quant_type != "nf4":
            raise NotImplementedError(f"quant_type {quant_type!r}: only 'nf4' is implemented")
        self.absmax = absmax
        self.shape = torch.Size(shape) if shape is not None else None
        self.code = code
        self.blocksize = blocksize
        self.quant_type = quant_type
        self.dtype = dtype
        self.nested = False

    def to(self, device):
        self.absmax = self.absmax.to(device)
        self.code = self.code.to(device)
        return self


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor (got device {t.device}); the NF4 kernels have no CPU path")


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def quantize_4bit(A: torch.Tensor, absmax=None, out=None, blocksize: int = 64, compress_statistics: bool = False,
                  quant_type: str = "nf4", quant_storage=torch.uint8):
    """Blockwise NF4 quantization of `A` (fp32/fp16/bf16, any shape).  Returns (packed, QuantState)."""
    if quant_type != "nf4":
        raise NotImplementedError(f"quant_type {quant_type!r}: only 'nf4' is implemented")
    if compress_statistics:
        raise NotImplementedError("compress_statistics: use nf4_b200.double_quant for nested absmax")
    if quant_storage != torch.uint8:
        raise NotImplementedError("quant_storage: only torch.uint8")
    if A.dtype not in _DTYPE_CODE:
        raise ValueError(f"quantize_4bit: unsupported dtype {A.dtype}")
    _require_cuda(A, "quantize_4bit input")
    A = A.contiguous()
    n = A.numel()
    with torch.cuda.device(A.device):
        if out is None:
            out = torch.empty(((n + 1) // 2, 1), dtype=torch.uint8, device=A.device)
        if absmax is None:
            absmax = torch.empty(((n + blocksize - 1) // blocksize,), dtype=torch.float32, device=A.device)
        code = nf4_code(A.device)
        lib = _lib.load()
        _lib.check(
            lib.nf4_b200_quantize(A.data_ptr(), n, _DTYPE_CODE[A.dtype], blocksize, code.data_ptr(), out.data_ptr(),
                                  absmax.data_ptr(), _stream_ptr(A.device)),
            "nf4_b200_quantize",
        )
    state = QuantState(absmax=absmax, shape=A.shape, dtype=A.dtype, blocksize=blocksize, code=code.clone(),
                       quant_type=quant_type)
    return out, state


def dequantize_4bit(A: torch.Tensor, quant_state: QuantState = None, absmax=None, out=None, blocksize: int = 64,
                    quant_type: str = "nf4"):
    """Inverse of quantize_4bit: returns a tensor of quant_state.shape / quant_state.dtype."""
    if quant_state is None:
        raise ValueError("dequantize_4bit needs a quant_state")
    _require_cuda(A, "dequantize_4bit input")
    shape = quant_state.shape
    n = 1
    for s in shape:
        n *= int(s)
    dtype = quant_state.dtype
    with torch.cuda.device(A.device):
        if out is None:
            out = torch.empty(tuple(shape), dtype=dtype, device=A.device)
        lib = _lib.load()
        _lib.check(
            lib.nf4_b200_dequantize(A.data_ptr(), quant_state.absmax.data_ptr(), quant_state.code.data_ptr(), n,
                                    quant_state.blocksize, out.data_ptr(), _DTYPE_CODE[dtype], _stream_ptr(A.device)),
            "nf4_b200_dequantize",
        )
    return out


def linear_nf4(x: torch.Tensor, packed: torch.Tensor, bias, absmax: torch.Tensor, code: torch.Tensor, blocksize: int,
               shape: Sequence[int], out=None) -> torch.Tensor:
    """y = x @ dequant(W).T + bias for W of logical `shape` = (N, K) stored as packed/absmax/code."""
    N, K = int(shape[0]), int(shape[1])
    if x.shape[-1] != K:
        raise RuntimeError(f"linear_nf4: x.shape={tuple(x.shape)} does not match weight shape {(N, K)}")
    if x.dtype not in _DTYPE_CODE:
        raise ValueError(f"linear_nf4: unsupported dtype {x.dtype}")
    _require_cuda(x, "linear_nf4 input")
    _require_cuda(packed, "linear_nf4 weight")
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty((*x.shape[:-1], N), dtype=x.dtype, device=x.device)
        lib = _lib.load()
        _lib.check(
            lib.nf4_b200_linear(x2.data_ptr(), M, K, packed.data_ptr(), absmax.data_ptr(), code.data_ptr(), N,
                                int(blocksize), bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                _DTYPE_CODE[x.dtype], None, 0, _stream_ptr(x.device)),
            "nf4_b200_linear",
        )
    return out


def matmul_4bit(A: torch.Tensor, B: torch.Tensor, quant_state: QuantState, out=None, bias=None) -> torch.Tensor:
    """A @ dequant(B) + bias with B = packed.t() (shape [1, N*K/2]) as the reference passes it
    (thunder/transforms/quantization.py:39); quant_state.shape = (N, K)."""
    if quant_state is None:
        raise ValueError("matmul_4bit needs a quant_state")
    return linear_nf4(A, B, bias, quant_state.absmax, quant_state.code, quant_state.blocksize, quant_state.shape, out=out)
