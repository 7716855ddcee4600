"""B200-native NF4 (4-bit NormalFloat) weight-only quantized linear: hand-written sm_100a
kernels behind a C ABI, plus the host code that mirrors the reference's interface."""

from . import codebook
from .functional import QuantState, dequantize_4bit, linear_nf4, matmul_4bit, nf4_code, quantize_4bit

__all__ = ["codebook", "QuantState", "dequantize_4bit", "linear_nf4", "matmul_4bit", "nf4_code", "quantize_4bit"]
