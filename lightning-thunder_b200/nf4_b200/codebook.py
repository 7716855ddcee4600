"""Code tables of the NF4 path.

``NF4_LEVELS`` are the 16 values of the 4-bit NormalFloat data type as published in
Dettmers, Pagnoni, Holtzman, Zettlemoyer, "QLoRA: Efficient Finetuning of Quantized LLMs"
(2023), appendix E ("NormalFloat 4-bit data type"): quantiles of N(0,1) normalised to
[-1, 1] with an exact zero, seven negative and eight positive levels.  The reference passes
this table to its op at run time as ``quant_map`` (thunder/transforms/quantization.py:34,
89, 262), so every kernel here reads it from that argument and nothing depends on these
constants beyond the default that ``quantize_4bit`` attaches to a new ``QuantState``.

``NF4_SHA256`` is the sha256 of the 16 values as little-endian fp32; ``check_nf4_table``
verifies it and the structural invariants.

``dq_code256`` is the 256-entry signed table used for the optional double quantization of
absmax.  Double quantization does not exist in the reference (quantization.py:84 "TODO:
double quant support"), so the table is defined here: quadratic spacing (denser near 0),
strictly increasing, containing -1, 0 and +1 exactly.
"""

from __future__ import annotations

import hashlib
import struct

NF4_LEVELS = (
    -1.0,
    -0.6961928009986877,
    -0.5250730514526367,
    -0.39491748809814453,
    -0.28444138169288635,
    -0.18477343022823334,
    -0.09105003625154495,
    0.0,
    0.07958029955625534,
    0.16093020141124725,
    0.24611230194568634,
    0.33791524171829224,
    0.44070982933044434,
    0.5626170039176941,
    0.7229568362236023,
    1.0,
)

NF4_SHA256 = "8501941daa1b8a90ad1bbfeb632e5101b5dddbc4bb52d6e55abcfd777e60c06a"


def nf4_bytes() -> bytes:
    return struct.pack("<16f", *NF4_LEVELS)


def nf4_sha256() -> str:
    return hashlib.sha256(nf4_bytes()).hexdigest()


def check_nf4_table(levels=NF4_LEVELS) -> None:
    f32 = struct.unpack("<16f", struct.pack("<16f", *levels))
    assert len(f32) == 16
    assert all(a < b for a, b in zip(f32, f32[1:])), "levels must be strictly increasing"
    assert f32[0] == -1.0 and f32[7] == 0.0 and f32[15] == 1.0
    assert all(v < 0 for v in f32[:7]) and all(v > 0 for v in f32[8:])
    if tuple(levels) == NF4_LEVELS:
        assert nf4_sha256() == NF4_SHA256


def dq_code256():
    """256 fp32 values: i<128 -> -((128-i)/128)^2, i==128 -> 0, i>128 -> ((i-128)/127)^2."""
    out = []
    for i in range(256):
        if i < 128:
            t = (128 - i) / 128.0
            v = -(t * t)
        elif i == 128:
            v = 0.0
        else:
            t = (i - 128) / 127.0
            v = t * t
        out.append(struct.unpack("<f", struct.pack("<f", v))[0])
    return tuple(out)
