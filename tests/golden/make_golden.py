"""Regenerates tests/golden/*.json from the CPU oracle.

The reference pins no bytes for the NF4 path (its tests compare bitsandbytes with itself), so
these vectors freeze the oracle's output on seeded inputs: a change in the oracle, in the code
table or in torch's CPU generator shows up as a checksum mismatch.  Run from the repo root:

    python tests/golden/make_golden.py
"""

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "lightning-thunder_b200"), os.path.join(ROOT, "tests")]

import oracle  # noqa: E402
from helpers import bf16_bits, seeded_act, seeded_weight, sha256  # noqa: E402
from nf4_b200.codebook import NF4_LEVELS, nf4_sha256  # noqa: E402

CODE = np.array(NF4_LEVELS, dtype=np.float32)


def config1(seed_w=1234, seed_x=4321):
    """W bf16 [4096,4096] ~ N(0,0.02), x bf16 [16,4096] ~ N(0,1), blocksize 64, no double quant."""
    N = K = 4096
    w = seeded_weight((N, K), seed_w)
    x = seeded_act((16, K), seed_x)
    wb = bf16_bits(w)
    packed, absmax = oracle.quantize(wb, CODE, 64)
    deq = oracle.dequantize(packed, absmax, CODE, N * K, 64, out="bf16")
    y = oracle.linear_bf16(bf16_bits(x), packed, absmax, CODE, N, K, 64, mode=oracle.GEMV_MODE)
    return {
        "name": "config1",
        "seed_w": seed_w,
        "seed_x": seed_x,
        "shape": [N, K],
        "blocksize": 64,
        "nf4_table_sha256": nf4_sha256(),
        "w_sha256": sha256(wb),
        "x_sha256": sha256(bf16_bits(x)),
        "packed_sha256": sha256(packed),
        "absmax_sha256": sha256(absmax),
        "dequant_bf16_sha256": sha256(deq),
        "packed_head_hex": packed.reshape(-1)[:32].tobytes().hex(),
        "absmax_head_hex": absmax[:8].tobytes().hex(),
        "y_bf16_row0_head_hex": y[0, :32].tobytes().hex(),
        "y_bf16_sha256": sha256(y),
    }


def edge_cases():
    rng = np.random.default_rng(7)
    cases = {}
    # all-zero block, a block whose extreme is negative, exact code points, tiny and odd tensors
    z = np.zeros(128, np.float32)
    z[64:] = rng.standard_normal(64).astype(np.float32)
    cases["zero_block"] = z
    neg = rng.standard_normal(64).astype(np.float32) * 0.1
    neg[17] = -3.0
    cases["negative_extreme"] = neg
    cases["code_points"] = np.concatenate([CODE * 0.5, CODE * 2.0, CODE, CODE * 0.25]).astype(np.float32)
    mid = ((CODE[:-1].astype(np.float64) + CODE[1:].astype(np.float64)) / 2).astype(np.float32)
    cases["midpoints"] = np.concatenate([mid, [1.0], mid * 1.0000001, [-1.0], mid * 0.9999999, [1.0], np.zeros(17)]).astype(np.float32)
    cases["numel4"] = np.array([0.3, -0.7, 0.05, 0.0], np.float32)
    cases["numel1"] = np.array([-2.5], np.float32)
    cases["odd_numel_131"] = rng.standard_normal(131).astype(np.float32)
    out = {}
    for name, w in cases.items():
        packed, absmax = oracle.quantize(w, CODE, 64)
        out[name] = {
            "w_f32_hex": w.tobytes().hex(),
            "packed_hex": packed.tobytes().hex(),
            "absmax_hex": absmax.tobytes().hex(),
            "dequant_f32_hex": oracle.dequantize(packed, absmax, CODE, w.size, 64, out="f32").tobytes().hex(),
        }
    return out


if __name__ == "__main__":
    with open(os.path.join(HERE, "config1.json"), "w") as f:
        json.dump(config1(), f, indent=1)
    with open(os.path.join(HERE, "edge_cases.json"), "w") as f:
        json.dump(edge_cases(), f, indent=1)
    print("wrote", os.listdir(HERE))
