"""CPU tests of the oracle: C restatement vs numpy restatement vs the committed golden vectors."""

import json
import os

import numpy as np
import pytest

import oracle
from helpers import bf16_bits, seeded_act, seeded_weight, sha256

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _hex(a):
    return np.ascontiguousarray(a).tobytes().hex()


def test_nf4_table_invariants():
    from nf4_b200 import codebook

    codebook.check_nf4_table()
    d = codebook.dq_code256()
    assert len(d) == 256 and all(a < b for a, b in zip(d, d[1:]))
    assert d[0] == -1.0 and d[128] == 0.0 and d[255] == 1.0


def test_edge_case_goldens(nf4_code_np):
    with open(os.path.join(GOLDEN, "edge_cases.json")) as f:
        cases = json.load(f)
    assert set(cases) >= {"zero_block", "negative_extreme", "code_points", "midpoints", "numel4", "numel1", "odd_numel_131"}
    for name, c in cases.items():
        w = np.frombuffer(bytes.fromhex(c["w_f32_hex"]), dtype=np.float32)
        packed, absmax = oracle.quantize(w, nf4_code_np, 64)
        assert _hex(packed) == c["packed_hex"], name
        assert _hex(absmax) == c["absmax_hex"], name
        deq = oracle.dequantize(packed, absmax, nf4_code_np, w.size, 64, out="f32")
        assert _hex(deq) == c["dequant_f32_hex"], name
        # the independent numpy restatement agrees bit for bit
        p2, a2 = oracle.numpy_quantize(w, nf4_code_np, 64)
        assert np.array_equal(p2, packed), name
        assert np.array_equal(a2, absmax), name
        assert np.array_equal(oracle.numpy_dequantize(packed, absmax, nf4_code_np, w.size, 64), deq), name


def test_edge_case_semantics(nf4_code_np):
    # all-zero block -> index of level 0.0 (7) everywhere, absmax 0, dequant 0
    packed, absmax = oracle.quantize(np.zeros(64, np.float32), nf4_code_np, 64)
    assert absmax[0] == 0.0 and np.all(packed == 0x77)
    assert np.all(oracle.dequantize(packed, absmax, nf4_code_np, 64, 64, out="f32") == 0.0)
    # negative extreme maps to index 0, positive extreme to 15; high nibble holds the even element
    w = np.zeros(64, np.float32)
    w[0], w[1] = -2.0, 2.0
    packed, absmax = oracle.quantize(w, nf4_code_np, 64)
    assert absmax[0] == 2.0 and packed[0, 0] == 0x0F
    # exact levels times absmax survive a round trip
    w = (nf4_code_np * 3.0).astype(np.float32)
    w = np.concatenate([w, np.zeros(48, np.float32)])
    packed, absmax = oracle.quantize(w, nf4_code_np, 64)
    idx = np.stack([packed[:, 0] >> 4, packed[:, 0] & 15], 1).reshape(-1)[:16]
    assert list(idx) == list(range(16))
    # tie goes to the lower index: v exactly between level 7 (0.0) and a symmetric pair is impossible
    # for NF4, so build a table with an exact midpoint instead
    code = np.array([-1, -.9, -.8, -.7, -.6, -.5, -.4, 0, .25, .5, .6, .7, .8, .9, .95, 1], np.float32)
    v = np.array([1.0, 0.125] + [0.0] * 62, np.float32)
    packed, _ = oracle.quantize(v, code, 64)
    assert (packed[0, 0] & 15) == 7
    # shapes: [ceil(numel/2), 1] and ceil(numel/64)
    for n in (1, 2, 63, 64, 65, 131):
        p, a = oracle.quantize(np.ones(n, np.float32), nf4_code_np, 64)
        assert p.shape == ((n + 1) // 2, 1) and a.shape == ((n + 63) // 64,)
    p, a = oracle.quantize(np.zeros(0, np.float32), nf4_code_np, 64)
    assert p.shape == (0, 1) and a.shape == (0,)


@pytest.mark.parametrize("blocksize", [64, 128, 256])
def test_c_vs_numpy_random(nf4_code_np, blocksize):
    rng = np.random.default_rng(blocksize)
    w = (rng.standard_normal(64 * 1024 + 37) * 0.02).astype(np.float32)
    p1, a1 = oracle.quantize(w, nf4_code_np, blocksize)
    p2, a2 = oracle.numpy_quantize(w, nf4_code_np, blocksize)
    assert np.array_equal(p1, p2) and np.array_equal(a1, a2)
    d1 = oracle.dequantize(p1, a1, nf4_code_np, w.size, blocksize, out="f32")
    assert np.array_equal(d1, oracle.numpy_dequantize(p1, a1, nf4_code_np, w.size, blocksize))
    # quantize(dequantize(q)) is the identity on codes (idempotence) for complete blocks
    p3, a3 = oracle.quantize(d1, nf4_code_np, blocksize)
    full = (w.size // blocksize) * blocksize // 2
    assert np.array_equal(a3[: w.size // blocksize], a1[: w.size // blocksize])
    assert np.array_equal(p3[:full], p1[:full])


def test_bf16_input_path_matches_f32_path(nf4_code_np):
    w = seeded_weight((256, 320), 5)
    p1, a1 = oracle.quantize(bf16_bits(w), nf4_code_np, 64)
    p2, a2 = oracle.quantize(w.float().numpy(), nf4_code_np, 64)
    assert np.array_equal(p1, p2) and np.array_equal(a1, a2)
    assert np.array_equal(oracle.bf16_bits_to_f32(bf16_bits(w)), w.float().numpy())
    assert np.array_equal(oracle.f32_to_bf16_bits(w.float().numpy()), bf16_bits(w))


def test_config1_golden(nf4_code_np):
    """The first benchmark configuration: W [4096,4096] N(0,0.02) bf16, x [16,4096] N(0,1), blocksize 64."""
    with open(os.path.join(GOLDEN, "config1.json")) as f:
        g = json.load(f)
    N, K = g["shape"]
    w = seeded_weight((N, K), g["seed_w"])
    x = seeded_act((16, K), g["seed_x"])
    assert sha256(bf16_bits(w)) == g["w_sha256"], "torch CPU generator changed: regenerate the golden file"
    assert sha256(bf16_bits(x)) == g["x_sha256"]
    packed, absmax = oracle.quantize(bf16_bits(w), nf4_code_np, 64)
    assert sha256(packed) == g["packed_sha256"]
    assert sha256(absmax) == g["absmax_sha256"]
    assert packed.reshape(-1)[:32].tobytes().hex() == g["packed_head_hex"]
    deq = oracle.dequantize(packed, absmax, nf4_code_np, N * K, 64, out="bf16")
    assert sha256(deq) == g["dequant_bf16_sha256"]
    y = oracle.linear_bf16(bf16_bits(x), packed, absmax, nf4_code_np, N, K, 64, mode=oracle.GEMV_MODE)   # the pinned regime
    assert sha256(y) == g["y_bf16_sha256"]
    xs = x.float().numpy().astype(np.float64)[:2]
    # regime "dequantize then matmul": float64 matmul on the bf16-rounded dequantised weight
    wd = oracle.bf16_bits_to_f32(deq).reshape(N, K).astype(np.float64)
    y0 = oracle.linear_bf16(bf16_bits(x[:2]), packed, absmax, nf4_code_np, N, K, 64, mode=oracle.REF_DEQUANT_MATMUL_MODE)
    assert np.allclose(oracle.bf16_bits_to_f32(y0).astype(np.float64), xs @ wd.T, rtol=1.6e-2, atol=1e-3)
    # regime "fused GEMV": levels rounded to bf16, scaled by the fp32 absmax
    lv = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(nf4_code_np)).astype(np.float64)
    pb = packed.reshape(-1)
    idx = np.stack([pb >> 4, pb & 15], 1).reshape(N, K)
    wg = lv[idx] * np.repeat(absmax.astype(np.float64), 64).reshape(N, K)
    assert np.allclose(oracle.bf16_bits_to_f32(y[:2]).astype(np.float64), xs @ wg.T, rtol=1.6e-2, atol=1e-3)
    # the tensor-core regime: the GEMV's weights rounded to bf16
    y2 = oracle.linear_bf16(bf16_bits(x[:2]), packed, absmax, nf4_code_np, N, K, 64, mode=oracle.GEMM_MODE)
    wg2 = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(wg.astype(np.float32))).astype(np.float64)
    assert np.allclose(oracle.bf16_bits_to_f32(y2).astype(np.float64), xs @ wg2.T, rtol=1.6e-2, atol=1e-3)
    # the regimes differ only by bf16 rounding noise of the weights (a few 1e-3 at K=4096)
    d = np.abs(oracle.bf16_bits_to_f32(y0).astype(np.float64) - oracle.bf16_bits_to_f32(y[:2]).astype(np.float64))
    assert d.max() < 0.1 and np.sqrt((d ** 2).mean()) < 1e-2
    # quantization error vs the original weight stays within the NF4 step (max gap/2 * absmax)
    err = np.abs(oracle.dequantize(packed, absmax, nf4_code_np, N * K, 64, out="f32") - w.float().numpy().reshape(-1))
    assert err.max() <= 0.16 * absmax.max() + 1e-6


def test_linear_f32_and_bias(nf4_code_np):
    rng = np.random.default_rng(3)
    N, K, M = 48, 192, 5
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    packed, absmax = oracle.quantize(w, nf4_code_np, 64)
    wd = oracle.dequantize(packed, absmax, nf4_code_np, N * K, 64, out="f32").reshape(N, K)
    y = oracle.linear_f32(x, packed, absmax, nf4_code_np, N, K, 64, bias=b)
    assert np.allclose(y, x.astype(np.float64) @ wd.astype(np.float64).T + b, rtol=1e-5, atol=1e-5)


def test_double_quant_roundtrip():
    from nf4_b200.codebook import dq_code256

    code256 = np.array(dq_code256(), np.float32)
    rng = np.random.default_rng(11)
    absmax = (np.abs(rng.standard_normal(1000)) * 0.02 + 0.03).astype(np.float32)
    u8, scale2, offset = oracle.dq_quantize(absmax, code256, 256)
    assert u8.shape == (1000,) and scale2.shape == (4,)
    assert offset == np.float32(absmax.astype(np.float64).sum() / 1000)
    back = oracle.dq_dequantize(u8, scale2, offset, code256, 256)
    # quadratic 8-bit table: worst-case step near +-1 is ~1/64 of the block scale
    assert np.max(np.abs(back - absmax)) <= scale2.max() / 60
    # constant absmax -> all residuals zero -> index of 0.0 and exact reconstruction
    u8, scale2, offset = oracle.dq_quantize(np.full(300, 0.5, np.float32), code256, 256)
    assert np.all(u8 == 128) and np.all(scale2 == 0)
    assert np.all(oracle.dq_dequantize(u8, scale2, offset, code256, 256) == 0.5)
