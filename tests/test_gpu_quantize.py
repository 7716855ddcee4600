"""GPU parity of quantize / dequantize against the CPU oracle, through the C ABI (bit-exact)."""

import json
import os

import numpy as np
import pytest
import torch

import oracle
from helpers import bf16_bits, seeded_weight, sha256

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _quant_gpu(w_cpu, blocksize=64):
    import nf4_b200

    packed, qs = nf4_b200.quantize_4bit(w_cpu.cuda(), blocksize=blocksize)
    torch.cuda.synchronize()
    return packed, qs


def _oracle_input(w_cpu):
    if w_cpu.dtype == torch.bfloat16:
        return bf16_bits(w_cpu)
    return w_cpu.float().numpy()   # fp16 -> fp32 is exact


def test_library_is_loaded_and_device_is_b200():
    from nf4_b200 import _lib

    assert os.path.exists(_lib.LIB_PATH)
    assert torch.cuda.get_device_capability(0)[0] == 10


def test_config1_bit_exact(nf4_code_np):
    import nf4_b200

    with open(os.path.join(GOLDEN, "config1.json")) as f:
        g = json.load(f)
    N, K = g["shape"]
    w = seeded_weight((N, K), g["seed_w"])
    assert sha256(bf16_bits(w)) == g["w_sha256"]
    packed, qs = _quant_gpu(w)
    assert packed.shape == (N * K // 2, 1) and packed.dtype == torch.uint8
    assert qs.absmax.shape == (N * K // 64,) and qs.absmax.dtype == torch.float32
    assert tuple(qs.shape) == (N, K) and qs.blocksize == 64 and qs.dtype == torch.bfloat16
    assert qs.code.shape == (16,) and qs.code.dtype == torch.float32
    assert sha256(packed.cpu().numpy()) == g["packed_sha256"]
    assert sha256(qs.absmax.cpu().numpy()) == g["absmax_sha256"]
    deq = nf4_b200.dequantize_4bit(packed, qs)
    assert deq.shape == (N, K) and deq.dtype == torch.bfloat16
    assert sha256(bf16_bits(deq)) == g["dequant_bf16_sha256"]


def test_edge_case_goldens(nf4_code_np):
    import nf4_b200

    with open(os.path.join(GOLDEN, "edge_cases.json")) as f:
        cases = json.load(f)
    for name, c in cases.items():
        w = np.frombuffer(bytes.fromhex(c["w_f32_hex"]), dtype=np.float32).copy()
        packed, qs = _quant_gpu(torch.from_numpy(w))
        assert packed.cpu().numpy().tobytes().hex() == c["packed_hex"], name
        assert qs.absmax.cpu().numpy().tobytes().hex() == c["absmax_hex"], name
        deq = nf4_b200.dequantize_4bit(packed, qs)
        assert deq.cpu().numpy().tobytes().hex() == c["dequant_f32_hex"], name


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("numel", [4, 64, 8 * 64, 64 * 333 + 21, 1 << 20, (1 << 20) + 8])
def test_random_bit_exact(nf4_code_np, dtype, numel):
    import nf4_b200

    w = seeded_weight((numel,), numel, std=0.05, dtype=dtype)
    packed, qs = _quant_gpu(w)
    p_ref, a_ref = oracle.quantize(_oracle_input(w), nf4_code_np, 64)
    assert np.array_equal(packed.cpu().numpy(), p_ref)
    assert np.array_equal(qs.absmax.cpu().numpy(), a_ref)
    deq = nf4_b200.dequantize_4bit(packed, qs)
    ref32 = oracle.dequantize(p_ref, a_ref, nf4_code_np, numel, 64, out="f32")
    ref = torch.from_numpy(ref32).to(dtype)   # torch rounds to nearest even like the kernel
    assert torch.equal(deq.cpu().view(-1), ref)


@pytest.mark.parametrize("blocksize", [128, 256, 512, 1024, 2048, 4096])
def test_other_blocksizes(nf4_code_np, blocksize):
    import nf4_b200

    numel = 4096 * 37 + 100
    w = seeded_weight((numel,), blocksize, std=1.0)
    packed, qs = _quant_gpu(w, blocksize)
    p_ref, a_ref = oracle.quantize(bf16_bits(w), nf4_code_np, blocksize)
    assert np.array_equal(qs.absmax.cpu().numpy(), a_ref)
    assert np.array_equal(packed.cpu().numpy(), p_ref)
    deq = nf4_b200.dequantize_4bit(packed, qs)
    ref = oracle.dequantize(p_ref, a_ref, nf4_code_np, numel, blocksize, out="bf16")
    assert np.array_equal(bf16_bits(deq).reshape(-1), ref)


def test_unaligned_input_view(nf4_code_np):
    """A view that starts 2 bytes into an allocation takes the unaligned path and still matches."""
    import nf4_b200

    base = seeded_weight((64 * 50 + 1,), 99).cuda()
    w = base[1:]
    packed, qs = nf4_b200.quantize_4bit(w)
    p_ref, a_ref = oracle.quantize(bf16_bits(w.cpu()), nf4_code_np, 64)
    assert np.array_equal(packed.cpu().numpy(), p_ref) and np.array_equal(qs.absmax.cpu().numpy(), a_ref)


def test_exhaustive_levels_against_thresholds(nf4_code_np):
    """Every fp32 in a dense sweep of [-1,1] maps to the same index as the oracle's argmin:
    one block whose absmax is exactly 1.0 makes v = w."""
    import nf4_b200

    rng = np.random.default_rng(0)
    mids = ((nf4_code_np[:-1].astype(np.float64) + nf4_code_np[1:]) / 2).astype(np.float32)
    near = []
    for m in mids:   # +-64 ulps around each decision midpoint
        k = np.array([m], np.float32).view(np.int32)[0]
        near.append((np.arange(k - 64, k + 65, dtype=np.int32)).view(np.float32))
    vals = np.concatenate(near + [rng.uniform(-1, 1, 200000).astype(np.float32)])
    pad = (-len(vals)) % 63
    vals = np.concatenate([vals, np.zeros(pad, np.float32)]).reshape(-1, 63)
    w = np.concatenate([np.ones((vals.shape[0], 1), np.float32), vals], axis=1).reshape(-1)   # absmax = 1 per block
    packed, qs = _quant_gpu(torch.from_numpy(w))
    p_ref, a_ref = oracle.quantize(w, nf4_code_np, 64)
    assert np.all(a_ref == 1.0)
    assert np.array_equal(packed.cpu().numpy(), p_ref)


def test_division_near_thresholds_with_arbitrary_scales(nf4_code_np):
    """The kernel divides with its own reciprocal + FMA sequence: quotients within a few ulps of every
    decision point, for many block scales (not only 1.0), must still land on the oracle's index."""
    import nf4_b200

    rng = np.random.default_rng(42)
    mids = ((nf4_code_np[:-1].astype(np.float64) + nf4_code_np[1:]) / 2)
    blocks = []
    for scale in np.concatenate([rng.uniform(1e-3, 10.0, 300), 2.0 ** rng.integers(-90, 90, 40), [0.02, 0.0625, 3.0e-30, 1.0e30]]).astype(np.float32):
        for m in mids:
            center = np.float32(m * np.float64(scale))
            k = np.array([center], np.float32).view(np.int32)[0]
            cand = np.arange(k - 31, k + 32, dtype=np.int32).view(np.float32)      # 63 neighbours
            cand = np.clip(cand, -scale, scale)
            blocks.append(np.concatenate([[scale], cand]).astype(np.float32))
    w = np.concatenate(blocks)
    packed, qs = _quant_gpu(torch.from_numpy(w))
    p_ref, a_ref = oracle.quantize(w, nf4_code_np, 64)
    assert np.array_equal(qs.absmax.cpu().numpy(), a_ref)
    assert np.array_equal(packed.cpu().numpy(), p_ref)


def test_full_size_properties(nf4_code_np):
    """Size-independent checks on the largest weight of the metric's model (lm_head 128256x4096):
    idempotence of quantize(dequantize(.)) and a checksum of per-slice checksums vs the oracle."""
    import nf4_b200

    N, K = 128256, 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    w = (torch.randn((N, K), generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    packed, qs = nf4_b200.quantize_4bit(w)
    deq = nf4_b200.dequantize_4bit(packed, qs)
    packed2, qs2 = nf4_b200.quantize_4bit(deq)
    assert torch.equal(qs2.absmax, qs.absmax)   # the block extreme maps to +-1 exactly
    assert torch.equal(packed2, packed)
    # |w - deq| <= half the widest level gap times absmax
    err = (w.float() - deq.float()).abs().view(-1, 64).amax(dim=1)
    assert bool((err <= 0.16 * qs.absmax + 1e-6).all())
    # oracle on three slices of 1M elements
    for start in (0, (N * K // 2) & ~63, N * K - (1 << 20)):
        sl = w.view(-1)[start : start + (1 << 20)].cpu()
        p_ref, a_ref = oracle.quantize(bf16_bits(sl), nf4_code_np, 64)
        assert np.array_equal(packed.view(-1)[start // 2 : start // 2 + (1 << 19)].cpu().numpy(), p_ref.reshape(-1))
        assert np.array_equal(qs.absmax[start // 64 : start // 64 + (1 << 14)].cpu().numpy(), a_ref)
