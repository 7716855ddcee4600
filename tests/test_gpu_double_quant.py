"""Double quantization of absmax (8-bit, blocks of 256) against the CPU oracle: bit-exact indices,
scales, offset and expanded absmax; the linear on a double-quantized weight within tolerance."""

import numpy as np
import pytest
import torch

import oracle
from helpers import bf16_bits, bits_to_bf16, seeded_act, seeded_weight

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K", [(4096, 4096), (1000, 512), (3, 64), (14336, 4096)])
def test_dq_bit_exact(nf4_code_np, N, K):
    import nf4_b200
    from nf4_b200 import functional
    from nf4_b200.codebook import dq_code256

    code256 = np.array(dq_code256(), np.float32)
    w = seeded_weight((N, K), N + K).cuda()
    packed, qs = nf4_b200.quantize_4bit(w)
    absmax = qs.absmax.cpu().numpy().copy()
    functional.compress_absmax(qs)
    assert qs.nested and qs.absmax.dtype == torch.uint8 and qs.state2.absmax.shape == ((absmax.size + 255) // 256,)
    u8, scale2, offset = oracle.dq_quantize(absmax, code256, 256)
    assert np.float32(qs.offset.item()) == np.float32(offset)
    assert np.array_equal(qs.state2.absmax.cpu().numpy(), scale2)
    assert np.array_equal(qs.absmax.cpu().numpy(), u8)
    back = functional.expand_absmax(qs).cpu().numpy()
    assert np.array_equal(back, oracle.dq_dequantize(u8, scale2, offset, code256, 256))
    # 8-bit absmax costs little accuracy: relative error of the scale below 1 %
    assert np.max(np.abs(back - absmax) / absmax.max()) < 1e-2


def test_dq_edge_cases():
    from nf4_b200 import functional
    from nf4_b200.codebook import dq_code256

    code256 = np.array(dq_code256(), np.float32)
    for am in (np.full(300, 0.5, np.float32), np.zeros(7, np.float32), np.array([1.0], np.float32),
               np.linspace(0.01, 3.0, 1025).astype(np.float32)):
        st = functional.QuantState(absmax=torch.from_numpy(am).cuda(), shape=(am.size * 64,), blocksize=64,
                                   code=functional.nf4_code("cuda"), dtype=torch.bfloat16)
        functional.compress_absmax(st)
        u8, scale2, offset = oracle.dq_quantize(am, code256, 256)
        assert np.array_equal(st.absmax.cpu().numpy(), u8)
        assert np.array_equal(st.state2.absmax.cpu().numpy(), scale2)
        assert np.float32(st.offset.item()) == np.float32(offset)


@pytest.mark.parametrize("M", [1, 16, 64])
def test_linear_on_double_quantized_weight(nf4_code_np, M):
    """The second benchmark configuration uses double-quantized weights: y against the oracle's linear on
    the oracle's expanded absmax."""
    import nf4_b200
    from nf4_b200.codebook import dq_code256

    code256 = np.array(dq_code256(), np.float32)
    N, K = 1024, 4096
    w = seeded_weight((N, K), 5)
    x = seeded_act((M, K), M + 9)
    packed, qs = nf4_b200.quantize_4bit(w.cuda(), compress_statistics=True)
    y = nf4_b200.matmul_4bit(x.cuda(), packed.t(), quant_state=qs)
    p_np, a_np = oracle.quantize(bf16_bits(w), nf4_code_np, 64)
    assert np.array_equal(packed.cpu().numpy(), p_np)
    u8, scale2, offset = oracle.dq_quantize(a_np, code256, 256)
    a2 = oracle.dq_dequantize(u8, scale2, offset, code256, 256)
    ref = bits_to_bf16(oracle.linear_bf16(bf16_bits(x), p_np, a2, nf4_code_np, N, K, 64)).float()
    torch.testing.assert_close(y.float().cpu(), ref, rtol=1.6e-2, atol=1e-2)
    deq = nf4_b200.dequantize_4bit(packed, qs)
    assert np.array_equal(bf16_bits(deq).reshape(-1), oracle.dequantize(p_np, a2, nf4_code_np, N * K, 64, out="bf16"))


@pytest.mark.parametrize("N,K", [(4096, 4096), (14336, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [1, 4, 16, 256])
def test_sweep_shapes_with_double_quant(nf4_code_np, M, N, K):
    """The weight shapes and activation-row counts of the linear sweep with double quantization ON: up to 16 rows
    the 8-bit absmax is expanded inside the fused GEMV (no workspace), above that it is expanded once and the
    tensor-core GEMM runs.  Output rows are sampled against the oracle's linear on the oracle's expanded absmax,
    in the kernel's own rounding mode and in the dequantize-then-matmul mode."""
    import nf4_b200
    from nf4_b200 import _lib
    from nf4_b200.codebook import dq_code256

    code256 = np.array(dq_code256(), np.float32)
    w = seeded_weight((N, K), N + K + 11)
    x = seeded_act((M, K), M + 21)
    packed, qs = nf4_b200.quantize_4bit(w.cuda(), compress_statistics=True)
    y = nf4_b200.matmul_4bit(x.cuda(), packed.t(), quant_state=qs)
    torch.cuda.synchronize()
    assert _lib.device_error()[0] == 0
    p_np, a_np = oracle.quantize(bf16_bits(w), nf4_code_np, 64)
    u8, scale2, offset = oracle.dq_quantize(a_np, code256, 256)
    assert np.array_equal(qs.absmax.cpu().numpy(), u8)
    a2 = oracle.dq_dequantize(u8, scale2, offset, code256, 256)
    rows = sorted(set([0, M - 1, M // 2] + ([17, 255] if M > 255 else [])))
    xs = x[rows]
    from test_gpu_linear import assert_close_to_reference_mode

    got = y[rows].float().cpu()
    ref = bits_to_bf16(oracle.linear_bf16(bf16_bits(xs), p_np, a2, nf4_code_np, N, K, 64, mode=oracle.linear_mode_for(M))).float()
    torch.testing.assert_close(got, ref, rtol=1.6e-2, atol=1e-2)
    ref0 = bits_to_bf16(oracle.linear_bf16(bf16_bits(xs), p_np, a2, nf4_code_np, N, K, 64, mode=oracle.REF_DEQUANT_MATMUL_MODE)).float()
    assert_close_to_reference_mode(got, ref0, K)


@pytest.mark.parametrize("M", [1, 16, 2048])
def test_output_head_shape_with_double_quant(nf4_code_np, M):
    """128256 x 4096 with double quantization on: sampled output columns (a slice of weight rows through the
    oracle -- the whole product would take the CPU minutes)."""
    import nf4_b200
    from nf4_b200.codebook import dq_code256

    code256 = np.array(dq_code256(), np.float32)
    N, K = 128256, 4096
    g = torch.Generator(device="cuda").manual_seed(4)
    w = (torch.randn((N, K), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn((M, K), device="cuda", generator=g).to(torch.bfloat16)
    packed, qs = nf4_b200.quantize_4bit(w, compress_statistics=True)
    y = nf4_b200.matmul_4bit(x, packed.t(), quant_state=qs)
    torch.cuda.synchronize()
    a2 = nf4_b200.functional.expand_absmax(qs).cpu().numpy()
    p_all = packed.cpu().numpy().reshape(N, K // 2)
    rows_x = sorted(set([0, M - 1, M // 3]))
    for r0 in (0, 64000, N - 256):                      # 256-row slices: first, middle, ragged end of the grid
        p_np = np.ascontiguousarray(p_all[r0:r0 + 256]).reshape(-1)
        a_np = np.ascontiguousarray(a2.reshape(N, K // 64)[r0:r0 + 256]).reshape(-1)
        from test_gpu_linear import assert_close_to_reference_mode

        got = y[rows_x][:, r0:r0 + 256].float().cpu()
        xb = bf16_bits(x[rows_x].cpu())
        ref = bits_to_bf16(oracle.linear_bf16(xb, p_np, a_np, nf4_code_np, 256, K, 64, mode=oracle.linear_mode_for(M))).float()
        torch.testing.assert_close(got, ref, rtol=1.6e-2, atol=1e-2)
        ref0 = bits_to_bf16(oracle.linear_bf16(xb, p_np, a_np, nf4_code_np, 256, K, 64, mode=oracle.REF_DEQUANT_MATMUL_MODE)).float()
        assert_close_to_reference_mode(got, ref0, K)
