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
    """Config 2 of the benchmark set uses double-quantized weights: y against the oracle's linear on
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
