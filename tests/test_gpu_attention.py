"""The decode-step attention kernels (tensor-core tiles of 16 cached positions, split along the sequence)
against a plain PyTorch fp32 restatement: every group size, ragged contexts per batch row, context
lengths around the tile size, more splits than positions, and the fused rotary + append form.
torch is only the checker."""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DH = 128


def _rope(x, pos, theta):
    # x [B, H, Dh], interleaved pairs; result rounded to bf16 like the kernels do
    B, H, Dh = x.shape
    i = torch.arange(Dh // 2, device=x.device, dtype=torch.float32)
    ang = pos.float().view(B, 1, 1) * torch.pow(torch.tensor(theta, device=x.device), -2.0 * i / Dh).view(1, 1, -1)
    xr = x.float().view(B, H, Dh // 2, 2)
    c, s = torch.cos(ang), torch.sin(ang)
    out = torch.stack([xr[..., 0] * c - xr[..., 1] * s, xr[..., 0] * s + xr[..., 1] * c], dim=-1)
    return out.view(B, H, Dh).to(torch.bfloat16)


def _reference(q, k_cache, v_cache, lens):
    """q [B, Hq, Dh] bf16, caches [B, Hkv, S, Dh] bf16, lens[b] positions attended."""
    B, Hq, _ = q.shape
    Hkv = k_cache.shape[1]
    G = Hq // Hkv
    out = torch.zeros((B, Hq, DH), device=q.device)
    for b in range(B):
        n = int(lens[b])
        for h in range(Hq):
            kk, vv = k_cache[b, h // G, :n].float(), v_cache[b, h // G, :n].float()
            p = torch.softmax((kk @ q[b, h].float()) / math.sqrt(DH), dim=0)
            out[b, h] = p @ vv
    return out


@pytest.mark.parametrize("G", [1, 2, 4, 8])
@pytest.mark.parametrize("nsplit", [1, 3, 8])
def test_attention_over_the_cache(G, nsplit):
    from nf4_b200 import _lib

    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    Hkv, S = 2, 300
    Hq = Hkv * G
    positions = torch.tensor([0, 1, 14, 15, 16, 17, 63, 64, 65, 130, 255, 299], device="cuda", dtype=torch.int32)
    B = positions.numel()
    g = torch.Generator(device="cuda").manual_seed(G * 10 + nsplit)
    q = torch.randn((B, Hq, DH), device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn((B, Hkv, S, DH), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, DH), device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty((B, Hq * DH), device="cuda", dtype=torch.bfloat16)
    ws = torch.empty((lib.nf4_b200_attn_decode_workspace_bytes(B, Hq, nsplit),), device="cuda", dtype=torch.uint8)
    _lib.check(lib.nf4_b200_attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), positions.data_ptr(), out.data_ptr(),
                                        ws.data_ptr(), B, Hq, Hkv, DH, S, nsplit, st), "attn_decode")
    ref = _reference(q, k, v, positions + 1)
    torch.testing.assert_close(out.view(B, Hq, DH).float(), ref, rtol=2e-2, atol=2e-2)
    assert _lib.device_error()[0] == 0


@pytest.mark.parametrize("G,nsplit", [(4, 1), (4, 5), (8, 2), (8, 16), (1, 3)])
@pytest.mark.parametrize("flags", [0, 1])
def test_fused_rotary_append_attention(G, nsplit, flags):
    """One launch: rotate q and k, append k/v at positions[b], attend to [0, positions[b]], merge the splits.
    Run twice on advancing positions, so the second call reads the row the first one appended."""
    from nf4_b200 import _lib

    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    Hkv, S, theta = 2, 200, 500000.0
    Hq = Hkv * G
    positions = torch.tensor([0, 5, 15, 16, 31, 32, 47, 100, 198], device="cuda", dtype=torch.int32)
    B = positions.numel()
    g = torch.Generator(device="cuda").manual_seed(G + 100 * nsplit)
    k = torch.randn((B, Hkv, S, DH), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, DH), device="cuda", generator=g).to(torch.bfloat16)
    k_ref, v_ref = k.clone(), v.clone()
    ws = torch.empty((lib.nf4_b200_attn_decode_workspace_bytes(B, Hq, nsplit),), device="cuda", dtype=torch.uint8)
    counters = torch.zeros((B * Hkv,), device="cuda", dtype=torch.int32)
    out = torch.empty((B, Hq * DH), device="cuda", dtype=torch.bfloat16)
    for step in range(2):
        pos = positions + step
        qkv = torch.randn((B, (Hq + 2 * Hkv) * DH), device="cuda", generator=g).to(torch.bfloat16)
        _lib.check(lib.nf4_b200_attn_decode_fused(qkv.data_ptr(), pos.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                                  ws.data_ptr(), counters.data_ptr(), B, Hq, Hkv, DH, S, nsplit, theta, flags, st),
                   "attn_decode_fused")
        q3 = qkv.view(B, Hq + 2 * Hkv, DH)
        qr = _rope(q3[:, :Hq], pos, theta)
        kr = _rope(q3[:, Hq:Hq + Hkv], pos, theta)
        for b in range(B):
            k_ref[b, :, int(pos[b])] = kr[b]
            v_ref[b, :, int(pos[b])] = q3[b, Hq + Hkv:]
        ref = _reference(qr, k_ref, v_ref, pos + 1)
        torch.testing.assert_close(out.view(B, Hq, DH).float(), ref, rtol=2e-2, atol=2e-2)
        torch.cuda.synchronize()
        for b in range(B):
            p = int(pos[b])
            torch.testing.assert_close(k[b, :, p].float(), k_ref[b, :, p].float(), rtol=2e-2, atol=2e-2)   # one bf16 ulp of slack
            assert torch.equal(v[b, :, p], v_ref[b, :, p])
        assert int(counters.abs().sum()) == 0
    assert _lib.device_error()[0] == 0


def test_position_outside_the_cache_is_refused_in_the_kernel():
    """A position outside [0, S_max) read from device memory: that sequence's cache rows stay untouched, its output
    is zero, the other sequences are served as usual, and the status word holds code 9 with the row and the position
    until it is cleared.  (The bounds test is a compare in the kernel: nothing faults.)"""
    from nf4_b200 import _lib

    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    Hq, Hkv, S, theta, nsplit = 8, 2, 64, 500000.0, 3
    g = torch.Generator(device="cuda").manual_seed(9)
    assert _lib.device_error()[0] == 0
    for bad in (S, -1, 1 << 20):
        pos = torch.tensor([3, bad, 10], device="cuda", dtype=torch.int32)
        B = 3
        k = torch.randn((B, Hkv, S, DH), device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn((B, Hkv, S, DH), device="cuda", generator=g).to(torch.bfloat16)
        k0, v0 = k.clone(), v.clone()
        ws = torch.empty((lib.nf4_b200_attn_decode_workspace_bytes(B, Hq, nsplit),), device="cuda", dtype=torch.uint8)
        counters = torch.zeros((B * Hkv,), device="cuda", dtype=torch.int32)
        out = torch.full((B, Hq * DH), 7.0, device="cuda", dtype=torch.bfloat16)
        qkv = torch.randn((B, (Hq + 2 * Hkv) * DH), device="cuda", generator=g).to(torch.bfloat16)
        _lib.check(lib.nf4_b200_attn_decode_fused(qkv.data_ptr(), pos.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                                  ws.data_ptr(), counters.data_ptr(), B, Hq, Hkv, DH, S, nsplit, theta, 0, st),
                   "attn_decode_fused")
        torch.cuda.synchronize()
        assert torch.equal(k[1], k0[1]) and torch.equal(v[1], v0[1])       # nothing written for the refused row
        assert not out[1].any()                                            # ... and it attends to nothing
        assert not torch.equal(k[0], k0[0]) and out[0].any() and out[2].any()
        code, row, where, count = _lib.device_error()
        assert code == 9 and row == 1 and where == (bad & 0xffffffff) and count >= 1
        # the prompt form: the same refusal per token
        q4 = functional_rope_prefill(qkv.view(1, B, -1).contiguous(), pos, torch.zeros_like(k[:1]), torch.zeros_like(v[:1]), Hq, Hkv, theta)
        assert q4.shape == (1, Hq, B, DH)
        _lib.device_error_clear()
        assert _lib.device_error() == (0, 0, 0, 0)


def functional_rope_prefill(qkv, pos, kc, vc, Hq, Hkv, theta):
    from nf4_b200 import _lib, functional

    k0, v0 = kc.clone(), vc.clone()
    q4 = functional.rope_prefill(qkv, pos, kc, vc, Hq, Hkv, theta)
    torch.cuda.synchronize()
    changed = (kc != k0).any(dim=-1).any(dim=1)[0].nonzero().flatten().tolist()     # cache rows that were written
    assert sorted(changed) == sorted(int(p) for p in pos.tolist() if 0 <= int(p) < kc.shape[2])
    assert _lib.device_error()[0] == 9
    return q4
