"""The allocation-free attention entry point (nf4_b200_attn_decode_static) against the regular one.

Some hosts of this library have no way to allocate device memory for scratch: they run inside a
process whose memory pool they cannot reach, or in a serving loop where cudaMalloc is forbidden
after start-up.  For them the per-split partial results live in an array built into the library.
This file is named so that pytest collects it last: it checks the static entry point through the
C ABI, twice in a row with different inputs, and it must pass both on its own and after every
other test has used the GPU."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, B, Hq, Hkv, S_max, lens):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((B, Hq * 128), device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn((B, Hkv, S_max, 128), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S_max, 128), device="cuda", generator=g).to(torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lens], device="cuda", dtype=torch.int32)
    return q, k, v, pos


def _both(lib, _lib, q, k, v, pos, B, Hq, Hkv, S_max, nsplit):
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty((lib.nf4_b200_attn_decode_workspace_bytes(B, Hq, nsplit),), device="cuda", dtype=torch.uint8)
    ref = torch.empty((B, Hq * 128), device="cuda", dtype=torch.bfloat16)
    out = torch.full((B, Hq * 128), float("nan"), device="cuda", dtype=torch.bfloat16)
    _lib.check(lib.nf4_b200_attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(), ref.data_ptr(),
                                        ws.data_ptr(), B, Hq, Hkv, 128, S_max, nsplit, st), "attn_decode")
    _lib.check(lib.nf4_b200_attn_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                               B, Hq, Hkv, 128, S_max, nsplit, st), "attn_decode_static")
    torch.cuda.synchronize()
    return ref, out


def test_static_scratch_matches_caller_scratch_twice():
    from nf4_b200 import _lib

    lib = _lib.load()
    # first call: 3 rows, 8 query heads over 2 KV heads, 5 splits
    q, k, v, pos = _inputs(1, 3, 8, 2, 96, [96, 17, 1])
    ref, out = _both(lib, _lib, q, k, v, pos, 3, 8, 2, 96, 5)
    torch.testing.assert_close(out.float(), ref.float(), rtol=1.6e-2, atol=1e-2)
    assert torch.equal(out, ref)          # same kernels, same order: identical bits
    # and against plain softmax attention (torch is only the checker)
    for b, n in enumerate([96, 17, 1]):
        for h in range(8):
            kk, vv = k[b, h // 4, :n].float(), v[b, h // 4, :n].float()
            p = torch.softmax(kk @ q[b, h * 128:(h + 1) * 128].float() / 128 ** 0.5, dim=0)
            torch.testing.assert_close(out[b, h * 128:(h + 1) * 128].float(), p @ vv, rtol=2e-2, atol=2e-2)
    # second call right after it: a different, smaller shape, so the array still holds the first
    # call's partial results where this call does not write -- they must not leak into the output
    q, k, v, pos = _inputs(2, 2, 4, 4, 40, [40, 9])
    ref, out = _both(lib, _lib, q, k, v, pos, 2, 4, 4, 40, 2)
    torch.testing.assert_close(out.float(), ref.float(), rtol=1.6e-2, atol=1e-2)
    assert torch.equal(out, ref)


def test_static_scratch_refuses_oversized_shapes():
    from nf4_b200 import _lib

    lib = _lib.load()
    assert lib.nf4_b200_attn_decode_static_max_bytes() == 16 * 64 * 8 * 130 * 4
    d = ctypes.c_void_p(256)
    rc = lib.nf4_b200_attn_decode_static(d, d, d, d, d, 16, 64, 8, 128, 64, 9, None)   # one split too many
    assert rc == 6 and "built-in array" in _lib.last_error()


def test_static_scratch_at_its_exact_maximum():
    """The largest shape the built-in array holds (16 sequences x 64 query heads x 8 splits) runs and fills
    every slot of it; one split more is refused (above)."""
    from nf4_b200 import _lib

    lib = _lib.load()
    B, Hq, Hkv, S_max, ns = 16, 64, 8, 200, 8
    assert lib.nf4_b200_attn_decode_workspace_bytes(B, Hq, ns) == lib.nf4_b200_attn_decode_static_max_bytes()
    lens = [200, 1, 7, 8, 9, 64, 65, 127, 128, 129, 150, 199, 16, 33, 100, 2]
    q, k, v, pos = _inputs(3, B, Hq, Hkv, S_max, lens)
    ref, out = _both(lib, _lib, q, k, v, pos, B, Hq, Hkv, S_max, ns)
    assert torch.equal(out, ref)
    assert _lib.device_error()[0] == 0
