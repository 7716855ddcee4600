"""The one-shot all-reduce over peer memory, with all ranks of an exchange emulated on ONE GPU as a single
cooperative launch (nf4_b200_tp_allreduce_emulated: blockIdx.y is the rank, every "rank" has its own buffer,
partial tile and output).  The sums must equal an fp32 sum in rank order rounded once to bf16, be identical on
all ranks, and stay right over repeated calls on the same buffers (both buffer sets, advancing epochs) and
when the tile size changes between calls."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _arr(ts):
    return (ctypes.c_uint64 * len(ts))(*[t.data_ptr() if t is not None else 0 for t in ts])


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_emulated_ranks_sum_in_rank_order(world):
    from nf4_b200 import _lib

    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    max_numel = 16 * 8192
    nbytes = lib.nf4_b200_tp_allreduce_buffer_bytes(max_numel)
    bufs = [torch.zeros((nbytes,), device="cuda", dtype=torch.uint8) for _ in range(world)]
    g = torch.Generator(device="cuda").manual_seed(world)
    for call, numel in enumerate([16 * 8192, 16 * 8192, 8, 4096, 16 * 8192, 2 * 4096 + 8, 16 * 8192]):
        parts = [torch.randn((numel,), device="cuda", generator=g).to(torch.bfloat16) for _ in range(world)]
        res = torch.randn((numel,), device="cuda", generator=g).to(torch.bfloat16)
        use_res = call % 2 == 0
        outs = [torch.full((numel,), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        rc = lib.nf4_b200_tp_allreduce_emulated(_arr(parts), _arr([res] * world) if use_res else None, _arr(outs), numel,
                                                _arr(bufs), nbytes, world, st)
        _lib.check(rc, "tp_allreduce_emulated")
        torch.cuda.synchronize()
        acc = torch.zeros((numel,), device="cuda", dtype=torch.float32)
        for p in parts:
            acc += p.float()
        if use_res:
            acc += res.float()
        want = acc.to(torch.bfloat16)
        for r in range(world):
            assert torch.equal(outs[r], want), (call, r)
        assert _lib.device_error()[0] == 0


def test_in_place_residual_and_argument_checks():
    from nf4_b200 import _lib

    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    nbytes = lib.nf4_b200_tp_allreduce_buffer_bytes(4096)
    bufs = [torch.zeros((nbytes,), device="cuda", dtype=torch.uint8) for _ in range(2)]
    x = [torch.ones((4096,), device="cuda", dtype=torch.bfloat16) * (r + 1) for r in range(2)]
    part = [torch.full((4096,), 0.5 * (r + 1), device="cuda", dtype=torch.bfloat16) for r in range(2)]
    # y aliases the residual (x += sum of the partial tiles), as the decode step uses it
    _lib.check(lib.nf4_b200_tp_allreduce_emulated(_arr(part), _arr(x), _arr(x), 4096, _arr(bufs), nbytes, 2, st), "emulated")
    torch.cuda.synchronize()
    assert torch.all(x[0] == 2.5) and torch.all(x[1] == 3.5)
    assert lib.nf4_b200_tp_allreduce_emulated(_arr(part), None, _arr(x), 4100, _arr(bufs), nbytes, 2, st) == 1      # numel % 8
    assert lib.nf4_b200_tp_allreduce_emulated(_arr(part), None, _arr(x), 8192, _arr(bufs), nbytes, 2, st) == 3      # buffers too small
    assert lib.nf4_b200_tp_allreduce_emulated(_arr(part), None, _arr(x), 4096, _arr(bufs), nbytes, 9, st) == 6      # world > 8
