"""Tensor-parallel host logic on CPU: two `gloo` ranks shard the weights as the decode engine does
(`nf4_b200.parallel`), quantize their shards with the oracle, run the oracle's linear on them and meet
in the collectives the engine uses (all-reduce of partial sums, all-gather of argmax candidates)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from helpers import bf16_bits, bits_to_bf16, seeded_act, seeded_weight

WORLD = 2
RTOL, ATOL = 1.6e-2, 1e-2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _quant(w):
    from nf4_b200.codebook import NF4_LEVELS

    code = np.array(NF4_LEVELS, np.float32)
    packed, absmax = oracle.quantize(bf16_bits(w), code, 64)
    return packed, absmax, code


def _linear(x, w):
    packed, absmax, code = _quant(w)
    N, K = w.shape
    y = oracle.linear_bf16(bf16_bits(x), packed, absmax, code, N, K, 64, mode=oracle.GEMV_MODE)
    return bits_to_bf16(y).float()


def _worker(rank: int, port: int, results):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=WORLD)
        from nf4_b200 import parallel

        D, F, HQ, HKV, DH, V = 256, 512, 4, 2, 64, 96
        parallel.check_shardable(HQ, HKV, DH, F, V, WORLD)
        x = seeded_act((3, D), 1)

        # column-parallel (gate): the gathered shard outputs ARE the unsharded output, bit for bit
        wg = seeded_weight((F, D), 2)
        wu = seeded_weight((F, D), 3)
        y_r = _linear(x, parallel.shard_rows(wg, rank, WORLD).contiguous())
        parts = [torch.empty_like(y_r) for _ in range(WORLD)]
        dist.all_gather(parts, y_r)
        assert torch.equal(torch.cat(parts, dim=1), _linear(x, wg))

        # gate/up interleave: row 2i is gate_i, row 2i+1 is up_i of this rank's slice
        gu = parallel.shard_gate_up(wg, wu, rank, WORLD)
        c = F // WORLD
        assert torch.equal(gu[0::2], wg[rank * c:(rank + 1) * c]) and torch.equal(gu[1::2], wu[rank * c:(rank + 1) * c])

        # Q/K/V stack: whole heads of this rank
        wq, wk, wv = seeded_weight((HQ * DH, D), 4), seeded_weight((HKV * DH, D), 5), seeded_weight((HKV * DH, D), 6)
        qkv = parallel.shard_qkv(wq, wk, wv, rank, WORLD)
        hq, hk = HQ * DH // WORLD, HKV * DH // WORLD
        assert qkv.shape == (hq + 2 * hk, D)
        assert torch.equal(qkv[:hq], wq[rank * hq:(rank + 1) * hq]) and torch.equal(qkv[hq + hk:], wv[rank * hk:(rank + 1) * hk])

        # row-parallel (down): the shard's codes are the full matrix's codes (no block straddles ranks) ...
        wd = seeded_weight((D, F), 7)
        wd_r = parallel.shard_cols(wd, rank, WORLD)
        p_full, a_full, _ = _quant(wd)
        p_r, a_r, _ = _quant(wd_r)
        kc = F // WORLD
        assert np.array_equal(p_full.reshape(D, F // 2)[:, rank * kc // 2:(rank + 1) * kc // 2], p_r.reshape(D, kc // 2))
        assert np.array_equal(a_full.reshape(D, F // 64)[:, rank * kc // 64:(rank + 1) * kc // 64], a_r.reshape(D, kc // 64))
        # ... and the all-reduced bf16 partial sums match the unsharded linear within the linear tolerance
        h = seeded_act((3, F), 8)
        part = _linear(h[:, rank * kc:(rank + 1) * kc].contiguous(), wd_r)
        dist.all_reduce(part)
        torch.testing.assert_close(part, _linear(h, wd), rtol=RTOL, atol=ATOL)

        # vocabulary split: local argmax + gathered candidates = argmax over the full vocabulary, ties included
        g = torch.Generator().manual_seed(9)
        logits = torch.randn((5, V), generator=g).to(torch.bfloat16)
        logits[1, 7] = logits[1, 60] = 9.0          # a tie across the two slices: the lower id wins
        logits[2, 50] = logits[2, 51] = 8.0         # a tie inside one slice
        vr = V // WORLD
        mine = parallel.shard_rows(logits.t().contiguous(), rank, WORLD).t().contiguous()    # [5, V/tp]
        local_ids = mine.float().argmax(dim=1)
        cand = parallel.local_candidates(mine, local_ids, rank, vr)
        gathered = [torch.empty_like(cand) for _ in range(WORLD)]
        dist.all_gather(gathered, cand)
        ids = parallel.merge_candidates(torch.stack(gathered))
        assert torch.equal(ids, logits.float().argmax(dim=1))
        assert int(ids[1]) == 7 and int(ids[2]) == 50

        dist.barrier()
        dist.destroy_process_group()
        results[rank] = "ok"
    except Exception as e:  # noqa: BLE001 - reported to the parent
        import traceback

        results[rank] = traceback.format_exc() + repr(e)


def test_two_gloo_ranks_shard_quantize_reduce():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as m:
        results = m.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, port, results)) for r in range(WORLD)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=240)
        for p in procs:
            if p.is_alive():
                p.kill()
        out = dict(results)
    assert out.get(0) == "ok" and out.get(1) == "ok", out


def test_check_shardable_rejects_straddling_blocks():
    from nf4_b200 import parallel

    parallel.check_shardable(64, 8, 128, 28672, 128256, 8)
    with pytest.raises(ValueError):
        parallel.check_shardable(64, 8, 128, 28672, 128256, 3)
    with pytest.raises(ValueError):
        parallel.check_shardable(4, 2, 64, 64 * 3, 96, 2)           # ffn/tp = 96 is not a multiple of 64
    with pytest.raises(ValueError):
        parallel.shard_cols(torch.zeros((4, 96)), 0, 2)
