"""Tensor parallelism on real GPUs: two ranks (NCCL for the plumbing, the one-shot exchange over peer memory for
the partial sums) decode a small model and must reproduce the single-GPU run -- the check `bench.py` makes
before it times any multi-GPU run, here as a test.  Needs two GPUs; skipped on a one-GPU box."""

import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("exchange", ["oneshot", "nccl"])
def test_two_ranks_reproduce_one(exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NF4_TP_REDUCE=exchange, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--workload", "tiny", "--steps", "4",
           "--warmup", "3", "--no-anchor"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT, env=env)
    assert out.returncode == 0, out.stderr[-3000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    par = line["tp_parity"]
    assert par["logits_outside_tolerance"] == 0.0, par
    assert par["tokens_equal_where_clear"] and par["clear_steps"] > 0, par
    assert line["device_error"][0] == 0
    assert line["n_gpus"] == 2 and line["value"] > 0
