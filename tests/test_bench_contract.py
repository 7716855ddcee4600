"""The benchmark's reference arm runs on CPU: its JSON line must carry the contract's keys and the same
`config` object the GPU arm prints for the same workload."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_json_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    assert len(out.stdout.strip().splitlines()) == 1, "stdout must hold the JSON line and nothing else"
    line = json.loads(out.stdout.strip().splitlines()[-1])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["unit"] == "tok/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["vs_baseline"] is None and line["data"] == "synthetic"
    assert set(line["cpu_baseline"]) >= {"value", "unit", "cores", "kind", "sample"} and line["cpu_baseline"]["kind"] == "port"
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the same config object as the GPU arm's
    sys.path.insert(0, ROOT)
    import bench

    want = bench.workload_config("llama3-8b-shape", 1, 512, 1, 0.0)
    assert set(line["config"]) == set(want)
    for k in ("workload", "parallelism", "global_batch", "context", "blocksize", "double_quant"):
        assert line["config"][k] == want[k], k


def test_only_the_result_line_reaches_stdout():
    """Whatever else writes to file descriptor 1 after start-up (NCCL prints its version banner there when NCCL_DEBUG
    is set) lands on stderr: bench.py keeps a private copy of stdout for its one JSON line."""
    code = ("import os, sys; sys.argv=['bench.py']; sys.path.insert(0, %r); import bench; bench._claim_stdout(); "
            "os.write(1, b'library banner\\n'); print('python-level chatter'); bench.emit({'ok': 1})" % ROOT)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout == '{"ok": 1}\n'
    assert "library banner" in out.stderr and "python-level chatter" in out.stderr
