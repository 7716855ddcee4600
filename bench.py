"""Benchmark of the NF4 W4A16 decode path.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torch.distributed.run)
    python bench.py --impl reference ...                   the CPU restatement of the same path, host cores
    python bench.py --kernel gemv --N 14336 --K 4096 --M 1 one kernel in isolation (used for ncu captures)
    python bench.py --workload llama3-8b-prefill --steps 3 the prefill configuration (batch 8 x 2048) through the jitted module

Workload (synthetic, random-init, seeded; no dataset or benchmark suite is involved):
  N = 1  -> a Llama-3-8B-shaped NF4 decoder, batch 1, a 512-token random prompt in the KV cache, greedy decode; a
            "step" is one decode step (one token through all 225 quantized linears + attention over the cache).
            `value` / `e2e` come from the path a user of the reference takes: the nn.Module of nf4_b200.llama
            jitted by thunder.jit with the NF4 transform, the decode fusion pass and the CUDA-graph transform
            (`value`: ids stay on the device; `e2e`: ids and position come from pinned host memory every step and
            the sampled ids are read back).  `engine` holds the same numbers for the decode engine that calls the
            C ABI directly; `roofline` times the step's GEMV launches alone.
  N > 1  -> the Llama-3-70B-shaped decoder, batch 16, 1024-token context, tensor-parallel over the N GPUs on the
            engine (strong scaling: the model is fixed).  Rank 0 first runs the SAME workload on one GPU
            (`tp1_same_workload_tok_s`), all ranks check a small model against its single-GPU run (`tp_parity`), and
            the step is timed with the one-shot exchange over peer memory and with NCCL (`exchange`).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "lightning-thunder_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

UNIT = "tok/s"

_result_out = None


def _claim_stdout() -> None:
    """The contract is ONE JSON line on stdout.  Libraries write there too (NCCL prints its version banner to
    stdout when NCCL_DEBUG is set in the environment), so file descriptor 1 is pointed at stderr for the rest of
    the process and the result line goes to a saved copy of the original stdout."""
    global _result_out
    if _result_out is None:
        sys.stdout.flush()
        _result_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(obj) -> None:
    out = _result_out if _result_out is not None else sys.stdout
    out.write(json.dumps(obj) + "\n")
    out.flush()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for j, n in enumerate(names) if any(len(r) >= 7 and r[3 + j].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's linears on the host cores
# --------------------------------------------------------------------------------------------

# DRAM traffic of the fused dequant-GEMV relative to its algorithmic bytes, from one ncu capture of the kernel
# (N=32064, K=4096, M=1: 73.95 MB read + 1.05 MB written against 73.95 MB algorithmic); the kernel streams
# every weight byte exactly once, so traffic grows in proportion to N*K.
NCU_TRAFFIC_RATIO = 75.006 / 73.948


def workload_config(name: str, batch: int, prompt_len: int, world: int, step_bytes: float) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": f"{name} NF4 decode, batch {batch}, {prompt_len}-token prompt in the KV cache, greedy",
            "parallelism": f"tp{world}", "global_batch": batch, "context": prompt_len,
            "l2": f"{step_bytes / 1e9:.2f} GB of weights stream per step per GPU (> L2), no flush needed",
            "blocksize": 64, "double_quant": False}


def cpu_decode_sample(cfg_name: str, batch: int, reps: int, warmup: int = 0):
    """Times the quantized linears of ONE decoder layer (QKV, attention output, gate+up, down) at
    `batch` activation rows with the CPU oracle (OpenMP, all host threads), `reps` times, and scales
    to a whole model: tok/s = batch / (n_layers * t_layer + t_head_estimate).  Weights come from the
    oracle's own quantizer on seeded N(0, 0.02) data."""
    import numpy as np

    import oracle
    from nf4_b200.codebook import NF4_LEVELS
    from nf4_b200.decoder import LLAMA3_8B, LLAMA3_70B

    cfg = LLAMA3_70B if "70b" in cfg_name else LLAMA3_8B
    code = np.array(NF4_LEVELS, np.float32)
    rng = np.random.default_rng(0)
    D, F = cfg.d_model, cfg.ffn
    shapes = [((cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim, D), (D, cfg.n_heads * cfg.head_dim), (2 * F, D), (D, F)]
    mats = []
    for (N, K) in shapes:
        w = (rng.standard_normal((N, K), dtype=np.float32) * 0.02)
        packed, absmax = oracle.quantize(oracle.f32_to_bf16_bits(w), code, 64)
        x = oracle.f32_to_bf16_bits(rng.standard_normal((batch, K), dtype=np.float32))
        mats.append((x, packed, absmax, N, K))
    times = []
    budget_s = 90.0                      # the CPU arm stays a bounded sample: stop adding passes beyond this
    t_start = time.perf_counter()
    for it in range(warmup + reps):
        t0 = time.perf_counter()
        for (x, packed, absmax, N, K) in mats:
            oracle.linear_bf16(x, packed, absmax, code, N, K, 64, mode=oracle.GEMV_MODE)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
        if times and time.perf_counter() - t_start > budget_s:
            break
    t_layer = statistics.median(times)
    layer_weights = sum(N * K for (_, _, _, N, K) in mats)
    t_head = t_layer * (cfg.vocab * D) / layer_weights
    tok_s = batch / (cfg.n_layers * t_layer + t_head)
    return tok_s, t_layer, os.cpu_count(), len(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from nf4_b200.decoder import LLAMA3_8B, LLAMA3_70B

    workload = args.workload or ("llama3-8b" if args.gpus == 1 else "llama3-70b")
    if workload not in ("llama3-8b", "llama3-70b"):
        workload = "llama3-8b"
    cfg, batch, prompt_len = (LLAMA3_8B, 1, 512) if workload == "llama3-8b" else (LLAMA3_70B, 16, 1024)
    if args.prompt is not None:
        prompt_len = args.prompt
    # the CPU arm has one host: it runs the whole (unsharded) model whatever --gpus says; each "step" is a
    # bounded sample (one decoder layer's linears) scaled to the model, so the run ends within minutes
    tok_s, t_layer, cores, passes = cpu_decode_sample(workload, batch, max(1, args.steps), min(1, max(0, args.warmup)))
    D, F = cfg.d_model, cfg.ffn
    weights = cfg.n_layers * (((cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim) * D + D * cfg.n_heads * cfg.head_dim + 3 * F * D) + cfg.vocab * D
    config = workload_config(cfg.name, batch, prompt_len, args.gpus, weights * 0.5625 / args.gpus)
    line = {
        "impl": "reference", "metric": metric_name(workload, args.gpus), "value": tok_s, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * batch / tok_s, "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"the 4 quantized linears of one decoder layer at M={batch}, median of {passes} "
                                   f"passes ({t_layer * 1e3:.1f} ms each; at most 90 s of them), scaled to all layers + output head"},
        "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        # no whole step runs on the CPU: ms_per_step is one layer's linears scaled to the model
        "extrapolated": True,
    }
    emit(line)


# --------------------------------------------------------------------------------------------
# single-kernel mode (profiling driver)
# --------------------------------------------------------------------------------------------

def run_kernel(args):
    import ctypes

    import torch

    import nf4_b200
    from nf4_b200 import _lib

    torch.cuda.set_device(0)
    lib = _lib.load()
    N, K, M = args.N, args.K, args.M
    # bytes of one weight: codes + fp32 absmax, or (double quantization) codes + 8-bit absmax + one fp32 scale per 256
    wbytes = N * K // 2 + (N * K // 64 + N * K // 4096 + 1028 if args.dq else N * K // 16)
    nbuf = args.nbuf or max(2, int(4 * 126e6 // wbytes) + 1)     # the rotating set is > 4x the L2
    g = torch.Generator(device="cuda").manual_seed(0)
    ws = []
    for _ in range(nbuf):
        w = (torch.randn((N, K), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        ws.append(nf4_b200.quantize_4bit(w, compress_statistics=args.dq))
        del w
    x = torch.randn((M, K), device="cuda", generator=g).to(torch.bfloat16)
    y = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    # gemv: the fused GEMV whatever M (up to 16); gemm: the library's dispatch, with its split-K scratch
    need = lib.nf4_b200_linear_workspace_bytes(M, N, K, _lib.NF4_BF16) if args.kernel == "gemm" else 0
    scratch = torch.zeros((max(need, 16),), device="cuda", dtype=torch.uint8)
    dq_ws = torch.empty((lib.nf4_b200_linear_dq_workspace_bytes(N, K),), device="cuda", dtype=torch.uint8) if args.dq else None

    def launch_all():
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for p, qs in ws:
            if args.dq:
                # double-quantized weight: the fused GEMV expands the 8-bit absmax in its stages (M <= 16), larger M
                # expands it into dq_ws and runs the tensor-core GEMM
                rc = lib.nf4_b200_linear_dq(x.data_ptr(), M, K, p.data_ptr(), qs.absmax.data_ptr(), qs.state2.absmax.data_ptr(),
                                            qs.offset.data_ptr(), qs.state2.code.data_ptr(), qs.code.data_ptr(), N, None,
                                            y.data_ptr(), _lib.NF4_BF16, dq_ws.data_ptr(), dq_ws.numel(), st)
            elif args.kernel == "gemv":
                rc = lib.nf4_b200_gemv(x.data_ptr(), M, K, p.data_ptr(), qs.absmax.data_ptr(), qs.code.data_ptr(), N,
                                       None, y.data_ptr(), _lib.NF4_BF16, st)
            elif args.kernel == "gemm":
                rc = lib.nf4_b200_linear(x.data_ptr(), M, K, p.data_ptr(), qs.absmax.data_ptr(), qs.code.data_ptr(), N, 64,
                                         None, y.data_ptr(), _lib.NF4_BF16, scratch.data_ptr(), scratch.numel(), st)
            elif args.kernel == "dequantize":
                rc = lib.nf4_b200_dequantize(p.data_ptr(), qs.absmax.data_ptr(), qs.code.data_ptr(), N * K, 64,
                                             deq.data_ptr(), _lib.NF4_BF16, st)
            else:
                rc = lib.nf4_b200_quantize(deq.data_ptr(), N * K, _lib.NF4_BF16, 64, qs.code.data_ptr(), p.data_ptr(),
                                           qs.absmax.data_ptr(), st)
            _lib.check(rc, args.kernel)

    deq = torch.empty((N, K), device="cuda", dtype=torch.bfloat16) if args.kernel not in ("gemv", "gemm") else None
    if deq is not None:
        deq.copy_(nf4_b200.dequantize_4bit(*ws[0]))
    for _ in range(max(1, args.warmup)):
        launch_all()
    torch.cuda.synchronize()
    run = launch_all
    if args.kernel in ("gemv", "gemm"):
        # one CUDA graph of the nbuf launches: small shapes would otherwise time the host's launch rate
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launch_all()
        run = graph.replay
        run()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(max(1, args.steps)):
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / nbuf)
    us = statistics.median(ts)
    if args.kernel in ("gemv", "gemm"):
        alg = wbytes + 2 * M * K + 2 * M * N
    else:
        alg = 2 * N * K + wbytes
    peaks, src = measured_peaks()
    out = {"kernel": args.kernel + ("+dq" if args.dq else ""), "N": N, "K": K, "M": M, "us_per_launch": us, "algorithmic_bytes": alg,
           "GBps": alg / us / 1e3, "hbm_frac_of_" + src: alg / us / 1e3 / peaks["hbm_gbs"], "buffers": nbuf}
    if args.kernel == "gemm":
        tf = 2.0 * M * N * K / us / 1e6
        out.update({"TFLOPs": tf, "tensor_frac_of_" + src: tf / peaks["bf16_tflops"]})
    emit(out)


def run_attention(args):
    """The decode step's attention launch (rotary + KV append + attention over the cache + merge of the
    splits) by itself: one CUDA graph of one launch per layer over distinct caches (cold reads), timed with
    events; bytes = the K and V rows read."""
    import ctypes

    import torch

    from nf4_b200 import _lib

    torch.cuda.set_device(0)
    lib = _lib.load()
    B, Hq, Hkv, ctx, Dh = args.B, args.Hq, args.Hkv, args.ctx, 128
    S = ctx + 8
    per_layer = B * Hkv * S * Dh * 2 * 2
    L = args.nbuf or max(2, int(4 * 126e6 // per_layer) + 1)          # rotating caches exceed four times the L2
    ns = args.splits or max(1, min(16, 296 // max(1, Hkv * B), S // 128))
    g = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn((L, B, Hkv, S, Dh), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((L, B, Hkv, S, Dh), device="cuda", generator=g).to(torch.bfloat16)
    qkv = torch.randn((B, (Hq + 2 * Hkv) * Dh), device="cuda", generator=g).to(torch.bfloat16)
    out = torch.empty((B, Hq * Dh), device="cuda", dtype=torch.bfloat16)
    pos = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    cnt = torch.zeros((B * Hkv,), device="cuda", dtype=torch.int32)
    ws = torch.empty((lib.nf4_b200_attn_decode_workspace_bytes(B, Hq, ns),), device="cuda", dtype=torch.uint8)

    def launch_all():
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for l in range(L):
            _lib.check(lib.nf4_b200_attn_decode_fused(qkv.data_ptr(), pos.data_ptr(), k[l].data_ptr(), v[l].data_ptr(), out.data_ptr(),
                                                      ws.data_ptr(), cnt.data_ptr(), B, Hq, Hkv, Dh, S, ns, 500000.0, 0, st), "attention")

    for _ in range(max(1, args.warmup)):
        launch_all()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch_all()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ts = []
    for _ in range(max(1, args.steps)):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / L)
    us = statistics.median(ts)
    alg = B * Hkv * (ctx + 1) * Dh * 2 * 2
    peaks, src = measured_peaks()
    emit(({"kernel": "attention", "B": B, "Hq": Hq, "Hkv": Hkv, "ctx": ctx, "splits": ns, "us_per_launch": us,
                      "algorithmic_bytes": alg, "GBps": alg / us / 1e3, "hbm_frac_of_" + src: alg / us / 1e3 / peaks["hbm_gbs"],
                      "buffers": L, "device_error": list(_lib.device_error())}))


# --------------------------------------------------------------------------------------------
# the decode benchmark
# --------------------------------------------------------------------------------------------

def _log(msg):
    if os.environ.get("NF4_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')} {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


WORKLOADS = {
    # name: (config attribute, batch, prompt tokens, new tokens of the configuration)
    "llama3-8b": ("LLAMA3_8B", 1, 512, 128),
    "llama3-70b": ("LLAMA3_70B", 16, 1024, 256),
    "tiny": (None, 1, 16, 16),
}


def metric_name(workload: str, world: int) -> str:
    shape = {"llama3-8b": "Llama-3-8B shape", "llama3-70b": "Llama-3-70B shape", "tiny": "tiny test shape"}[workload]
    tp = f", tensor parallel over {world} GPUs" if world > 1 else ""
    return f"NF4 W4A16 decode tok/s ({shape}{tp}); dequant-GEMV HBM GB/s vs 8 TB/s"


def engine_decode(cfg, batch, prompt_len, steps, warmup, dev, rank, world, group, *, feed_prompt=True, roofline=True,
                  sampler=None):
    """The decode engine (nf4_b200.decoder.NF4Decoder: this library's kernels called directly, one CUDA graph per
    step).  Returns tok/s with the ids staying on the device, tok/s with host-fed ids, and the GEMV chain's
    roofline figures."""
    import torch

    from nf4_b200 import _lib
    from nf4_b200.decoder import NF4Decoder

    max_seq = prompt_len + 2 * warmup + 3 * steps + 32
    t_build = time.perf_counter()
    dec = NF4Decoder(cfg, batch=batch, max_seq=max_seq, device=dev, seed=1, tp_rank=rank, tp_size=world, group=group,
                     tp_reduce=os.environ.get("NF4_TP_REDUCE", "oneshot"))
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    _log(f"engine built in {t_build:.1f}s; capturing")
    g_host = dec.capture(feed_back=False)
    g_dev = dec.capture(feed_back=True)
    launches = dec.launches_per_step

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    gen = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=gen)
    prompt_dev = prompt.to(dev)
    dec.reset()
    dec.graph = g_host
    if feed_prompt:
        # prompt -> KV cache, one token per step (the same decode path)
        for t in range(prompt_len):
            dec.ids_in.copy_(prompt_dev[:, t])
            dec.run_step()
    else:
        # timing only: a cache of random rows up to the prompt length reads the same bytes as a real one
        g = torch.Generator(device=dev).manual_seed(99)
        for c in (dec.k_cache, dec.v_cache):
            c[:, :, :, :prompt_len].copy_(torch.randn(c[:, :, :, :prompt_len].shape, generator=g, device=dev, dtype=torch.float32) * 0.5)
        dec.set_positions(prompt_len)
        dec.ids_in.copy_(prompt_dev[:, -1])
        dec.run_step()
    torch.cuda.synchronize()

    dec.graph = g_dev
    dec.ids_in.copy_(dec.ids_out)
    for _ in range(warmup):
        dec.run_step()
    barrier()
    if sampler is not None:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        dec.run_step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())

    # host-fed ids: every step the ids come from pinned host memory and the sampled ids go back
    dec.graph = g_host
    ids_host = torch.empty((batch,), dtype=torch.int64).pin_memory()
    out_host = torch.empty((batch,), dtype=torch.int64).pin_memory()
    ids_host.copy_(dec.ids_out.cpu())
    barrier()
    w0 = time.perf_counter()
    for _ in range(steps):
        dec.ids_in.copy_(ids_host, non_blocking=True)
        dec.run_step()
        out_host.copy_(dec.ids_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        ids_host.copy_(out_host)
    barrier()
    e2e_s = time.perf_counter() - w0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_s = float(t.item())
    res = {"tok_s": steps * batch / (ms / 1e3), "ms_per_step": ms / steps, "e2e_tok_s": steps * batch / e2e_s,
           "launches_per_step": launches, "build_s": t_build, "step_bytes": dec.weight_bytes()}
    if world > 1 and dec.oneshot is not None:
        # the same engine with the library all-reduce (NCCL) in place of the one-shot exchange over peer memory
        res["exchange"] = "one-shot all-reduce over peer memory (nf4_b200_tp_allreduce)"
        saved, dec.oneshot = dec.oneshot, None
        g_nccl = dec.capture(feed_back=True)
        dec.graph = g_nccl
        dec.ids_in.copy_(dec.ids_out)
        for _ in range(warmup):
            dec.run_step()
        barrier()
        e0.record()
        for _ in range(steps):
            dec.run_step()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        res["nccl_exchange_tok_s"] = steps * batch / (float(t.item()) / 1e3)
        res["nccl_exchange_ms_per_step"] = float(t.item()) / steps
        dec.oneshot = saved
        del g_nccl
    if not roofline:
        del dec
        torch.cuda.empty_cache()
        return res

    # ---- roofline of the dominant kernel (the fused dequant-GEMV).  Algorithmic bytes of every GEMV launch
    # of a step come from one uncaptured step (a hook records them); the duration comes from a CUDA graph
    # holding exactly those launches (no glue kernels, no collectives), replayed and timed with events on
    # the launching stream: cold weights and dependent back-to-back launches, as inside the step.
    dec.graph = None
    dec.gemv_events = ev = []
    dec.ids_in.copy_(dec.ids_out)
    dec.step()
    torch.cuda.synchronize()
    dec.gemv_events = None
    gemv_bytes = [n for _, _, n in ev]
    for t in (dec.x, dec.attn, dec.h):
        t.zero_()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        dec.linears_only()
        side.synchronize()
        chain = torch.cuda.CUDAGraph()
        with torch.cuda.graph(chain, stream=side, capture_error_mode="thread_local"):
            dec.linears_only()
        chain.replay()
        side.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, min(steps, 16))
        c0.record(side)
        for _ in range(reps):
            chain.replay()
        c1.record(side)
        side.synchronize()
    chain_us = c0.elapsed_time(c1) * 1e3 / reps
    res.update({"gemv_bytes": gemv_bytes, "chain_us": chain_us, "device_error": list(_lib.device_error())})
    del dec, chain
    torch.cuda.empty_cache()
    return res


def thunder_decode(cfg, batch, prompt_len, steps, warmup, dev, sampler=None):
    """The same workload through the reference's API: the Llama-shaped nn.Module (nf4_b200.llama) jitted by
    thunder.jit with NF4LinearQuant4bit + NF4DecodeFusion + PrunePrologueChecks + CUDAGraphTransform on the NF4
    executor (nf4_b200.thunder_decode.compile_decoder).  Timed as thunder/benchmarks/benchmark_inference.py:467-529
    times decode: one module call per token, the sampled id fed back."""
    import torch

    from nf4_b200 import _lib
    from nf4_b200.llama import LlamaArgs, LlamaDecoder
    from nf4_b200.thunder_decode import GreedyStep, compile_decoder

    max_seq = prompt_len + 2 * warmup + 2 * steps + 16
    args = LlamaArgs(dim=cfg.d_model, n_layers=cfg.n_layers, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads,
                     vocab_size=cfg.vocab, hidden_dim=cfg.ffn, norm_eps=cfg.norm_eps, rope_theta=cfg.rope_theta,
                     max_seq_len=max_seq, max_batch=batch)
    t0 = time.perf_counter()
    with torch.device(dev):
        model = LlamaDecoder(args).to(torch.bfloat16).eval().requires_grad_(False)
    model.init_weights(seed=1)
    model.reset_rope_tables()
    jstep = compile_decoder(GreedyStep(model))
    gen = torch.Generator().manual_seed(1234)
    prompt_dev = torch.randint(0, cfg.vocab, (batch, prompt_len), generator=gen).to(dev)
    tok = torch.empty((batch, 1), dtype=torch.int64, device=dev)
    pos = torch.zeros((1,), dtype=torch.int64, device=dev)
    tok.copy_(prompt_dev[:, :1])
    out = jstep(tok, pos)                       # first call: quantize, trace, fuse, capture
    torch.cuda.synchronize()
    t_first = time.perf_counter() - t0
    _log(f"thunder: first call after {t_first:.1f}s")
    # the rest of the prompt through the decode trace, token by token
    for t in range(1, prompt_len):
        tok.copy_(prompt_dev[:, t:t + 1])
        pos.fill_(t)
        out = jstep(tok, pos)
    pos.fill_(prompt_len)
    for _ in range(warmup):
        out = jstep(out, pos)
        pos.add_(1)
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        out = jstep(out, pos)                   # ids stay on the device
        pos.add_(1)
    host_issue_s = time.perf_counter() - w0
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)

    # end to end: ids and position come from pinned host memory every step, the sampled ids go back
    ids_host = torch.empty((batch, 1), dtype=torch.int64).pin_memory()
    pos_host = torch.empty((1,), dtype=torch.int64).pin_memory()
    out_host = torch.empty((batch, 1), dtype=torch.int64).pin_memory()
    ids_host.copy_(out.cpu())
    p = int(pos.item())
    for _ in range(warmup):
        pos_host[0] = p
        tok.copy_(ids_host, non_blocking=True)
        pos.copy_(pos_host, non_blocking=True)
        out = jstep(tok, pos)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        ids_host.copy_(out_host)
        p += 1
    torch.cuda.synchronize()
    w0 = time.perf_counter()
    for _ in range(steps):
        pos_host[0] = p
        tok.copy_(ids_host, non_blocking=True)
        pos.copy_(pos_host, non_blocking=True)
        out = jstep(tok, pos)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        ids_host.copy_(out_host)
        p += 1
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - w0

    # kernels per step: count the launches of one more call (outside the timed regions)
    launches = None
    try:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            jstep(tok, pos)
            torch.cuda.synchronize()
        launches = sum(1 for e in prof.events() if str(e.device_type).endswith("CUDA") and "Memcpy" not in e.name and "Memset" not in e.name)
    except Exception as exc:      # noqa: BLE001 - the count is informative only
        _log(f"kernel count unavailable: {exc}")
    fusion = jstep.nf4_fusion
    res = {"tok_s": steps * batch / (ms / 1e3), "ms_per_step": ms / steps, "e2e_tok_s": steps * batch / e2e_s,
           "e2e_ms_per_step": 1e3 * e2e_s / steps, "host_issue_ms_per_step": 1e3 * host_issue_s / steps,
           "launches_per_step": launches, "first_call_s": t_first, "fused_blocks": dict(fusion.fused),
           "declined": list(fusion.declined), "h2d_bytes_per_step": 8 * batch + 8, "d2h_bytes_per_step": 8 * batch,
           "device_error": list(_lib.device_error())}
    del jstep, model
    torch.cuda.empty_cache()
    return res


def run_prefill(args):
    """The prefill configuration (batch 8 x 2048 random token ids, causal) through the SAME jitted module: one call
    processes the whole prompt (16384 activation rows: the fused blocks run every linear on the tensor-core
    dequant-GEMM, RMSNorm / rotary + cache write / SiLU * up as single launches of this library, and the attention
    itself on torch's fused SDPA kernel).  Timed as thunder/benchmarks/benchmark_inference.py:200-206, 467-529 times prefill: synchronise,
    perf_counter around the call; tok/s = batch * prompt / time.  The GEMM's share of the step comes from a
    profiler pass over one more call."""
    import torch

    from nf4_b200 import decoder as D
    from nf4_b200.llama import LlamaArgs, LlamaDecoder
    from nf4_b200.thunder_decode import GreedyStep, compile_decoder

    torch.cuda.set_device(0)
    dev = "cuda:0"
    cfg = D.LLAMA3_8B
    B, T = args.B if args.B != 16 else 8, args.prompt or 2048
    la = LlamaArgs(dim=cfg.d_model, n_layers=cfg.n_layers, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads, vocab_size=cfg.vocab,
                   hidden_dim=cfg.ffn, norm_eps=cfg.norm_eps, rope_theta=cfg.rope_theta, max_seq_len=T, max_batch=B)
    with torch.device(dev):
        model = LlamaDecoder(la).to(torch.bfloat16).eval().requires_grad_(False)
    model.init_weights(seed=1)
    jstep = compile_decoder(GreedyStep(model), cuda_graph=False)
    gen = torch.Generator().manual_seed(1234)
    prompt = torch.randint(0, cfg.vocab, (B, T), generator=gen).to(dev)
    pos = torch.arange(T, device=dev)
    t0 = time.perf_counter()
    jstep(prompt, pos)
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    for _ in range(max(1, args.warmup)):
        jstep(prompt, pos)
    sampler = ClockSampler(0)
    sampler.start()
    times = []
    for _ in range(max(1, args.steps)):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        jstep(prompt, pos)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    clocks = sampler.stop()
    sec = statistics.median(times)
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        jstep(prompt, pos)
        torch.cuda.synchronize()
    by = {}
    for e in prof.events():
        if str(e.device_type).endswith("CUDA"):
            by[e.name] = by.get(e.name, 0.0) + e.device_time
    total_us = sum(by.values())
    gemm_us = sum(v for k, v in by.items() if "gemm_tcgen05" in k)
    top = sorted(by.items(), key=lambda kv: -kv[1])[:8]
    weights = cfg.n_layers * (((cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim) * cfg.d_model + cfg.d_model * cfg.n_heads * cfg.head_dim
                              + 3 * cfg.ffn * cfg.d_model)
    flops = 2.0 * B * T * weights
    peaks, src = measured_peaks()
    emit(({
        "metric": "NF4 W4A16 prefill tok/s (Llama-3-8B shape)", "value": B * T / sec, "unit": UNIT, "n_gpus": 1,
        "steps": len(times), "warmup": max(1, args.warmup), "ms_per_step": sec * 1e3, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": f"llama3-8b-shape NF4 prefill, batch {B} x {T} tokens, causal", "parallelism": "tp1"},
        "path": "thunder.jit(model, transforms=[NF4LinearQuant4bit, NF4DecodeFusion, PrunePrologueChecks]) on the NF4 executor: per layer RMSNorm, GEMM(q|k|v), rotary + cache write, torch SDPA over the cache, GEMM(wo), RMSNorm, GEMM(gate|up), SiLU*up, GEMM(w2)",
        "clocks": clocks, "first_call_s": first,
        "gemm": {"kernel": "gemm_tcgen05_kernel", "share_of_gpu_time": gemm_us / total_us if total_us else None,
                 "ms": gemm_us / 1e3, "TFLOPs_in_gemm_time": flops / (gemm_us * 1e-6) / 1e12 if gemm_us else None,
                 "frac_of_" + src: flops / (gemm_us * 1e-6) / 1e12 / peaks["bf16_tflops_sustained" if "bf16_tflops_sustained" in peaks else "bf16_tflops"]
                 if gemm_us else None},
        "gpu_time_ms": total_us / 1e3, "top_kernels_ms": [[k[:60], round(v / 1e3, 2)] for k, v in top],
    }))


def tp_parity(world, rank, group, dev):
    """Before timing a tensor-parallel run: a small model decoded at tp=world by all ranks and at tp=1 on rank 0
    from the same seeds and the SAME input ids every step (so one early near-tie cannot send the two runs down
    different sequences); the logits of every step are compared, and the sampled ids wherever the single-GPU
    run's best two logits are further apart than the tolerance."""
    import torch

    from nf4_b200.decoder import NF4Decoder, tiny_config

    cfg = tiny_config(n_layers=2, d_model=1024, n_heads=8, n_kv_heads=8, ffn=2048, vocab=4096)
    B, steps = 2, 8
    gen = torch.Generator().manual_seed(7)
    feed = torch.randint(0, cfg.vocab, (steps, B), generator=gen).to(dev)

    def run(tp_rank, tp_size, grp):
        dec = NF4Decoder(cfg, batch=B, max_seq=32, device=dev, seed=3, tp_rank=tp_rank, tp_size=tp_size, group=grp)
        ids, logits = [], []
        for t in range(steps):
            dec.ids_in.copy_(feed[t])
            dec.step()
            ids.append(dec.ids_out.clone())
            logits.append(dec.logits.float().clone())
        torch.cuda.synchronize()
        return torch.stack(ids), torch.stack(logits)

    ids_tp, logits_tp = run(rank, world, group)
    gathered = [torch.empty_like(logits_tp) for _ in range(world)]
    torch.distributed.all_gather(gathered, logits_tp, group=group)
    if rank != 0:
        return None
    ids_1, logits_1 = run(0, 1, None)
    full = torch.cat(gathered, dim=2)
    diff = (full - logits_1).abs()
    tol = 1e-2 + 1.6e-2 * logits_1.abs()
    top2 = logits_1.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 2 * (1e-2 + 1.6e-2 * top2[..., 0].abs())
    return {"config": "2 layers, d 1024, 8 heads, ffn 2048, vocab 4096, batch 2, 8 steps on the same input ids",
            "max_abs_logit_diff": float(diff.max()), "logit_scale": float(logits_1.abs().max()),
            "logits_outside_tolerance": float((diff > 3 * tol).float().mean()),
            "tokens_equal_where_clear": bool(torch.equal(ids_tp[clear], ids_1[clear])), "clear_steps": int(clear.sum()),
            "tokens_equal": bool(torch.equal(ids_tp, ids_1)),
            "tolerance": "3 x (atol 1e-2 + rtol 1.6e-2): the per-linear tolerance through a 2-layer model; partial sums are "
                         "rounded to bf16 before the exchange"}


def run_decode(args):
    import torch

    from nf4_b200 import decoder as D

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    workload = args.workload or ("llama3-8b" if world == 1 else "llama3-70b")
    attr, batch, prompt_len, new_tokens = WORKLOADS[workload]
    cfg = getattr(D, attr) if attr else D.tiny_config()
    if args.prompt is not None:
        prompt_len = args.prompt
    steps, warmup = args.steps, max(3, args.warmup)
    peaks, src = measured_peaks()

    # Rank 0 does its host-only and single-GPU work BEFORE the process group exists: the other ranks wait in the
    # rendezvous (a socket, no GPU work) instead of spinning a GPU in a collective.
    cpu = anchor = None
    if rank == 0:
        _log("CPU baseline")
        # (one pass when other ranks are waiting for this one: at 16 rows a pass of the 70B layer takes ~8 s)
        cpu = cpu_decode_sample(workload if workload != "tiny" else "llama3-8b", batch, 3 if world == 1 else 1)
        if world > 1 and not args.no_anchor:
            _log("tp1 anchor of the same workload")
            anchor = engine_decode(cfg, batch, prompt_len, steps, warmup, dev, 0, 1, None, feed_prompt=False, roofline=False)
    group = None
    parity = None
    if world > 1:
        import datetime

        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(dev), timeout=datetime.timedelta(minutes=30))
        group = dist.group.WORLD
        parity = tp_parity(world, rank, group, dev)

    sampler = ClockSampler(local) if rank == 0 else None
    th = None
    if world == 1 and not args.no_thunder:
        try:
            th = thunder_decode(cfg, batch, prompt_len, steps, warmup, dev, sampler=sampler)
        except ImportError as exc:
            th = {"unavailable": f"thunder is not importable here: {exc}"}
    eng = engine_decode(cfg, batch, prompt_len, steps, warmup, dev, rank, world, group, feed_prompt=(world == 1),
                        sampler=sampler if (th is None or "unavailable" in th) else None)
    clocks = sampler.stop() if sampler is not None else None

    def finish():
        # Tearing down NCCL communicators that captured graphs still reference can block at exit:
        # meet once more, flush, and leave without running destructors.
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            torch.distributed.barrier()
            torch.cuda.synchronize()
            os._exit(0)

    if rank != 0:
        finish()
        return

    cpu_tok_s, t_layer, cores, _ = cpu
    gemv_bytes, chain_us = eng["gemv_bytes"], eng["chain_us"]
    achieved = sum(gemv_bytes) / chain_us / 1e3           # GB/s over all GEMV launches of a step
    use_thunder = th is not None and "unavailable" not in th
    head = th if use_thunder else eng
    line = {
        "metric": metric_name(workload, world), "value": head["tok_s"], "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
        "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(cfg.name, batch, prompt_len, world, eng["step_bytes"]),
        "clocks": clocks,
        "path": ("thunder.jit(model, transforms=[NF4LinearQuant4bit, NF4DecodeFusion, PrunePrologueChecks, CUDAGraphTransform], "
                 "executors=[quant_nf4_b200]) called once per token, ids fed back on the device") if use_thunder else
                "decode engine (NF4Decoder: the C ABI called directly, one CUDA graph per step), ids fed back on the device",
        "e2e": {"value": head["e2e_tok_s"], "unit": UNIT,
                "h2d_bytes_per_step": th["h2d_bytes_per_step"] if use_thunder else 8 * batch,
                "d2h_bytes_per_step": 8 * batch,
                "path": "the jitted module called with token ids and position from pinned host memory; sampled ids read back each step"
                        if use_thunder else "NF4Decoder.run_step() with ids from pinned host memory; sampled ids read back each step"},
        "gpu_launches": (head["launches_per_step"] or eng["launches_per_step"]) * steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_source": src,
                     "traffic": NCU_TRAFFIC_RATIO * sum(gemv_bytes) / len(gemv_bytes),
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at 32064x4096, M=1 "
                                       "(75.01 MB for 73.95 MB algorithmic), scaled by algorithmic bytes",
                     "kernel": "gemv_staged_kernel (fused NF4 dequant-GEMV)", "launches_per_step": len(gemv_bytes),
                     "avg_launch_us": chain_us / len(gemv_bytes), "algorithmic_bytes_per_launch": sum(gemv_bytes) / len(gemv_bytes),
                     "frac_of_8TBps": achieved / 8000.0,
                     "whole_step_GBps": eng["step_bytes"] / (head["ms_per_step"] / 1e3) / 1e9},
        "cpu_baseline": {"value": cpu_tok_s, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"the 4 quantized linears of one decoder layer at M={batch} on the CPU oracle, median of "
                                   f"{cpu[3]} pass(es) ({t_layer * 1e3:.1f} ms each), scaled to all layers + output head"},
        "engine": {"tok_s": eng["tok_s"], "ms_per_step": eng["ms_per_step"], "e2e_tok_s": eng["e2e_tok_s"],
                   "launches_per_step": eng["launches_per_step"], "build_s": eng["build_s"]},
        "device_error": eng["device_error"],
    }
    if th is not None:
        line["thunder"] = {k: v for k, v in th.items() if k != "device_error"}
        if use_thunder:
            line["thunder"]["vs_engine"] = th["tok_s"] / eng["tok_s"]
    if anchor is not None:
        line["tp1_same_workload_tok_s"] = anchor["tok_s"]
        line["tp1_same_workload_ms_per_step"] = anchor["ms_per_step"]
        line["speedup_vs_tp1_same_workload"] = eng["tok_s"] / anchor["tok_s"]
    if parity is not None:
        line["tp_parity"] = parity
    if "nccl_exchange_tok_s" in eng:
        line["exchange"] = {"kind": eng["exchange"], "tok_s": eng["tok_s"], "nccl_all_reduce_tok_s": eng["nccl_exchange_tok_s"],
                            "nccl_all_reduce_ms_per_step": eng["nccl_exchange_ms_per_step"]}
    emit(line)
    finish()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128, help="timed steps (decode: tokens generated; the workload's 128 new tokens by default)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "llama3-8b", "llama3-70b", "tiny", "llama3-8b-prefill"])
    ap.add_argument("--prompt", type=int, default=None, help="override the prompt length")
    ap.add_argument("--no-thunder", action="store_true", help="N = 1: time only the decode engine, not the jitted module")
    ap.add_argument("--no-anchor", action="store_true", help="N > 1: skip the single-GPU run of the same workload")
    ap.add_argument("--kernel", default=None, choices=[None, "gemv", "gemm", "quantize", "dequantize", "attention"])
    ap.add_argument("--B", type=int, default=16, help="attention: sequences")
    ap.add_argument("--Hq", type=int, default=64, help="attention: query heads")
    ap.add_argument("--Hkv", type=int, default=8, help="attention: key/value heads")
    ap.add_argument("--ctx", type=int, default=1024, help="attention: cached positions per sequence")
    ap.add_argument("--splits", type=int, default=0, help="attention: splits along the sequence (0: the decoder's rule)")
    ap.add_argument("--N", type=int, default=14336)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--M", type=int, default=1)
    ap.add_argument("--nbuf", type=int, default=None)
    ap.add_argument("--dq", action="store_true", help="--kernel gemv/gemm: double-quantized absmax (8-bit, blocks of 256)")
    args = ap.parse_args()
    _claim_stdout()
    if args.impl == "reference":
        run_reference(args)
    elif args.kernel == "attention":
        run_attention(args)
    elif args.kernel:
        run_kernel(args)
    elif args.workload == "llama3-8b-prefill":
        run_prefill(args)
    else:
        run_decode(args)


if __name__ == "__main__":
    main()
