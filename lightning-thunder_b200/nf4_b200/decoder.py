"""A Llama-shaped decoder whose every nn.Linear is an NF4 weight (the model the reference's
transform produces from thunder/tests/llama2_model.py:129-290 -- RMSNorm, rotary embedding on
interleaved pairs, grouped-query attention with a KV cache, SwiGLU MLP, untied output head), run
as a chain of launches of this library's kernels and captured in one CUDA graph per decode step.

Weights are random (N(0, 0.02), seeded per tensor) because the benchmark configurations are
random-init.  Q, K and V share one quantized matrix
(rows concatenated), as do gate and up (rows interleaved): a 64-element quantization block never
crosses a row when K % 64 == 0, so the fused matrix holds exactly the bytes of the separate ones.

Tensor parallelism (one process per GPU): Q/K/V and gate/up are split by rows (heads, FFN columns),
the attention-output and down projections by columns (each rank quantizes its own shard, no
collective), their partial outputs meet in an NCCL all-reduce, and the vocabulary is split for the
output head (local argmax, then an all-gather of the candidates).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib, parallel
from .functional import nf4_code, quantize_4bit


@dataclass(frozen=True)
class DecoderConfig:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    name: str = "custom"


LLAMA3_8B = DecoderConfig(32, 4096, 32, 8, 128, 14336, 128256, name="llama3-8b-shape")
LLAMA3_70B = DecoderConfig(80, 8192, 64, 8, 128, 28672, 128256, name="llama3-70b-shape")


def tiny_config(n_layers=2, d_model=512, n_heads=4, n_kv_heads=2, ffn=1024, vocab=2048) -> DecoderConfig:
    """A small model with the same head geometry (head_dim 128, grouped KV heads) for tests."""
    return DecoderConfig(n_layers, d_model, n_heads, n_kv_heads, d_model // n_heads, ffn, vocab, name="tiny")


class NF4Weight:
    """packed / absmax / code of one [N, K] matrix."""

    __slots__ = ("packed", "absmax", "code", "N", "K")

    def __init__(self, w: torch.Tensor):
        assert w.dim() == 2 and w.is_cuda
        self.N, self.K = w.shape
        self.packed, qs = quantize_4bit(w.contiguous())
        self.absmax = qs.absmax
        self.code = nf4_code(w.device)

    def nbytes(self) -> int:
        return self.packed.numel() + self.absmax.numel() * 4


def _seeded_normal(shape, seed: int, device, std=0.02) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


class NF4Decoder:
    def __init__(self, cfg: DecoderConfig, batch: int, max_seq: int, device="cuda:0", seed: int = 0, tp_rank: int = 0,
                 tp_size: int = 1, group=None, attn_splits: int | None = None, fused: bool = True, pdl: bool = True,
                 tensor_core_from: int = 17, prefetch_next: bool = True, tp_reduce: str = "oneshot"):
        assert cfg.head_dim == 128, "the attention kernel is written for head_dim 128"
        parallel.check_shardable(cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, tp_size)
        assert batch <= 16
        self.cfg, self.B, self.S = cfg, batch, max_seq
        self.dev = torch.device(device)
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        self.lib = _lib.load()
        if attn_splits is None:
            # enough CTAs (kv heads x rows x splits) to cover the SMs twice, but at least ~96 cached
            # positions per CTA (shorter ranges are all start-up and merge); the rule of functional.attn_splits
            attn_splits = max(1, min(16, 296 // max(1, (cfg.n_kv_heads // tp_size) * batch), max_seq // 96))
        self.attn_splits = attn_splits
        # fused: RMSNorm and SiLU*up run as prologues of the following GEMV (where the activations fit
        # in shared memory), rotary embedding + KV append + attention + merge are one launch.
        # pdl: those launches use programmatic dependent launch (weight streaming of a kernel overlaps
        # the tail of its predecessor).
        self.fused = fused
        self.flags = 1 if (fused and pdl) else 0
        # from this many sequences on, the fused step's linears run on the tensor-core kernel (K split over
        # thread blocks, residual / SwiGLU epilogues) with RMSNorm as a separate small kernel before it;
        # up to 16 sequences the GEMV measures faster on every layer shape, so that is the default
        self.tensor_core = fused and batch >= tensor_core_from
        # every GEMV of the fused step tells the library which weight the next launch streams, so the head
        # of it is pulled into L2 across the kernel boundary
        self.prefetch_next = fused and prefetch_next
        self.Hq = cfg.n_heads // tp_size
        self.Hkv = cfg.n_kv_heads // tp_size
        self.F = cfg.ffn // tp_size
        self.V = cfg.vocab // tp_size
        D, Dh = cfg.d_model, cfg.head_dim
        dev, bf = self.dev, torch.bfloat16
        with torch.cuda.device(dev):
            self.embed = _seeded_normal((cfg.vocab, D), seed * 1000003 + 1, dev)
            self.layers = []
            for li in range(cfg.n_layers):
                base = seed * 1000003 + 100 * (li + 1)
                self.layers.append(self._make_layer(base))
            self.final_norm = torch.ones(D, device=dev, dtype=bf)
            w = _seeded_normal((cfg.vocab, D), seed * 1000003 + 7, dev)
            self.lm_head = NF4Weight(parallel.shard_rows(w, self.tp_rank, tp_size))
            del w
            L, B, S = cfg.n_layers, batch, max_seq
            self.k_cache = torch.zeros((L, B, self.Hkv, S, Dh), device=dev, dtype=bf)
            self.v_cache = torch.zeros((L, B, self.Hkv, S, Dh), device=dev, dtype=bf)
            self.ids_in = torch.zeros((B,), device=dev, dtype=torch.int64)
            self.ids_out = torch.zeros((B,), device=dev, dtype=torch.int64)
            self.positions = torch.zeros((B,), device=dev, dtype=torch.int32)
            self.x = torch.empty((B, D), device=dev, dtype=bf)
            self.xn = torch.empty((B, D), device=dev, dtype=bf)
            self.qkv = torch.empty((B, (self.Hq + 2 * self.Hkv) * Dh), device=dev, dtype=bf)
            self.q = torch.empty((B, self.Hq * Dh), device=dev, dtype=bf)
            self.attn = torch.empty((B, self.Hq * Dh), device=dev, dtype=bf)
            self.gu = torch.empty((B, 2 * self.F), device=dev, dtype=bf)
            self.h = torch.empty((B, self.F), device=dev, dtype=bf)
            self.part = torch.empty((B, D), device=dev, dtype=bf)
            self.logits = torch.empty((B, self.V), device=dev, dtype=bf)
            ws = self.lib.nf4_b200_attn_decode_workspace_bytes(B, self.Hq, attn_splits)
            self.attn_ws = torch.empty((ws,), device=dev, dtype=torch.uint8)
            self.attn_counters = torch.zeros((B * self.Hkv,), device=dev, dtype=torch.int32)
            shapes = [(self.lm_head.N, self.lm_head.K)] + [(l[k].N, l[k].K) for l in self.layers[:1] for k in ("qkv", "o", "gu", "down")]
            gws = max(self.lib.nf4_b200_gemm_workspace_bytes(B, n, k) for n, k in shapes) if self.tensor_core else 0
            self.gemm_ws = torch.zeros((max(gws, 16),), device=dev, dtype=torch.uint8)   # zero once; the kernels keep it so
            if tp_size > 1:
                self.cand = torch.empty((B, 2), device=dev, dtype=torch.float32)
                self.cand_all = torch.empty((tp_size, B, 2), device=dev, dtype=torch.float32)
        # the exchange after the row-parallel projections: "oneshot" = this library's all-reduce over peer
        # memory (x += sum of the ranks' partial tiles in one launch), "nccl" = torch.distributed.all_reduce
        self.oneshot = None
        if tp_size > 1 and tp_reduce == "oneshot":
            from .tp_comm import OneShotAllReduce

            self.oneshot = OneShotAllReduce(group, dev, batch * cfg.d_model)
        self.graph = None
        self.next_pos = 0           # host mirror of the highest position the next step writes (see _guard)
        self.launches_per_step = 0
        self.gemv_events = None     # set to a list to collect (start, stop, algorithmic bytes) per GEMV launch

    # ------------------------------------------------------------------------------ weights
    def _make_layer(self, base: int) -> dict:
        cfg, dev, r, tp = self.cfg, self.dev, self.tp_rank, self.tp_size
        D, Dh = cfg.d_model, cfg.head_dim
        wq = _seeded_normal((cfg.n_heads * Dh, D), base + 1, dev)
        wk = _seeded_normal((cfg.n_kv_heads * Dh, D), base + 2, dev)
        wv = _seeded_normal((cfg.n_kv_heads * Dh, D), base + 3, dev)
        qkv = parallel.shard_qkv(wq, wk, wv, r, tp)
        del wq, wk, wv
        wo = parallel.shard_cols(_seeded_normal((D, cfg.n_heads * Dh), base + 4, dev), r, tp)
        wg = _seeded_normal((cfg.ffn, D), base + 5, dev)
        wu = _seeded_normal((cfg.ffn, D), base + 6, dev)
        # rows interleaved (gate_0, up_0, gate_1, up_1, ...) so the GEMV epilogue can apply SwiGLU
        gu = parallel.shard_gate_up(wg, wu, r, tp)
        del wg, wu
        wd = parallel.shard_cols(_seeded_normal((D, cfg.ffn), base + 7, dev), r, tp)
        layer = {
            "qkv": NF4Weight(qkv), "o": NF4Weight(wo), "gu": NF4Weight(gu), "down": NF4Weight(wd),
            "norm1": torch.ones(D, device=dev, dtype=torch.bfloat16),
            "norm2": torch.ones(D, device=dev, dtype=torch.bfloat16),
        }
        del qkv, wo, gu, wd
        return layer

    def weight_bytes(self) -> int:
        """Bytes of packed codes + absmax one decode step streams on this rank."""
        n = self.lm_head.nbytes()
        for layer in self.layers:
            n += sum(layer[k].nbytes() for k in ("qkv", "o", "gu", "down"))
        return n

    # ------------------------------------------------------------------------------ one step
    def _linear(self, x, w: NF4Weight, y, residual=None, stream=None):
        M = x.shape[0]
        ev = self._ev_begin()
        _lib.check(self.lib.nf4_b200_gemv_fused(x.data_ptr(), M, w.K, w.packed.data_ptr(), w.absmax.data_ptr(),
                                                w.code.data_ptr(), w.N, None,
                                                residual.data_ptr() if residual is not None else None, y.data_ptr(),
                                                _lib.NF4_BF16, stream), "nf4_b200_gemv_fused")
        self._ev_end(ev, w, M)
        self._n += 1

    def _all_reduce(self, t):
        torch.distributed.all_reduce(t, group=self.group)

    def _row_parallel(self, inp, w: "NF4Weight", st, next_w=None) -> None:
        """x <- x + sum over ranks of (inp . W_shard^T): a row-parallel projection and its exchange."""
        if self.oneshot is not None:
            self._linear_decode(inp, w, self.part, stream=st, next_w=next_w)
            self.oneshot(self.part, residual=self.x, out=self.x, pdl=bool(self.flags & 1))
            self._n += 1
        else:
            # rank 0 carries the residual into the sum; the all-reduce completes x = x + inp . W^T
            self._linear_decode(inp, w, self.part, residual=self.x if self.tp_rank == 0 else None, stream=st, next_w=next_w)
            self._all_reduce(self.part)
            self.x, self.part = self.part, self.x          # two swaps per layer: the roles are back after the step

    def _linear_decode(self, x, w: NF4Weight, y, residual=None, prologue=0, norm_w=None, swiglu=False, stream=None,
                       next_w: NF4Weight | None = None):
        """GEMV with an optional fused prologue (RMSNorm) and epilogue (SwiGLU over interleaved gate/up
        rows); falls back to separate glue kernels around a plain GEMV when the shape does not fit."""
        lib, cfg, B = self.lib, self.cfg, self.B
        ck = _lib.check
        if self.tensor_core:
            if prologue == 1:
                ck(lib.nf4_b200_rmsnorm(x.data_ptr(), norm_w.data_ptr(), self.xn.data_ptr(), B, w.K, cfg.norm_eps, stream), "rmsnorm")
                x = self.xn
                self._n += 1
            elif prologue == 2:
                ck(lib.nf4_b200_silu_mul(x.data_ptr(), self.h.data_ptr(), B, w.K, 0, stream), "silu_mul")
                x = self.h
                self._n += 1
            ev = self._ev_begin()
            ck(lib.nf4_b200_gemm_decode(x.data_ptr(), B, w.K, w.packed.data_ptr(), w.absmax.data_ptr(), w.code.data_ptr(), w.N,
                                        residual.data_ptr() if residual is not None else None, y.data_ptr(), 1 if swiglu else 0,
                                        self.gemm_ws.data_ptr(), self.gemm_ws.numel(), self.flags, stream),
               "nf4_b200_gemm_decode")
            self._ev_end(ev, w, B)
            self._n += 1
            return
        if prologue and not lib.nf4_b200_gemv_decode_fits(B, w.N, w.K, prologue):
            # the activations do not fit beside the kernel's tables (more than 8 rows of a wide model): the prologue
            # runs as its own launch; the epilogue does not depend on that and stays fused
            if prologue == 1:
                ck(lib.nf4_b200_rmsnorm(x.data_ptr(), norm_w.data_ptr(), self.xn.data_ptr(), B, w.K, cfg.norm_eps, stream), "rmsnorm")
                x = self.xn
            else:
                ck(lib.nf4_b200_silu_mul(x.data_ptr(), self.h.data_ptr(), B, w.K, 0, stream), "silu_mul")
                x = self.h
            self._n += 1
            prologue, norm_w = 0, None
        if swiglu and not lib.nf4_b200_gemv_decode_fits(B, w.N, w.K, prologue):
            self._linear_decode(x, w, self.gu, prologue=prologue, norm_w=norm_w, stream=stream)
            ck(lib.nf4_b200_silu_mul(self.gu.data_ptr(), y.data_ptr(), B, w.N // 2, 1, stream), "silu_mul")
            self._n += 1
            return
        if next_w is not None and self.prefetch_next:
            ck(lib.nf4_b200_gemv_decode_next_weight(next_w.packed.data_ptr(), next_w.absmax.data_ptr(), next_w.N, next_w.K),
               "nf4_b200_gemv_decode_next_weight")
        ev = self._ev_begin()
        ck(lib.nf4_b200_gemv_decode(x.data_ptr(), B, w.K, w.packed.data_ptr(), w.absmax.data_ptr(), w.code.data_ptr(), w.N,
                                    residual.data_ptr() if residual is not None else None, y.data_ptr(), prologue,
                                    norm_w.data_ptr() if norm_w is not None else None, cfg.norm_eps, 1 if swiglu else 0,
                                    self.flags, stream),
           "nf4_b200_gemv_decode")
        self._ev_end(ev, w, B)
        self._n += 1

    def _ev_begin(self):
        if self.gemv_events is None:
            return None
        a = torch.cuda.Event(enable_timing=True)
        a.record()
        return a

    def _ev_end(self, a, w, M):
        if a is not None:
            b = torch.cuda.Event(enable_timing=True)
            b.record()
            self.gemv_events.append((a, b, w.nbytes() + 2 * M * (w.K + w.N)))

    def _guard(self) -> None:
        """The kernels index the KV cache at `positions`; refuse on the host to step past the cache."""
        if self.next_pos >= self.S:
            raise RuntimeError(f"NF4Decoder: the KV cache holds {self.S} positions and all are used; "
                               "reset() or build the decoder with a larger max_seq")
        self.next_pos += 1

    def set_positions(self, pos: int) -> None:
        """All sequences continue at cache row `pos` (rows below it keep their contents)."""
        if not 0 <= pos < self.S:
            raise ValueError(f"position {pos} outside the cache [0, {self.S})")
        self.positions.fill_(pos)
        self.next_pos = pos

    def step(self) -> None:
        """One decode step on the current stream: ids_in, positions -> ids_out; positions += 1."""
        if not torch.cuda.is_current_stream_capturing():
            self._guard()
        if self.fused:
            return self._step_fused()
        return self._step_unfused()

    def _step_fused(self) -> None:
        cfg, lib, B = self.cfg, self.lib, self.B
        D, Dh = cfg.d_model, cfg.head_dim
        st = ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        ck = _lib.check
        self._n = 0
        tp = self.tp_size > 1
        ck(lib.nf4_b200_embed(self.ids_in.data_ptr(), self.embed.data_ptr(), self.x.data_ptr(), B, D, cfg.vocab, st), "embed")
        self._n += 1
        for li, layer in enumerate(self.layers):
            after = self.layers[li + 1]["qkv"] if li + 1 < len(self.layers) else self.lm_head
            self._linear_decode(self.x, layer["qkv"], self.qkv, prologue=1, norm_w=layer["norm1"], stream=st, next_w=layer["o"])
            ck(lib.nf4_b200_attn_decode_fused(self.qkv.data_ptr(), self.positions.data_ptr(), self.k_cache[li].data_ptr(),
                                              self.v_cache[li].data_ptr(), self.attn.data_ptr(), self.attn_ws.data_ptr(),
                                              self.attn_counters.data_ptr(), B, self.Hq, self.Hkv, Dh, self.S,
                                              self.attn_splits, cfg.rope_theta, self.flags, st), "attn_decode_fused")
            self._n += 1
            if tp:
                self._row_parallel(self.attn, layer["o"], st, next_w=layer["gu"])
            else:
                self._linear_decode(self.attn, layer["o"], self.x, residual=self.x, stream=st, next_w=layer["gu"])
            self._linear_decode(self.x, layer["gu"], self.h, prologue=1, norm_w=layer["norm2"], swiglu=True, stream=st,
                                next_w=layer["down"])
            if tp:
                self._row_parallel(self.h, layer["down"], st, next_w=after)
            else:
                self._linear_decode(self.h, layer["down"], self.x, residual=self.x, stream=st, next_w=after)
        self._linear_decode(self.x, self.lm_head, self.logits, prologue=1, norm_w=self.final_norm, stream=st)
        ck(lib.nf4_b200_argmax(self.logits.data_ptr(), self.ids_out.data_ptr(), B, self.V, st), "argmax")
        self._n += 1
        self._finish_step()

    def linears_only(self) -> None:
        """Launches only the quantized linears of one fused decode step (same shapes, prologues, epilogues and
        launch flags, no glue kernels, no collectives): the benchmark captures this chain in a CUDA graph to
        time the GEMV by itself under the step's own conditions (cold weights, back-to-back dependent launches)."""
        st = ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        self._n = 0
        tp = self.tp_size > 1
        for li, layer in enumerate(self.layers):
            after = self.layers[li + 1]["qkv"] if li + 1 < len(self.layers) else self.lm_head
            self._linear_decode(self.x, layer["qkv"], self.qkv, prologue=1, norm_w=layer["norm1"], stream=st, next_w=layer["o"])
            self._linear_decode(self.attn, layer["o"], self.part if tp else self.x, residual=self.x, stream=st, next_w=layer["gu"])
            self._linear_decode(self.x, layer["gu"], self.h, prologue=1, norm_w=layer["norm2"], swiglu=True, stream=st,
                                next_w=layer["down"])
            self._linear_decode(self.h, layer["down"], self.part if tp else self.x, residual=self.x, stream=st, next_w=after)
        self._linear_decode(self.x, self.lm_head, self.logits, prologue=1, norm_w=self.final_norm, stream=st)

    def _finish_step(self) -> None:
        if self.tp_size > 1:
            # candidates (value, global index) of every rank; the first maximum in rank order wins
            self.cand.copy_(parallel.local_candidates(self.logits, self.ids_out, self.tp_rank, self.V))
            torch.distributed.all_gather_into_tensor(self.cand_all, self.cand, group=self.group)
            self.ids_out.copy_(parallel.merge_candidates(self.cand_all))
        self.positions.add_(1)
        self.launches_per_step = self._n

    def _step_unfused(self) -> None:
        cfg, lib, B = self.cfg, self.lib, self.B
        D, Dh = cfg.d_model, cfg.head_dim
        st = ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        ck = _lib.check
        self._n = 0
        tp = self.tp_size > 1
        ck(lib.nf4_b200_embed(self.ids_in.data_ptr(), self.embed.data_ptr(), self.x.data_ptr(), B, D, cfg.vocab, st), "embed")
        self._n += 1
        for li, layer in enumerate(self.layers):
            ck(lib.nf4_b200_rmsnorm(self.x.data_ptr(), layer["norm1"].data_ptr(), self.xn.data_ptr(), B, D, cfg.norm_eps, st), "rmsnorm")
            self._linear(self.xn, layer["qkv"], self.qkv, stream=st)
            ck(lib.nf4_b200_rope_append(self.qkv.data_ptr(), self.positions.data_ptr(), self.q.data_ptr(),
                                        self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(), B, self.Hq, self.Hkv, Dh,
                                        self.S, cfg.rope_theta, st), "rope_append")
            ck(lib.nf4_b200_attn_decode(self.q.data_ptr(), self.k_cache[li].data_ptr(), self.v_cache[li].data_ptr(),
                                        self.positions.data_ptr(), self.attn.data_ptr(), self.attn_ws.data_ptr(), B, self.Hq,
                                        self.Hkv, Dh, self.S, self.attn_splits, st), "attn_decode")
            self._n += 4
            if tp:
                # rank 0 carries the residual into the sum; the all-reduce completes x = x + attn.Wo^T
                self._linear(self.attn, layer["o"], self.part, residual=self.x if self.tp_rank == 0 else None, stream=st)
                self._all_reduce(self.part)
                self.x, self.part = self.part, self.x   # two swaps per layer: the roles are back after the step
            else:
                self._linear(self.attn, layer["o"], self.x, residual=self.x, stream=st)
            ck(lib.nf4_b200_rmsnorm(self.x.data_ptr(), layer["norm2"].data_ptr(), self.xn.data_ptr(), B, D, cfg.norm_eps, st), "rmsnorm")
            self._linear(self.xn, layer["gu"], self.gu, stream=st)
            ck(lib.nf4_b200_silu_mul(self.gu.data_ptr(), self.h.data_ptr(), B, self.F, 1, st), "silu_mul")
            self._n += 2
            if tp:
                self._linear(self.h, layer["down"], self.part, residual=self.x if self.tp_rank == 0 else None, stream=st)
                self._all_reduce(self.part)
                self.x, self.part = self.part, self.x
            else:
                self._linear(self.h, layer["down"], self.x, residual=self.x, stream=st)
        ck(lib.nf4_b200_rmsnorm(self.x.data_ptr(), self.final_norm.data_ptr(), self.xn.data_ptr(), B, D, cfg.norm_eps, st), "rmsnorm")
        self._linear(self.xn, self.lm_head, self.logits, stream=st)
        ck(lib.nf4_b200_argmax(self.logits.data_ptr(), self.ids_out.data_ptr(), B, self.V, st), "argmax")
        self._n += 2
        self._finish_step()

    # ------------------------------------------------------------------------------ driving it
    def capture(self, feed_back: bool = False):
        """Captures step() in a CUDA graph and makes it the one run_step() replays.  feed_back=True
        also copies ids_out to ids_in inside the graph (a device-resident greedy loop); otherwise the
        host provides ids_in every step.  Returns the graph (several may be kept and swapped)."""
        # Warm-up outside capture: first calls create tensor maps, set kernel attributes, init NCCL.
        pos0, next0 = self.positions.clone(), self.next_pos
        if self.next_pos + 2 > self.S:
            raise RuntimeError("NF4Decoder.capture: needs two free cache rows for its warm-up steps")
        s = torch.cuda.Stream(device=self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            for _ in range(2):
                self.step()
        torch.cuda.current_stream(self.dev).wait_stream(s)
        torch.cuda.synchronize(self.dev)
        self.positions.copy_(pos0)
        self.graph = torch.cuda.CUDAGraph()
        # NCCL's watchdog thread polls events while we capture: keep its calls from invalidating it
        mode = "thread_local" if self.tp_size > 1 else "global"
        with torch.cuda.graph(self.graph, capture_error_mode=mode):
            self.step()
            if feed_back:
                self.ids_in.copy_(self.ids_out)
        self.positions.copy_(pos0)
        self.next_pos = next0
        return self.graph

    def run_step(self) -> None:
        if self.graph is not None:
            self._guard()
            self.graph.replay()
        else:
            self.step()

    def reset(self) -> None:
        self.positions.zero_()
        self.next_pos = 0

    def generate(self, prompt: torch.Tensor, n_new: int) -> torch.Tensor:
        """prompt [B, T] int64 (host or device).  Feeds the prompt one token per step (filling the KV
        cache), then decodes n_new tokens greedily.  Returns [B, n_new] int64 on the host."""
        B, T = prompt.shape
        assert B == self.B and T + n_new <= self.S
        prompt = prompt.to(self.dev)
        self.reset()
        out = torch.empty((B, n_new), dtype=torch.int64, device=self.dev)
        for t in range(T):
            self.ids_in.copy_(prompt[:, t])
            self.run_step()
        for t in range(n_new):
            out[:, t] = self.ids_out
            if t + 1 < n_new:
                self.ids_in.copy_(self.ids_out)
                self.run_step()
        torch.cuda.synchronize(self.dev)
        return out.cpu()
