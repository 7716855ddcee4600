"""Block fusions for Thunder-jitted Llama-shaped models on the NF4 executor.

After `NF4LinearQuant4bit` has replaced every `linear` by `nf4_b200_matmul`, a decoder layer is
still ~70 small torch ops around 7 quantized linears.  `NF4DecodeFusion` is a second trace pass
that recognises, by dataflow, the three shapes a Llama-shaped decode step is made of and replaces
each by ONE symbol of the same executor (`thunder.extend.OperatorExecutor.register_operator`,
thunder/extend/__init__.py:141-200), whose implementation is a short chain of this library's
fused kernels:

    attention block   x + wo(attention(rope(wq(n)), cache <- rope(wk(n)), cache <- wv(n))),  n = rms_norm(x)
                      -> GEMV(q|k|v rows, RMSNorm prologue) -> rotary + KV append + attention (one
                         launch) -> GEMV(wo, residual epilogue)                       3 launches
    MLP block         h + w2(silu(w1(n)) * w3(n)),  n = rms_norm(h)
                      -> GEMV(gate|up rows, RMSNorm prologue, SwiGLU epilogue) -> GEMV(w2, residual)
                                                                                      2 launches
    norm + linear     w(rms_norm(x))  (the output head)                               1 launch

The same three symbols also cover traces with more activation rows (a prompt of T > 1 tokens, or more
than 16 sequences): their implementations then run RMSNorm, the rotary embedding + cache write and
SiLU * up as single launches of this library around the tensor-core dequant-GEMM (one GEMM over the
q|k|v rows, one over the gate|up rows) and leave the attention itself to torch's fused SDPA kernels --
instead of the dozens of eager element-wise launches per layer the unfused trace is executed with.
The pass changes no parameter name, shape or value: to let Q, K and V (and gate and up) stream as
one matrix it re-homes their packed codes and absmax into one allocation each and leaves the
module's entries as views into it (a 64-element quantization block never crosses a row, so the
bytes are those of the separately quantized weights).

    jm = thunder.jit(model, executors=[get_nf4_executor()],
                     transforms=[NF4LinearQuant4bit(), NF4DecodeFusion(), CUDAGraphTransform()])
"""

from __future__ import annotations

import math
from collections import defaultdict

import torch

from . import functional
from .thunder_executor import get_nf4_executor, thunder

from thunder.core import prims  # noqa: E402
from thunder.core.proxies import TensorProxy  # noqa: E402
from thunder.core.trace import TraceProvenance, from_trace, tracectx  # noqa: E402
from thunder.core.transform_common import Transform, dce  # noqa: E402

HEAD_DIM = 128          # the attention kernel's head size
MAX_ROWS = 16           # the fused GEMV's limit on activation rows

_symbols = None


# ---------------------------------------------------------------------------------------------------
# run-time side: the implementations of the block symbols
# ---------------------------------------------------------------------------------------------------

_span_cache: dict = {}


def _span(parts, what: str) -> torch.Tensor:
    """One tensor covering `parts` (1-D or [n, 1] tensors that the pass placed back to back in one
    allocation).  If somebody has replaced a part since (e.g. load_state_dict(assign=True)), the parts
    are gathered into a new allocation, kept for later calls."""
    first = parts[0]
    total = sum(p.numel() for p in parts)
    end = first.data_ptr()
    adjacent = True
    for p in parts:
        adjacent = adjacent and p.data_ptr() == end and p.is_contiguous()
        end += p.numel() * p.element_size()
    if adjacent and first.untyped_storage().nbytes() - first.storage_offset() * first.element_size() >= total * first.element_size():
        return first.as_strided((total,), (1,), first.storage_offset())
    key = tuple((p.data_ptr(), p.numel(), p._version) for p in parts)
    hit = _span_cache.get(key)
    if hit is None:
        if first.is_cuda and torch.cuda.is_current_stream_capturing():
            raise RuntimeError(f"nf4_b200 fusion: the {what} tensors are no longer adjacent in memory and a CUDA graph is "
                               "being captured; call the module once outside of the capture first")
        hit = _span_cache[key] = torch.cat([p.reshape(-1) for p in parts])
    return hit


def _rmsnorm_rows(x2, norm_w, eps):
    return functional.rms_norm_rows(x2, norm_w, eps)


def _gemv(x2, packed, absmax, code, N, K, *, norm_w=None, eps=0.0, epilogue=0, residual=None, pdl=True, next_weight=None):
    """Fused GEMV with an optional RMSNorm prologue; when the activations do not fit beside the kernel's
    tables the norm runs as its own op first."""
    F = functional
    M = x2.shape[0]
    prologue = F.PROLOGUE_RMSNORM if norm_w is not None else F.PROLOGUE_NONE
    if prologue and not F.gemv_decode_fits(M, N, K, prologue):
        x2 = _rmsnorm_rows(x2, norm_w, eps)
        prologue, norm_w = F.PROLOGUE_NONE, None
    return F.gemv_decode(x2, packed, absmax, code, N, K, prologue=prologue, norm_w=norm_w, eps=eps, epilogue=epilogue,
                         residual=residual, pdl=pdl, next_weight=next_weight)


def _positions_impl(input_pos, B, T):
    """int32 positions for the kernels: one per sequence for a single-token step, one per token for a prompt."""
    p = input_pos.to(torch.int32)
    return p.expand(B).contiguous() if T == 1 else p.contiguous()


def _linear(x2, packed, absmax, code, N, K):
    return functional.linear_nf4(x2, packed, None, absmax, code, 64, (N, K))


_mask_rows: dict = {}


def _cache_mask(positions, S):
    """[T, S] boolean: cache row s is visible to the token at positions[t] (s <= position)."""
    key = (positions.device, S)
    rows = _mask_rows.get(key)
    if rows is None:
        if positions.is_cuda and torch.cuda.is_current_stream_capturing():
            rows = torch.arange(S, device=positions.device, dtype=torch.int32)
        else:
            rows = _mask_rows[key] = torch.arange(S, device=positions.device, dtype=torch.int32)
    return rows[None, :] <= positions[:, None]


def _attn_prefill(x, norm_w, eps, wq, aq, wk, ak, wv, av, wo, ao, code, k_cache, v_cache, positions, theta, Hq, Hkv):
    """The attention block over B x T rows: RMSNorm, one GEMM over the q|k|v rows, rotary embedding + cache write,
    torch's fused attention over the cache (grouped heads, visibility from the positions), output GEMM, residual."""
    F = functional
    B, T, D = x.shape
    n = F.rms_norm_rows(x.reshape(B * T, D), norm_w, eps)
    qkv = _linear(n, _span((wq, wk, wv), "q/k/v weight"), _span((aq, ak, av), "q/k/v absmax"), code, (Hq + 2 * Hkv) * HEAD_DIM, D)
    q4 = F.rope_prefill(qkv.view(B, T, -1), positions, k_cache, v_cache, Hq, Hkv, theta)
    att = torch.nn.functional.scaled_dot_product_attention(q4, k_cache, v_cache, attn_mask=_cache_mask(positions, k_cache.shape[2]),
                                                           enable_gqa=Hq != Hkv)
    y = _linear(att.transpose(1, 2).reshape(B * T, Hq * HEAD_DIM), wo, ao, code, D, Hq * HEAD_DIM)
    return y.view(x.shape).add_(x)


def _attn_block_impl(x, norm_w, eps, wq, aq, wk, ak, wv, av, wo, ao, code, k_cache, v_cache, positions, theta, Hq, Hkv,
                     nxt_w=None, nxt_a=None, nxt_N=0, nxt_K=0):
    # (nxt_*: the weight the launch after this block streams, hinted to this block's last GEMV)
    F = functional
    D = x.shape[-1]
    if x.dim() == 3 and x.shape[1] > 1:
        return _attn_prefill(x, norm_w, eps, wq, aq, wk, ak, wv, av, wo, ao, code, k_cache, v_cache, positions, theta, Hq, Hkv)
    B = x.numel() // D
    x2 = x.reshape(B, D)
    # (the weight the next GEMV streams is hinted to each GEMV: the attention launch in between reads no weights)
    qkv = _gemv(x2, _span((wq, wk, wv), "q/k/v weight"), _span((aq, ak, av), "q/k/v absmax"), code,
                (Hq + 2 * Hkv) * HEAD_DIM, D, norm_w=norm_w, eps=eps, next_weight=(wo, ao, D, Hq * HEAD_DIM))
    att = F.attn_decode_fused(qkv, positions, k_cache, v_cache, Hq, Hkv, theta, pdl=True)
    y = _gemv(att, wo, ao, code, D, Hq * HEAD_DIM, residual=x2, next_weight=(nxt_w, nxt_a, nxt_N, nxt_K) if nxt_w is not None else None)
    return y.view(x.shape)


def _mlp_block_impl(h, norm_w, eps, w1, a1, w3, a3, w2, a2, code, Fdim, nxt_w=None, nxt_a=None, nxt_N=0, nxt_K=0):
    F = functional
    D = h.shape[-1]
    B = h.numel() // D
    h2 = h.reshape(B, D)
    packed, absmax = _span((w1, w3), "gate/up weight"), _span((a1, a3), "gate/up absmax")
    if B > MAX_ROWS:
        # tensor-core regime: RMSNorm, one GEMM over the gate|up rows, SiLU * up, down GEMM, residual
        gu = _linear(F.rms_norm_rows(h2, norm_w, eps), packed, absmax, code, 2 * Fdim, D)
        y = _linear(F.silu_mul(gu, Fdim, interleaved=False), w2, a2, code, D, Fdim)
        return y.view(h.shape).add_(h)
    if F.gemv_decode_fits(B, 2 * Fdim, D, F.PROLOGUE_RMSNORM) and F.swiglu_halves_available():
        act = _gemv(h2, packed, absmax, code, 2 * Fdim, D, norm_w=norm_w, eps=eps, epilogue=F.EPILOGUE_SWIGLU_HALVES,
                    next_weight=(w2, a2, D, Fdim))
    else:
        gu = _gemv(h2, packed, absmax, code, 2 * Fdim, D, norm_w=norm_w, eps=eps)
        act = F.silu_mul(gu, Fdim, interleaved=False)
    y = _gemv(act, w2, a2, code, D, Fdim, residual=h2, next_weight=(nxt_w, nxt_a, nxt_N, nxt_K) if nxt_w is not None else None)
    return y.view(h.shape)


def _norm_linear_impl(x, norm_w, eps, w, a, code, N):
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if x2.shape[0] > MAX_ROWS:
        y = _linear(functional.rms_norm_rows(x2, norm_w, eps), w, a, code, N, K)
    else:
        y = _gemv(x2, w, a, code, N, K, norm_w=norm_w, eps=eps)
    return y.view(*x.shape[:-1], N)


def get_fusion_symbols():
    """Registers (once) the block symbols on the NF4 executor and returns them by name."""
    global _symbols
    if _symbols is not None:
        return _symbols
    ex = get_nf4_executor()

    def positions_meta(input_pos, B, T):
        return TensorProxy(like=input_pos, shape=(B,) if T == 1 else (T,), dtype=thunder.dtypes.int32)

    def attn_block_meta(x, norm_w, eps, wq, aq, wk, ak, wv, av, wo, ao, code, k_cache, v_cache, positions, theta, Hq, Hkv,
                        nxt_w=None, nxt_a=None, nxt_N=0, nxt_K=0):
        return TensorProxy(like=x)

    def mlp_block_meta(h, norm_w, eps, w1, a1, w3, a3, w2, a2, code, Fdim, nxt_w=None, nxt_a=None, nxt_N=0, nxt_K=0):
        return TensorProxy(like=h)

    def norm_linear_meta(x, norm_w, eps, w, a, code, N):
        return TensorProxy(like=x, shape=(*x.shape[:-1], N))

    # the implementations are looked up through the module at call time (tests substitute CPU checkers)
    _symbols = {
        "positions": ex.register_operator("nf4_b200_positions", meta=positions_meta,
                                          fn=lambda *a: _positions_impl(*a)),
        "attn_block": ex.register_operator("nf4_b200_attn_block", meta=attn_block_meta,
                                           fn=lambda *a: _attn_block_impl(*a)),
        "mlp_block": ex.register_operator("nf4_b200_mlp_block", meta=mlp_block_meta,
                                          fn=lambda *a: _mlp_block_impl(*a)),
        "norm_linear": ex.register_operator("nf4_b200_norm_linear", meta=norm_linear_meta,
                                            fn=lambda *a: _norm_linear_impl(*a)),
    }
    return _symbols


# ---------------------------------------------------------------------------------------------------
# trace side: dataflow matching
# ---------------------------------------------------------------------------------------------------

class _NoMatch(Exception):
    pass


def _need(cond, why="") -> None:
    if not cond:
        raise _NoMatch(why)


class _Graph:
    """Producer / consumer index over the top-level bound symbols of a trace."""

    def __init__(self, bsyms):
        self.bsyms = list(bsyms)
        self.prod: dict[str, int] = {}
        self.cons: dict[str, list[int]] = defaultdict(list)
        for i, b in enumerate(self.bsyms):
            if b.sym.name.startswith("unpack_"):       # the trace's arguments: inputs, not products
                continue
            for o in b.flat_proxy_outs:
                self.prod.setdefault(o.name, i)
            for a in b.flat_proxy_args:
                self.cons[a.name].append(i)

    def producer(self, proxy, name: str | None = None, used: list | None = None):
        """The bound symbol that produced `proxy` (must be called `name` when given); its index is
        appended to `used`.  `update_aliases` (the in-place bookkeeping prim) is looked through."""
        _need(isinstance(proxy, TensorProxy), "not a tensor proxy")
        i = self.prod.get(proxy.name)
        _need(i is not None, f"{proxy.name} is a trace input")
        b = self.bsyms[i]
        while b.sym.name == "update_aliases":
            outs, ins = b.flat_proxy_outs, b.flat_proxy_args
            j = [o.name for o in outs].index(proxy.name)
            if used is not None:
                used.append(i)
            proxy = ins[j]
            i = self.prod.get(proxy.name)
            _need(i is not None, f"{proxy.name} is a trace input")
            b = self.bsyms[i]
        _need(name is None or b.sym.name == name, f"{proxy.name}: produced by {b.sym.name}, wanted {name}")
        if used is not None:
            used.append(i)
        return b

    def through_aliases(self, proxy, used: list):
        """`proxy` with `update_aliases` hops removed (for proxies that may be trace inputs)."""
        while True:
            i = self.prod.get(proxy.name)
            if i is None or self.bsyms[i].sym.name != "update_aliases":
                return proxy
            b = self.bsyms[i]
            j = [o.name for o in b.flat_proxy_outs].index(proxy.name)
            used.append(i)
            proxy = b.flat_proxy_args[j]

    def is_input(self, proxy) -> bool:
        return proxy.name not in self.prod


def _is_nf4(b) -> bool:
    return b.sym.name == "nf4_b200_matmul"


def _nf4_parts(b):
    """(x, qweight, absmax, code, (N, K)) of an nf4_b200_matmul call this pass may fuse."""
    x, w, bias, absmax, code, blocksize, dtype, shape = b.args
    _need(bias is None and blocksize == 64 and dtype == torch.bfloat16, "biased / non-bf16 / other blocksize")
    return x, w, absmax, code, (int(shape[0]), int(shape[1]))


def _rows(proxy) -> int:
    return int(math.prod(proxy.shape[:-1]))


def _same(a, b) -> bool:
    return isinstance(a, TensorProxy) and isinstance(b, TensorProxy) and a.name == b.name


def _match_rms_norm(g: _Graph, proxy, used):
    b = g.producer(proxy, "rms_norm", used)
    args = list(b.args) + [None] * (4 - len(b.args))
    x, shape, w, eps = args[0], args[1], args[2], args[3]
    eps = b.kwargs.get("eps", eps)
    w = b.kwargs.get("weight", w)
    _need(isinstance(w, TensorProxy) and tuple(shape) == (x.shape[-1],) and eps is not None, "rms_norm form")
    _need(x.dtype == thunder.dtypes.bfloat16 and w.dtype == thunder.dtypes.bfloat16, "rms_norm dtype")
    return x, w, float(eps)


def _match_rope(g: _Graph, proxy, used, shared):
    """proxy = type_as(flatten(stack([xr*c - xi*s, xr*s + xi*c], -1), 3), src) over the (2i, 2i+1) pairs of
    src, with c / s = view(table[input_pos]).  Returns (src, cos_table, sin_table, input_pos).  Symbols that
    other layers use too (the table lookups) are recorded in `shared`, the rest in `used`."""
    ta = g.producer(proxy, "type_as", used)
    fl = g.producer(ta.args[0], "flatten", used)
    _need(tuple(fl.args[1:]) in ((3, -1), (3,), (3, 4)), "flatten dims")
    st = g.producer(fl.args[0], "stack", used)
    parts = st.args[0]
    _need(len(parts) == 2 and (st.args[1] if len(st.args) > 1 else st.kwargs.get("dim")) == -1, "stack form")
    sub = g.producer(parts[0], "sub", used)
    add = g.producer(parts[1], "add", used)
    m1, m2 = g.producer(sub.args[0], "mul", used), g.producer(sub.args[1], "mul", used)
    m3, m4 = g.producer(add.args[0], "mul", used), g.producer(add.args[1], "mul", used)
    xr, c = m1.args[0], m1.args[1]
    xi, s = m2.args[0], m2.args[1]
    _need(_same(m3.args[0], xr) and _same(m3.args[1], s) and _same(m4.args[0], xi) and _same(m4.args[1], c), "rotation form")
    gr, gi = g.producer(xr, "getitem", used), g.producer(xi, "getitem", used)
    _need(_same(gr.args[0], gi.args[0]) and tuple(gr.args[1]) == (Ellipsis, 0) and tuple(gi.args[1]) == (Ellipsis, 1), "pair split")
    rs = g.producer(gr.args[0], "reshape", used)
    cv = g.producer(rs.args[0], "convert_element_type", used)
    src = cv.args[0]
    _need(tuple(rs.args[1:]) == (*src.shape[:-1], src.shape[-1] // 2, 2), "pair reshape")
    _need(_same(ta.args[1], src), "type_as target")
    tables = []
    pos = None
    for t in (c, s):
        vw = g.producer(t, "view", used)
        gt = g.producer(vw.args[0], "getitem", shared)
        table, idx = gt.args
        _need(g.is_input(table) and isinstance(idx, TensorProxy), "table lookup")
        _need(pos is None or _same(pos, idx), "table index")
        pos = idx
        tables.append(table)
    return src, tables[0], tables[1], pos


def _match_cache_read(g: _Graph, proxy, used, n_rep: int):
    """proxy = the cache after index_copy_, optionally expanded over the query heads of a group.
    Returns (cache_input, index, source_of_new_rows)."""
    if n_rep > 1:
        rs = g.producer(proxy, "reshape", used)
        ex = g.producer(rs.args[0], "expand", used)
        gt = g.producer(ex.args[0], "getitem", used)
        key = tuple(gt.args[1])
        _need(len(key) == 5 and key[2] is None and all(k == slice(None) for i, k in enumerate(key) if i != 2), "group expand")
        proxy = gt.args[0]
    ic = g.producer(proxy, "index_copy_", used)
    cache, dim, idx, src = ic.args
    cache = g.through_aliases(cache, used)
    _need(dim == 2 and g.is_input(cache), "cache update form")
    return cache, idx, src


def _match_mask(g: _Graph, mask, pos, S: int, shared):
    le = g.producer(mask, "le", shared)
    a = g.producer(le.args[0], "getitem", shared)
    b = g.producer(le.args[1], "getitem", shared)
    _need(tuple(a.args[1]) == (None, slice(None)) and tuple(b.args[1]) == (slice(None), None), "mask broadcast")
    _need(_same(b.args[0], pos), "mask positions")
    ar = g.producer(a.args[0], "arange", shared)
    nums = [v for v in ar.args if isinstance(v, int)]
    _need(nums in ([S, 1], [0, S, 1], [S], [0, S]), "mask range")


def _single_use(g: _Graph, proxy, by: set[int]) -> None:
    _need(all(i in by for i in g.cons.get(proxy.name, ())), f"{proxy.name} is used outside of the pattern")


class _Found:
    def __init__(self, kind, anchor, region, out, args):
        self.kind, self.anchor, self.region, self.out, self.args = kind, anchor, region, out, args


def _find_mlp(g: _Graph, i: int):
    down = g.bsyms[i]
    used = [i]
    act, w2, a2, code, (D, Fdim) = _nf4_parts(down)
    mul = g.producer(act, "mul", used)
    for s_, u_ in ((mul.args[0], mul.args[1]), (mul.args[1], mul.args[0])):
        try:
            trial = list(used)
            silu = g.producer(s_, "silu", trial)
            gate, up = g.producer(silu.args[0], None, trial), g.producer(u_, None, trial)
            _need(_is_nf4(gate) and _is_nf4(up), "gate/up are not quantized linears")
            used = trial
            break
        except _NoMatch:
            continue
    else:
        raise _NoMatch("silu(gate) * up not found")
    n1, w1, a1, c1, (F1, D1) = _nf4_parts(gate)
    n3, w3, a3, c3, (F3, D3) = _nf4_parts(up)
    _need(_same(n1, n3) and (F1, D1) == (Fdim, D) and (F3, D3) == (Fdim, D), "gate/up shapes")
    h, nw, eps = _match_rms_norm(g, n1, used)
    _need(Fdim % 8 == 0, "hidden width")
    out_b = down
    res = [j for j in g.cons.get(down.output.name, ())]
    if len(res) == 1 and g.bsyms[res[0]].sym.name == "add":
        add = g.bsyms[res[0]]
        other = add.args[1] if _same(add.args[0], down.output) else add.args[0]
        _need(_same(other, h), "residual is not the block input")
        used.append(res[0])
        out_b = add
    else:
        raise _NoMatch("no residual add")
    region = set(used)
    for b in (gate, up, silu, mul, down):
        _single_use(g, b.output, region)
    _single_use(g, n1, region)
    return _Found("mlp", max(region), region, out_b.output, (h, nw, eps, w1, a1, w3, a3, w2, a2, code, Fdim))


def _find_attention(g: _Graph, i: int):
    sdpa = g.bsyms[i]
    used, shared = [i], []
    args = list(sdpa.args) + [None] * (6 - len(sdpa.args))
    q4, k4, v4, mask, dropout, causal = args[:6]
    _need(isinstance(mask, TensorProxy) and not causal and not dropout and sdpa.kwargs.get("scale") is None, "sdpa form")
    B, Hq, T, Dh = q4.shape
    _need(Dh == HEAD_DIM, "heads are not 128 wide")
    _need(T > 1 or B <= MAX_ROWS, "a single-token step of more than 16 sequences")
    S = k4.shape[2]
    # query side
    tq = g.producer(q4, "transpose", used)
    _need(tuple(tq.args[1:]) == (1, 2), "q transpose")
    qsrc, cos_t, sin_t, pos = _match_rope(g, tq.args[0], used, shared)
    vq = g.producer(qsrc, "view", used)
    lq = g.producer(vq.args[0], None, used)
    _need(_is_nf4(lq), "q is not a quantized linear")
    n, wq, aq, code, (Nq, D) = _nf4_parts(lq)
    _need(Nq == Hq * Dh, "q width")
    # key side
    Hkv = None
    for n_rep in (1, 2, 4, 8, 16, 32):
        if Hq % n_rep == 0:
            try:
                trial = list(used)
                k_cache, k_idx, k_new = _match_cache_read(g, k4, trial, n_rep)
                Hkv = Hq // n_rep
                _need(tuple(k_cache.shape[1:]) == (Hkv, S, Dh), "cache shape")
                used = trial
                break
            except _NoMatch:
                Hkv = None
    _need(Hkv is not None, "key cache read not recognised")
    n_rep = Hq // Hkv
    v_cache, v_idx, v_new = _match_cache_read(g, v4, used, n_rep)
    _need(tuple(v_cache.shape) == tuple(k_cache.shape) and _same(k_idx, pos) and _same(v_idx, pos), "cache index")
    tk = g.producer(k_new, "transpose", used)
    ksrc, cos_k, sin_k, pos_k = _match_rope(g, tk.args[0], used, shared)
    _need(_same(cos_k, cos_t) and _same(sin_k, sin_t) and _same(pos_k, pos), "k rotation differs from q's")
    vk = g.producer(ksrc, "view", used)
    lk = g.producer(vk.args[0], None, used)
    tv = g.producer(v_new, "transpose", used)
    vv = g.producer(tv.args[0], "view", used)
    lv = g.producer(vv.args[0], None, used)
    _need(_is_nf4(lk) and _is_nf4(lv), "k/v are not quantized linears")
    nk, wk, ak, _, (Nk, Dk) = _nf4_parts(lk)
    nv, wv, av, _, (Nv, Dv) = _nf4_parts(lv)
    _need(_same(nk, n) and _same(nv, n) and Nk == Nv == Hkv * Dh and Dk == Dv == D, "k/v shapes")
    _match_mask(g, mask, pos, S, shared)
    x, nw, eps = _match_rms_norm(g, n, used)
    # output side
    cons = g.cons.get(sdpa.output.name, [])
    _need(len(cons) == 1 and g.bsyms[cons[0]].sym.name == "transpose", "attention output transpose")
    t_o = g.bsyms[cons[0]]
    cons = g.cons.get(t_o.output.name, [])
    _need(len(cons) == 1 and g.bsyms[cons[0]].sym.name in ("reshape", "view"), "attention output reshape")
    r_o = g.bsyms[cons[0]]
    cons = g.cons.get(r_o.output.name, [])
    _need(len(cons) == 1 and _is_nf4(g.bsyms[cons[0]]), "output projection")
    lo = g.bsyms[cons[0]]
    _, wo, ao, _, (Do, Ko) = _nf4_parts(lo)
    _need(Do == D and Ko == Hq * Dh, "output projection shape")
    cons = g.cons.get(lo.output.name, [])
    _need(len(cons) == 1 and g.bsyms[cons[0]].sym.name == "add", "no residual add")
    add = g.bsyms[cons[0]]
    other = add.args[1] if _same(add.args[0], lo.output) else add.args[0]
    _need(_same(other, x), "residual is not the block input")
    tail = [g.prod[b.output.name] for b in (t_o, r_o, lo, add)]
    used += tail
    # the table lookups and the mask (`shared`) serve every layer: they stay, and dead-code elimination
    # removes them once no layer uses them; everything else must be private to this block
    region = set(used)
    for j in region:
        if g.bsyms[j] is not add:
            for o in g.bsyms[j].flat_proxy_outs:
                _single_use(g, o, region)
    return _Found("attn", max(region), region, add.output,
                  dict(x=x, nw=nw, eps=eps, wq=wq, aq=aq, wk=wk, ak=ak, wv=wv, av=av, wo=wo, ao=ao, code=code,
                       k_cache=k_cache, v_cache=v_cache, pos=pos, cos=cos_t, sin=sin_t, Hq=Hq, Hkv=Hkv, B=B, T=T, S=S))


def _find_norm_linear(g: _Graph, i: int, taken: set[int]):
    lin = g.bsyms[i]
    used = [i]
    n, w, a, code, (N, K) = _nf4_parts(lin)
    x, nw, eps = _match_rms_norm(g, n, used)
    region = set(used)
    _need(not (region & taken), "already fused")
    _single_use(g, n, region)
    return _Found("norm_linear", i, region, lin.output, (x, nw, eps, w, a, code, N))


# ---------------------------------------------------------------------------------------------------
# the transform
# ---------------------------------------------------------------------------------------------------

class NF4DecodeFusion(Transform):
    """Second pass after `NF4LinearQuant4bit` (see the module docstring); it rewrites single-token traces and
    prompt (prefill) traces alike.  `rope_theta` is the base of
    the rotary embedding the model's cos/sin tables were built with; when omitted it is read from
    `model.args.rope_theta`.  The tables found in the trace are checked against it before an attention
    block is rewritten (the fused kernel computes the angles itself)."""

    def __init__(self, rope_theta: float | None = None):
        self.rope_theta = rope_theta
        self.thunder_module = None
        self.fused = {"attn": 0, "mlp": 0, "norm_linear": 0}
        self.declined: list[str] = []
        get_fusion_symbols()

    def transform_module(self, model) -> None:
        self.thunder_module = model

    # ---- weights ------------------------------------------------------------------------------
    def _param_name(self, proxy, names_of_args) -> str | None:
        return names_of_args.get(proxy.name)

    def _rehome(self, names: list[str]) -> None:
        """Places the tensors `names` (module parameter names) back to back in one allocation and
        re-binds every alias of each name to its view.  Values, shapes and dtypes are unchanged."""
        tm = self.thunder_module
        ts = [tm.get_parameter(n) for n in names]
        if any(t.device.type == "meta" for t in ts):
            return
        end = ts[0].data_ptr()
        ok = True
        for t in ts:
            ok = ok and t.data_ptr() == end and t.is_contiguous()
            end += t.numel() * t.element_size()
        if ok and ts[0].untyped_storage().nbytes() - ts[0].storage_offset() * ts[0].element_size() >= sum(
                t.numel() for t in ts) * ts[0].element_size():
            return
        with torch.no_grad():
            flat = torch.cat([t.detach().reshape(-1) for t in ts])
        shared = tm._get_shared_names()
        off = 0
        for n, t in zip(names, ts):
            view = flat[off:off + t.numel()].view(t.shape)
            off += t.numel()
            for alias in shared.get(n, {n}):
                if alias in tm._overrides_parameters:
                    tm._overrides_parameters[alias] = view

    def _theta_ok(self, cos_name: str | None, sin_name: str | None, theta: float) -> bool:
        tm = self.thunder_module
        if cos_name is None or sin_name is None:
            return False
        try:
            cos, sin = tm.get_buffer(cos_name), tm.get_buffer(sin_name)
        except Exception:
            return False
        if cos.device.type == "meta" or cos.dim() != 2 or cos.shape[1] != HEAD_DIM // 2:
            return False
        n = min(cos.shape[0], 64)
        freqs = 1.0 / (theta ** (torch.arange(0, HEAD_DIM, 2).float() / HEAD_DIM))
        ang = torch.outer(torch.arange(n).float(), freqs)
        tol = 1e-2 if cos.dtype != torch.float32 else 1e-4
        return bool(torch.allclose(cos[:n].float().cpu(), torch.cos(ang), atol=tol) and
                    torch.allclose(sin[:n].float().cpu(), torch.sin(ang), atol=tol))

    # ---- traces -------------------------------------------------------------------------------
    def transform_traces_pre_prologue(self, prologue_trace, computation_trace, epilogue_trace, **kwargs):
        from thunder.transforms.utils import get_checks

        sym = get_fusion_symbols()
        tm = self.thunder_module
        theta = self.rope_theta
        if theta is None and tm is not None:
            theta = getattr(getattr(tm._model, "args", None), "rope_theta", None)

        # computation-trace argument -> module parameter / buffer name (through the prologue's unpacks)
        name_of: dict[str, str] = {}
        ret = prologue_trace.bound_symbols[-1].args[0][0]
        unpack_name = {}
        for b in prologue_trace.bound_symbols:
            if b.sym.name in ("unpack_parameter", "unpack_buffer"):
                unpack_name[b.output.name] = b.args[1]
        for p, c in zip(ret, computation_trace.args):
            if getattr(p, "name", None) in unpack_name:
                name_of[c.name] = unpack_name[p.name]

        g = _Graph(computation_trace.bound_symbols)
        found: list[_Found] = []
        taken: set[int] = set()
        for i, b in enumerate(g.bsyms):
            try:
                if b.sym.name == "scaled_dot_product_attention":
                    f = _find_attention(g, i)
                    a = f.args
                    _need(theta is not None, "rope_theta unknown")
                    _need(self._theta_ok(name_of.get(a["cos"].name), name_of.get(a["sin"].name), float(theta)),
                          "the rope tables are not cos/sin(position * theta^(-2i/128))")
                elif _is_nf4(b):
                    f = _find_mlp(g, i)
                else:
                    continue
            except _NoMatch as e:
                if b.sym.name == "scaled_dot_product_attention":
                    self.declined.append(f"attention at {b.output.name}: {e}")
                continue
            if f.region & taken:
                continue
            taken |= f.region
            found.append(f)
        for i, b in enumerate(g.bsyms):
            if _is_nf4(b) and i not in taken:
                try:
                    f = _find_norm_linear(g, i, taken)
                except _NoMatch:
                    continue
                taken |= f.region
                found.append(f)
        if not found:
            return prologue_trace, computation_trace, epilogue_trace

        # weights that stream as one matrix must be adjacent in memory
        if tm is not None:
            for f in found:
                if f.kind == "attn":
                    a = f.args
                    groups = [[a["wq"], a["wk"], a["wv"]], [a["aq"], a["ak"], a["av"]]]
                elif f.kind == "mlp":
                    groups = [[f.args[3], f.args[5]], [f.args[4], f.args[6]]]
                else:
                    continue
                for grp in groups:
                    names = [name_of.get(p.name) for p in grp]
                    if all(n is not None for n in names) and len(set(names)) == len(names):
                        self._rehome(names)

        # the weight each block's last GEMV should hint: the first one the next block (in trace order) streams
        # (only the first tensor of a q|k|v or gate|up group, with its own row count: the hint makes the kernel touch
        # that memory, and whether the group is still adjacent in memory is only known at call time)
        def first_weight(f):
            if f.kind == "attn":
                a = f.args
                return a["wq"], a["aq"], a["Hq"] * HEAD_DIM, int(a["x"].shape[-1])
            if f.kind == "mlp":
                return f.args[3], f.args[4], f.args[10], int(f.args[0].shape[-1])
            return f.args[3], f.args[4], f.args[6], int(f.args[0].shape[-1])

        ordered = sorted(found, key=lambda f: f.anchor)
        hint = {}
        for cur, nxt in zip(ordered, ordered[1:]):
            hint[cur.anchor] = first_weight(nxt)
        by_anchor = {f.anchor: f for f in found}
        new_trace = from_trace(computation_trace)
        new_bsyms = []
        pos32: dict[tuple[str, int], TensorProxy] = {}
        with tracectx(new_trace):
            for i, b in enumerate(g.bsyms):
                f = by_anchor.get(i)
                if f is None:
                    if i not in taken:
                        new_bsyms.append(b)
                    continue
                if f.kind == "attn":
                    a = f.args
                    key = (a["pos"].name, a["B"], a["T"])
                    p32 = pos32.get(key)
                    if p32 is None:
                        p32 = TensorProxy(like=a["pos"], shape=(a["B"],) if a["T"] == 1 else (a["T"],), dtype=thunder.dtypes.int32)
                        new_bsyms.append(sym["positions"].bind(a["pos"], a["B"], a["T"], output=p32))
                        pos32[key] = p32
                    new_bsyms.append(sym["attn_block"].bind(
                        a["x"], a["nw"], a["eps"], a["wq"], a["aq"], a["wk"], a["ak"], a["wv"], a["av"], a["wo"], a["ao"],
                        a["code"], a["k_cache"], a["v_cache"], p32, float(theta), a["Hq"], a["Hkv"],
                        *hint.get(f.anchor, (None, None, 0, 0)), output=f.out))
                elif f.kind == "mlp":
                    new_bsyms.append(sym["mlp_block"].bind(*f.args, *hint.get(f.anchor, (None, None, 0, 0)), output=f.out))
                else:
                    new_bsyms.append(sym["norm_linear"].bind(*f.args, output=f.out))
                self.fused[f.kind] += 1
        new_trace.bound_symbols = new_bsyms
        new_trace = dce(new_trace)
        new_trace.set_provenance(TraceProvenance("NF4 decode fusion"))
        return prologue_trace, new_trace, epilogue_trace
