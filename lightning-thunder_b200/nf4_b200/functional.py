"""Host-side mirror of the three bitsandbytes entry points the reference's NF4 path calls
(thunder/transforms/quantization.py:35-39, 63), backed by the sm_100a kernels:

    quantize_4bit(w, quant_type="nf4")            -> (packed uint8 [ceil(numel/2), 1], QuantState)
    QuantState(absmax, shape=, blocksize=, code=, quant_type="nf4", dtype=)
    matmul_4bit(x, qweight.t(), bias=, quant_state=)   -> x @ dequant(W).T + bias
    dequantize_4bit(packed, quant_state)          -> W in quant_state.dtype

Names, argument meaning and error behaviour follow those calls so that the reference's
transform can drive these functions unchanged.  Tensors must live on a CUDA device; there is
no CPU path.
"""

from __future__ import annotations

import ctypes
from collections.abc import Sequence

import torch

from . import _lib
from .codebook import NF4_LEVELS

_DTYPE_CODE = {torch.float32: _lib.NF4_F32, torch.float16: _lib.NF4_F16, torch.bfloat16: _lib.NF4_BF16}

_code_cache: dict = {}


def nf4_code(device) -> torch.Tensor:
    """The 16 NF4 levels as an fp32 tensor on `device` (one cached copy per device)."""
    device = torch.device(device)
    key = (device.type, device.index)
    t = _code_cache.get(key)
    if t is None:
        t = torch.tensor(NF4_LEVELS, dtype=torch.float32, device=device)
        _code_cache[key] = t
    return t


class QuantState:
    """Metadata of one NF4-quantized tensor; same fields the reference reads
    (thunder/transforms/quantization.py:90-101): absmax, shape, blocksize, code, dtype."""

    def __init__(self, absmax, shape=None, code=None, blocksize=64, quant_type="nf4", dtype=None):
        if quant_type != "nf4":
            raise NotImplementedError(f"quant_type {quant_type!r}: only 'nf4' is implemented")
        self.absmax = absmax
        self.shape = torch.Size(shape) if shape is not None else None
        self.code = code
        self.blocksize = blocksize
        self.quant_type = quant_type
        self.dtype = dtype
        self.nested = False     # True after compress_absmax: absmax is uint8, see offset / state2
        self.offset = None
        self.state2 = None

    def to(self, device):
        self.absmax = self.absmax.to(device)
        self.code = self.code.to(device)
        return self


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor (got device {t.device}); the NF4 kernels have no CPU path")


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def quantize_4bit(A: torch.Tensor, absmax=None, out=None, blocksize: int = 64, compress_statistics: bool = False,
                  quant_type: str = "nf4", quant_storage=torch.uint8):
    """Blockwise NF4 quantization of `A` (fp32/fp16/bf16, any shape).  Returns (packed, QuantState)."""
    if quant_type != "nf4":
        raise NotImplementedError(f"quant_type {quant_type!r}: only 'nf4' is implemented")
    if quant_storage != torch.uint8:
        raise NotImplementedError("quant_storage: only torch.uint8")
    if A.dtype not in _DTYPE_CODE:
        raise ValueError(f"quantize_4bit: unsupported dtype {A.dtype}")
    _require_cuda(A, "quantize_4bit input")
    A = A.contiguous()
    n = A.numel()
    with torch.cuda.device(A.device):
        if out is None:
            out = torch.empty(((n + 1) // 2, 1), dtype=torch.uint8, device=A.device)
        if absmax is None:
            absmax = torch.empty(((n + blocksize - 1) // blocksize,), dtype=torch.float32, device=A.device)
        code = nf4_code(A.device)
        lib = _lib.load()
        _lib.check(
            lib.nf4_b200_quantize(A.data_ptr(), n, _DTYPE_CODE[A.dtype], blocksize, code.data_ptr(), out.data_ptr(),
                                  absmax.data_ptr(), _stream_ptr(A.device)),
            "nf4_b200_quantize",
        )
    state = QuantState(absmax=absmax, shape=A.shape, dtype=A.dtype, blocksize=blocksize, code=code.clone(),
                       quant_type=quant_type)
    if compress_statistics:
        compress_absmax(state)
    return out, state


_code256_cache: dict = {}


def dq_code(device) -> torch.Tensor:
    """The 256-entry table of the double quantization as an fp32 tensor on `device`."""
    from .codebook import dq_code256

    device = torch.device(device)
    key = (device.type, device.index)
    t = _code256_cache.get(key)
    if t is None:
        t = torch.tensor(dq_code256(), dtype=torch.float32, device=device)
        _code256_cache[key] = t
    return t


def compress_absmax(state: QuantState) -> QuantState:
    """Double quantization in place: state.absmax becomes uint8 indices, state.state2 holds the
    per-256 fp32 scales and the table, state.offset the mean that was subtracted (a 1-element
    tensor on the device)."""
    am = state.absmax
    _require_cuda(am, "compress_absmax input")
    n = am.numel()
    with torch.cuda.device(am.device):
        u8 = torch.empty((n,), dtype=torch.uint8, device=am.device)
        scale2 = torch.empty(((n + 255) // 256,), dtype=torch.float32, device=am.device)
        offset = torch.empty((1,), dtype=torch.float32, device=am.device)
        code256 = dq_code(am.device)
        _lib.check(_lib.load().nf4_b200_dq_quantize(am.data_ptr(), n, code256.data_ptr(), u8.data_ptr(), scale2.data_ptr(),
                                                    offset.data_ptr(), _stream_ptr(am.device)), "nf4_b200_dq_quantize")
    state.absmax = u8
    state.offset = offset
    state.state2 = QuantState(absmax=scale2, shape=(n,), code=code256, blocksize=256, dtype=torch.float32)
    state.nested = True
    return state


def expand_absmax(state: QuantState, out=None) -> torch.Tensor:
    """fp32 absmax of a (possibly double-quantized) state."""
    if not state.nested:
        return state.absmax
    u8 = state.absmax
    n = u8.numel()
    with torch.cuda.device(u8.device):
        if out is None:
            out = torch.empty((n,), dtype=torch.float32, device=u8.device)
        _lib.check(_lib.load().nf4_b200_dq_dequantize(u8.data_ptr(), state.state2.absmax.data_ptr(), state.offset.data_ptr(),
                                                      state.state2.code.data_ptr(), n, out.data_ptr(),
                                                      _stream_ptr(u8.device)), "nf4_b200_dq_dequantize")
    return out


def dequantize_4bit(A: torch.Tensor, quant_state: QuantState = None, absmax=None, out=None, blocksize: int = 64,
                    quant_type: str = "nf4"):
    """Inverse of quantize_4bit: returns a tensor of quant_state.shape / quant_state.dtype."""
    if quant_state is None:
        raise ValueError("dequantize_4bit needs a quant_state")
    _require_cuda(A, "dequantize_4bit input")
    shape = quant_state.shape
    n = 1
    for s in shape:
        n *= int(s)
    dtype = quant_state.dtype
    absmax_f32 = expand_absmax(quant_state)
    with torch.cuda.device(A.device):
        if out is None:
            out = torch.empty(tuple(shape), dtype=dtype, device=A.device)
        lib = _lib.load()
        _lib.check(
            lib.nf4_b200_dequantize(A.data_ptr(), absmax_f32.data_ptr(), quant_state.code.data_ptr(), n,
                                    quant_state.blocksize, out.data_ptr(), _DTYPE_CODE[dtype], _stream_ptr(A.device)),
            "nf4_b200_dequantize",
        )
    return out


_WORKSPACES: dict = {}


def _linear_workspace(lib, M: int, N: int, K: int, dtype_code: int, device, stream_ptr):
    """Zero-initialised split-K scratch for (device, stream), grown on demand (earlier buffers are kept, never
    freed).  The kernels return it to its initial state, so one buffer serves every call on that stream.  While a CUDA graph is being
    captured no new buffer is created (it would belong to the graph's pool): the call then runs without
    a K split unless a large enough buffer already exists."""
    need = int(lib.nf4_b200_linear_workspace_bytes(M, N, K, dtype_code))
    if need == 0:
        return None, 0
    key = (torch.device(device).index, stream_ptr.value if hasattr(stream_ptr, "value") else int(stream_ptr or 0))
    held = _WORKSPACES.setdefault(key, [])
    if not held or held[-1].numel() < need:
        if torch.cuda.is_current_stream_capturing():
            return None, 0
        # superseded buffers stay alive: a CUDA graph captured earlier has their address baked in
        held.append(torch.zeros((max(need, 1 << 22),), dtype=torch.uint8, device=device))
    ws = held[-1]
    return ws, ws.numel()


def linear_nf4(x: torch.Tensor, packed: torch.Tensor, bias, absmax: torch.Tensor, code: torch.Tensor, blocksize: int,
               shape: Sequence[int], out=None) -> torch.Tensor:
    """y = x @ dequant(W).T + bias for W of logical `shape` = (N, K) stored as packed/absmax/code."""
    N, K = int(shape[0]), int(shape[1])
    if x.shape[-1] != K:
        raise RuntimeError(f"linear_nf4: x.shape={tuple(x.shape)} does not match weight shape {(N, K)}")
    if x.dtype not in _DTYPE_CODE:
        raise ValueError(f"linear_nf4: unsupported dtype {x.dtype}")
    _require_cuda(x, "linear_nf4 input")
    _require_cuda(packed, "linear_nf4 weight")
    for name, t in (("weight", packed), ("absmax", absmax), ("code", code)):
        if not t.is_cuda or t.device != x.device:
            raise RuntimeError(f"linear_nf4: {name} is on {t.device}, the activations on {x.device}")
    if absmax.dtype != torch.float32 or code.dtype != torch.float32:
        raise RuntimeError(f"linear_nf4: absmax and code must be fp32 (got {absmax.dtype}, {code.dtype})")
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty((*x.shape[:-1], N), dtype=x.dtype, device=x.device)
        lib = _lib.load()
        stream = _stream_ptr(x.device)
        ws, ws_bytes = _linear_workspace(lib, M, N, K, _DTYPE_CODE[x.dtype], x.device, stream) if int(blocksize) == 64 else (None, 0)
        _lib.check(
            lib.nf4_b200_linear(x2.data_ptr(), M, K, packed.data_ptr(), absmax.data_ptr(), code.data_ptr(), N,
                                int(blocksize), bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                _DTYPE_CODE[x.dtype], ws.data_ptr() if ws is not None else None, ws_bytes, stream),
            "nf4_b200_linear",
        )
    return out


def linear_nf4_input_grad(g: torch.Tensor, packed: torch.Tensor, absmax: torch.Tensor, code: torch.Tensor, blocksize: int,
                          shape: Sequence[int]) -> torch.Tensor:
    """dX = g @ dequant(W) for y = x @ dequant(W).T with W of logical `shape` = (N, K): the weight is
    dequantized to g's dtype by this library's kernel and multiplied by the vendor GEMM (the contraction
    runs over N, the dimension the packed layout strides over; this is also how the reference's library
    computes the gradient of a 4-bit linear).  The quantized weight gets no gradient."""
    N, K = int(shape[0]), int(shape[1])
    if g.shape[-1] != N:
        raise RuntimeError(f"linear_nf4_input_grad: g.shape={tuple(g.shape)} does not match weight shape {(N, K)}")
    _require_cuda(g, "linear_nf4_input_grad input")
    state = QuantState(absmax=absmax, shape=(N, K), code=code, blocksize=int(blocksize), dtype=g.dtype)
    w = dequantize_4bit(packed, state)
    return torch.matmul(g, w)


def matmul_4bit(A: torch.Tensor, B: torch.Tensor, quant_state: QuantState, out=None, bias=None) -> torch.Tensor:
    """A @ dequant(B) + bias with B = packed.t() (shape [1, N*K/2]) as the reference passes it
    (thunder/transforms/quantization.py:39); quant_state.shape = (N, K)."""
    if quant_state is None:
        raise ValueError("matmul_4bit needs a quant_state")
    if quant_state.nested:
        return linear_nf4_dq(A, B, bias, quant_state, out=out)
    return linear_nf4(A, B, bias, quant_state.absmax, quant_state.code, quant_state.blocksize, quant_state.shape, out=out)


_DQ_WORKSPACES: dict = {}


def _dq_workspace(device, need: int) -> torch.Tensor:
    """Scratch for the expanded absmax of the tensor-core path, one buffer per device, grown on demand and
    never freed (a captured CUDA graph may hold the address of an earlier, smaller one)."""
    key = torch.device(device).index
    held = _DQ_WORKSPACES.setdefault(key, [])
    if not held or held[-1].numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("linear_nf4_dq: the absmax workspace would have to grow during CUDA graph capture; "
                               "run the call once outside of the capture first")
        held.append(torch.empty((max(need, 1 << 22),), dtype=torch.uint8, device=device))
    return held[-1]


def linear_nf4_dq(x: torch.Tensor, packed: torch.Tensor, bias, state: QuantState, out=None, workspace=None) -> torch.Tensor:
    """linear_nf4 for a double-quantized state (C entry point nf4_b200_linear_dq).  Up to 16 activation rows
    (bf16, K a multiple of 1024) the fused GEMV expands the 8-bit absmax inside its stages; otherwise absmax
    is expanded into `workspace` (fp32, one value per 64 weights) and the regular kernels run on it."""
    N, K = int(state.shape[0]), int(state.shape[1])
    if x.shape[-1] != K:
        raise RuntimeError(f"linear_nf4_dq: x.shape={tuple(x.shape)} does not match weight shape {(N, K)}")
    if state.blocksize != 64:
        raise NotImplementedError("linear_nf4_dq: blocksize 64 only")
    _require_cuda(x, "linear_nf4_dq input")
    for name, t, dt in (("weight", packed, torch.uint8), ("absmax", state.absmax, torch.uint8),
                        ("scale", state.state2.absmax, torch.float32), ("offset", state.offset, torch.float32),
                        ("code256", state.state2.code, torch.float32), ("code", state.code, torch.float32)):
        if not t.is_cuda or t.device != x.device or t.dtype != dt:
            raise RuntimeError(f"linear_nf4_dq: {name} must be a {dt} tensor on {x.device} (got {t.dtype} on {t.device})")
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        fused = M <= 16 and x.dtype == torch.bfloat16 and K % 1024 == 0
        if workspace is None and not fused:
            workspace = _dq_workspace(x.device, int(lib.nf4_b200_linear_dq_workspace_bytes(N, K)))
        if out is None:
            out = torch.empty((*x.shape[:-1], N), dtype=x.dtype, device=x.device)
        if not fused and M > 16 and x.dtype == torch.bfloat16 and workspace.numel() >= 4 * (N * K // 64) and workspace.data_ptr() % 16 == 0:
            # tensor-core regime: expand once (this library's kernel), then the regular linear, which also plans
            # the split-K workspace the C entry point has no argument for
            absmax = expand_absmax(state, out=workspace[: 4 * (N * K // 64)].view(torch.float32))
            return linear_nf4(x, packed, bias, absmax, state.code, 64, (N, K), out=out)
        _lib.check(
            lib.nf4_b200_linear_dq(x2.data_ptr(), M, K, packed.data_ptr(), state.absmax.data_ptr(),
                                   state.state2.absmax.data_ptr(), state.offset.data_ptr(), state.state2.code.data_ptr(),
                                   state.code.data_ptr(), N, bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                   _DTYPE_CODE[x.dtype], workspace.data_ptr() if workspace is not None else None,
                                   workspace.numel() if workspace is not None else 0, _stream_ptr(x.device)),
            "nf4_b200_linear_dq",
        )
    return out


# ---------------------------------------------------------------------------------------------------
# Decode-step forms (one launch each).  The reference has no fused form of these: they fold the ops
# between two quantized linears of a Llama-shaped block (thunder/tests/llama2_model.py:142-190) into
# the linear.  The Thunder executor's block symbols (nf4_b200.fusion) are written in terms of these
# three functions and look them up at call time, so CPU tests can substitute checkers for them.
# ---------------------------------------------------------------------------------------------------

PROLOGUE_NONE, PROLOGUE_RMSNORM, PROLOGUE_SWIGLU = 0, 1, 2
EPILOGUE_NONE, EPILOGUE_SWIGLU_INTERLEAVED, EPILOGUE_SWIGLU_HALVES = 0, 1, 2


def gemv_decode_fits(M: int, N: int, K: int, prologue: int) -> bool:
    return bool(_lib.load().nf4_b200_gemv_decode_fits(int(M), int(N), int(K), int(prologue)))


def gemv_decode(x: torch.Tensor, packed: torch.Tensor, absmax: torch.Tensor, code: torch.Tensor, N: int, K: int, *,
                prologue: int = 0, norm_w=None, eps: float = 0.0, epilogue: int = 0, residual=None, out=None,
                pdl: bool = False, next_weight=None) -> torch.Tensor:
    """y = prologue(x) @ dequant(W[N, K]).T (+ residual), bf16, at most 16 activation rows.
    prologue 1: RMSNorm of x with weight norm_w; 2: x is [M, 2K] = [gate | up] and becomes silu(gate) * up.
    epilogue 1 / 2: W's rows are (gate_i, up_i) pairs / W is [gate rows; up rows], and y [M, N/2] =
    silu(x.gate_i) * (x.up_i).  next_weight = (packed, absmax, N, K) of the weight the NEXT launch on this stream
    streams: its head is pulled into L2 while this launch drains (a pure prefetch)."""
    _require_cuda(x, "gemv_decode input")
    if x.dtype != torch.bfloat16:
        raise ValueError("gemv_decode: bf16 activations only")
    in_cols = 2 * K if prologue == PROLOGUE_SWIGLU else K
    if x.shape[-1] != in_cols:
        raise RuntimeError(f"gemv_decode: x.shape={tuple(x.shape)} does not match K={K} (prologue {prologue})")
    x2 = x.reshape(-1, in_cols)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    n_out = N // 2 if epilogue else N
    with torch.cuda.device(x.device):
        if out is None:
            out = torch.empty((*x.shape[:-1], n_out), dtype=x.dtype, device=x.device)
        if next_weight is not None:
            nw_p, nw_a, nw_n, nw_k = next_weight
            _lib.check(_lib.load().nf4_b200_gemv_decode_next_weight(nw_p.data_ptr(), nw_a.data_ptr(), int(nw_n), int(nw_k)),
                       "nf4_b200_gemv_decode_next_weight")
        _lib.check(
            _lib.load().nf4_b200_gemv_decode(x2.data_ptr(), M, K, packed.data_ptr(), absmax.data_ptr(), code.data_ptr(), N,
                                             residual.data_ptr() if residual is not None else None, out.data_ptr(),
                                             int(prologue), norm_w.data_ptr() if norm_w is not None else None, float(eps),
                                             int(epilogue), 1 if pdl else 0, _stream_ptr(x.device)),
            "nf4_b200_gemv_decode",
        )
    return out


_ATTN_SCRATCH: dict = {}


def attn_splits(B: int, Hkv: int, S_max: int) -> int:
    """Splits along the cached sequence: enough thread blocks (kv heads x sequences x splits) to cover
    the SMs about twice, but at least ~96 cached positions per block (measured inside the 8B decode step at 512
    cached positions: 5 to 8 splits are equally fast, 4 cost 0.8 % of the step, 2 cost 4.6 %, 16 cost 0.6 %)."""
    return max(1, min(16, 296 // max(1, Hkv * B), S_max // 96))


def attn_decode_fused(qkv: torch.Tensor, positions: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      Hq: int, Hkv: int, theta: float, *, pdl: bool = False, out=None) -> torch.Tensor:
    """Single-query attention of a decode step in one launch: rotates q and the new k (interleaved
    pairs, base theta) at positions[b], writes k and v into the caches [B, Hkv, S_max, 128] at that
    row and attends over rows 0..positions[b].  qkv [B, (Hq + 2 Hkv) * 128] bf16, positions int32 [B].
    Returns [B, Hq * 128].  The caches are updated in place."""
    _require_cuda(qkv, "attn_decode_fused input")
    B = qkv.shape[0]
    Dh = 128
    S_max = k_cache.shape[2]
    if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise ValueError("attn_decode_fused: bf16 tensors only")
    if positions.dtype != torch.int32 or positions.numel() != B:
        raise ValueError("attn_decode_fused: positions must be int32 [B]")
    if tuple(k_cache.shape[1:]) != (Hkv, S_max, Dh) or k_cache.shape != v_cache.shape or k_cache.shape[0] < B:
        raise RuntimeError(f"attn_decode_fused: cache shape {tuple(k_cache.shape)} does not fit B={B}, Hkv={Hkv}")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous() and qkv.is_contiguous()):
        raise RuntimeError("attn_decode_fused: qkv and the caches must be contiguous")
    lib = _lib.load()
    ns = attn_splits(B, Hkv, S_max)
    key = (qkv.device.index, B, Hq, Hkv, ns)
    scratch = _ATTN_SCRATCH.get(key)
    with torch.cuda.device(qkv.device):
        if scratch is None:
            # kept for the life of the process (a captured CUDA graph holds these addresses)
            ws = torch.empty((lib.nf4_b200_attn_decode_workspace_bytes(B, Hq, ns),), dtype=torch.uint8, device=qkv.device)
            counters = torch.zeros((B * Hkv,), dtype=torch.int32, device=qkv.device)
            scratch = _ATTN_SCRATCH[key] = (ws, counters)
        ws, counters = scratch
        if out is None:
            out = torch.empty((B, Hq * Dh), dtype=qkv.dtype, device=qkv.device)
        _lib.check(
            lib.nf4_b200_attn_decode_fused(qkv.data_ptr(), positions.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                           out.data_ptr(), ws.data_ptr(), counters.data_ptr(), B, Hq, Hkv, Dh, S_max, ns,
                                           float(theta), 1 if pdl else 0, _stream_ptr(qkv.device)),
            "nf4_b200_attn_decode_fused",
        )
    return out


def rms_norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2, -1) + eps) * weight over the last dimension of a contiguous bf16 tensor (one launch)."""
    _require_cuda(x, "rms_norm_rows input")
    D = x.shape[-1]
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.numel() != D or D % 2:
        raise ValueError("rms_norm_rows: bf16 input and weight, an even last dimension")
    x2 = x.reshape(-1, D)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    with torch.cuda.device(x.device):
        out = torch.empty_like(x2)
        _lib.check(_lib.load().nf4_b200_rmsnorm(x2.data_ptr(), weight.data_ptr(), out.data_ptr(), x2.shape[0], D, float(eps),
                                                _stream_ptr(x.device)), "nf4_b200_rmsnorm")
    return out.view(x.shape)


def rope_prefill(qkv: torch.Tensor, positions: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, Hq: int, Hkv: int,
                 theta: float) -> torch.Tensor:
    """Rotary embedding of a whole prompt: qkv [B, T, (Hq+2*Hkv)*Dh] bf16, positions [T] int32.  Returns the rotated
    queries [B, Hq, T, Dh]; the rotated keys and the values are written to cache rows positions[t] of
    k_cache / v_cache [B, Hkv, S_max, Dh]."""
    _require_cuda(qkv, "rope_prefill input")
    B, T = qkv.shape[0], qkv.shape[1]
    Dh, S_max = k_cache.shape[-1], k_cache.shape[2]
    if (qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16 or positions.dtype != torch.int32
            or positions.numel() != T or qkv.shape[2] != (Hq + 2 * Hkv) * Dh or tuple(k_cache.shape) != (B, Hkv, S_max, Dh)
            or v_cache.shape != k_cache.shape or not (qkv.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous())):
        raise ValueError("rope_prefill: bf16 qkv [B, T, (Hq+2*Hkv)*Dh], int32 positions [T], contiguous bf16 caches [B, Hkv, S, Dh]")
    with torch.cuda.device(qkv.device):
        q = torch.empty((B, Hq, T, Dh), dtype=qkv.dtype, device=qkv.device)
        _lib.check(_lib.load().nf4_b200_rope_prefill(qkv.data_ptr(), positions.contiguous().data_ptr(), q.data_ptr(), k_cache.data_ptr(),
                                                     v_cache.data_ptr(), B, T, Hq, Hkv, Dh, S_max, float(theta),
                                                     _stream_ptr(qkv.device)), "nf4_b200_rope_prefill")
    return q


def silu_mul(gate_up: torch.Tensor, F: int, interleaved: bool) -> torch.Tensor:
    """[rows, 2F] -> [rows, F]: silu(gate) * up with gate/up as halves or as interleaved pairs."""
    _require_cuda(gate_up, "silu_mul input")
    g2 = gate_up.reshape(-1, 2 * F)
    with torch.cuda.device(gate_up.device):
        out = torch.empty((*gate_up.shape[:-1], F), dtype=gate_up.dtype, device=gate_up.device)
        _lib.check(_lib.load().nf4_b200_silu_mul(g2.data_ptr(), out.data_ptr(), g2.shape[0], F, 1 if interleaved else 0,
                                                 _stream_ptr(gate_up.device)), "nf4_b200_silu_mul")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """table[ids] for a bf16 table [vocab, D] and int64 ids of any shape (one launch, 16-byte row copies)."""
    _require_cuda(table, "embedding table")
    if table.dtype != torch.bfloat16 or ids.dtype != torch.int64 or table.dim() != 2 or not table.is_contiguous():
        raise ValueError("embedding: contiguous bf16 table [vocab, D] and int64 ids")
    flat = ids.reshape(-1).contiguous()
    with torch.cuda.device(table.device):
        out = torch.empty((*ids.shape, table.shape[1]), dtype=table.dtype, device=table.device)
        _lib.check(_lib.load().nf4_b200_embed(flat.data_ptr(), table.data_ptr(), out.data_ptr(), flat.numel(), table.shape[1],
                                              table.shape[0], _stream_ptr(table.device)), "nf4_b200_embed")
    return out


def argmax_last(logits: torch.Tensor, keepdim: bool = False) -> torch.Tensor:
    """argmax over the last dimension of a contiguous bf16 tensor; the first maximum wins (as torch.argmax)."""
    _require_cuda(logits, "argmax input")
    if logits.dtype != torch.bfloat16:
        raise ValueError("argmax_last: bf16 only")
    x2 = logits.reshape(-1, logits.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    with torch.cuda.device(logits.device):
        out = torch.empty((x2.shape[0],), dtype=torch.int64, device=logits.device)
        _lib.check(_lib.load().nf4_b200_argmax(x2.data_ptr(), out.data_ptr(), x2.shape[0], x2.shape[1], _stream_ptr(logits.device)),
                   "nf4_b200_argmax")
    shape = (*logits.shape[:-1], 1) if keepdim else logits.shape[:-1]
    return out.view(shape)


def swiglu_halves_available() -> bool:
    """Whether the fused GEMV has the SwiGLU epilogue over [gate rows; up rows] (epilogue 2)."""
    return _lib.HAS_SWIGLU_HALVES
