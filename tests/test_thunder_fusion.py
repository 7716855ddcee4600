"""The decode-step fusion pass (nf4_b200.fusion.NF4DecodeFusion) on the Llama-shaped module with a KV
cache (nf4_b200.llama): which symbols the rewritten trace holds, that parameters keep their names, shapes
and values, and that a fused and an unfused jitted copy of the same model decode the same logits.

CPU tests run the block symbols on CPU checkers (oracle for the quantized products, torch for the glue);
GPU tests run them on the kernels and compare with the oracle-backed unfused module."""

import pytest
import torch

from helpers import cpu_attn_decode_fused, cpu_gemv_decode, cpu_rms_norm_rows, cpu_rope_prefill, cpu_silu_mul
from test_thunder_integration import _oracle_linear_nf4, _oracle_quantize_4bit

thunder_support = pytest.importorskip("nf4_b200.thunder_support")
if not thunder_support.thunder_available():
    pytest.skip("thunder is not importable (no baseline/_ref)", allow_module_level=True)

import thunder  # noqa: E402

from nf4_b200 import functional  # noqa: E402
from nf4_b200.fusion import NF4DecodeFusion  # noqa: E402
from nf4_b200.llama import LlamaArgs, LlamaDecoder  # noqa: E402
from nf4_b200.thunder_executor import NF4LinearQuant4bit, get_nf4_executor  # noqa: E402


@pytest.fixture
def cpu_backend(monkeypatch):
    monkeypatch.setattr(functional, "quantize_4bit", _oracle_quantize_4bit)
    monkeypatch.setattr(functional, "linear_nf4", _oracle_linear_nf4)
    monkeypatch.setattr(functional, "gemv_decode", cpu_gemv_decode)
    monkeypatch.setattr(functional, "gemv_decode_fits", lambda M, N, K, prologue: True)
    monkeypatch.setattr(functional, "attn_decode_fused", cpu_attn_decode_fused)
    monkeypatch.setattr(functional, "silu_mul", cpu_silu_mul)
    monkeypatch.setattr(functional, "rms_norm_rows", cpu_rms_norm_rows)
    monkeypatch.setattr(functional, "rope_prefill", cpu_rope_prefill)
    monkeypatch.setattr(functional, "swiglu_halves_available", lambda: True)
    monkeypatch.setattr(NF4LinearQuant4bit, "quantize_weight", lambda self, w: functional.quantize_4bit(w, quant_type="nf4"))


def tiny_args(**kw):
    base = dict(dim=256, n_layers=2, n_heads=2, n_kv_heads=1, vocab_size=512, hidden_dim=512, max_seq_len=32, max_batch=2)
    base.update(kw)
    return LlamaArgs(**base)


def build(args, device="cpu", seed=1):
    # weights are drawn on the CPU generator whatever the device, so a CPU and a GPU copy are the same model
    m = LlamaDecoder(args).to(dtype=torch.bfloat16).eval().requires_grad_(False)
    m.init_weights(seed)
    m = m.to(device)
    m.reset_rope_tables()
    return m


def _names(trc):
    return [b.sym.name for b in trc.bound_symbols]


def _decode(jm, steps, B, vocab, seed=3):
    g = torch.Generator().manual_seed(seed)
    dev = next(iter(jm.state_dict().values())).device
    outs = []
    for p in range(steps):
        tok = torch.randint(0, vocab, (B, 1), generator=g).to(dev)
        outs.append(jm(tok, torch.tensor([p], device=dev)).float().cpu())
    return torch.stack(outs)


def test_trace_is_rewritten_and_matches_unfused_cpu(cpu_backend):
    args = tiny_args()
    ex = get_nf4_executor()
    fusion = NF4DecodeFusion()
    jf = thunder.jit(build(args), transforms=[NF4LinearQuant4bit(), fusion], executors=(ex,))
    ju = thunder.jit(build(args), transforms=[NF4LinearQuant4bit()], executors=(ex,))
    got = _decode(jf, 5, 2, args.vocab_size)
    want = _decode(ju, 5, 2, args.vocab_size)
    names = _names(thunder.last_traces(jf)[-1])
    assert names.count("nf4_b200_attn_block") == args.n_layers
    assert names.count("nf4_b200_mlp_block") == args.n_layers
    assert names.count("nf4_b200_norm_linear") == 1
    assert names.count("nf4_b200_positions") == 1
    assert "nf4_b200_matmul" not in names and "scaled_dot_product_attention" not in names
    assert not any(n in names for n in ("index_copy_", "index_copy", "rms_norm", "silu")), names
    assert fusion.fused == {"attn": 2, "mlp": 2, "norm_linear": 1} and not fusion.declined
    assert "NF4 decode fusion" in str([t.get_provenance() for t in thunder.last_traces(jf)])
    torch.testing.assert_close(got, want, rtol=1.6e-2, atol=1e-2)
    # the caches were written in place by the fused block, exactly where the unfused module wrote them
    for li in range(args.n_layers):
        kf = jf.get_buffer(f"layers.{li}.attention.k_cache")
        ku = ju.get_buffer(f"layers.{li}.attention.k_cache")
        assert kf[:, :, 5:].abs().max() == 0 and kf[:, :, :5].abs().max() > 0
        torch.testing.assert_close(kf.float(), ku.float(), rtol=1.6e-2, atol=1e-2)


def test_parameters_keep_names_shapes_and_values_cpu(cpu_backend):
    """Q/K/V and gate/up become views into one allocation each; the state dict is unchanged and loading the
    original weights again (thunder/core/module.py:137-190 copies in place) keeps them adjacent."""
    args = tiny_args()
    ex = get_nf4_executor()
    model = build(args)
    jf = thunder.jit(model, transforms=[NF4LinearQuant4bit(), NF4DecodeFusion()], executors=(ex,))
    ju = thunder.jit(build(args), transforms=[NF4LinearQuant4bit()], executors=(ex,))
    _decode(jf, 1, 2, args.vocab_size)
    sf, su = jf.state_dict(), ju.state_dict()
    assert list(sf) == list(su)
    for k in su:
        assert sf[k].shape == su[k].shape and sf[k].dtype == su[k].dtype and torch.equal(sf[k], su[k]), k
    p = "layers.0.attention."
    wq, wk, wv = (jf.get_parameter(p + n + ".weight") for n in ("wq", "wk", "wv"))
    assert wk.data_ptr() == wq.data_ptr() + wq.numel() and wv.data_ptr() == wk.data_ptr() + wk.numel()
    aq, ak = jf.get_parameter(p + "wq.weight.absmax"), jf.get_parameter(p + "wk.weight.absmax")
    assert ak.data_ptr() == aq.data_ptr() + 4 * aq.numel()
    w1, w3 = jf.get_parameter("layers.1.feed_forward.w1.weight"), jf.get_parameter("layers.1.feed_forward.w3.weight")
    assert w3.data_ptr() == w1.data_ptr() + w1.numel()
    other = build(args, seed=7)
    jf.load_original_state_dict(other.state_dict())
    jo = thunder.jit(other, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    assert jf.get_parameter(p + "wk.weight").data_ptr() == jf.get_parameter(p + "wq.weight").data_ptr() + wq.numel()
    for k, v in jo.state_dict().items():
        assert torch.equal(jf.state_dict()[k], v), k


def test_prefill_trace_is_rewritten_too_cpu(cpu_backend):
    """A prompt of 24 tokens (more than the fused GEMV's 16 rows): the same block symbols, whose implementations run
    on the GEMM and the one-launch glue kernels; logits and KV cache match the unfused jitted module, and decoding
    continues from that cache on the single-token blocks."""
    args = tiny_args(max_batch=1)
    fusion = NF4DecodeFusion()
    ex = get_nf4_executor()
    jf = thunder.jit(build(args), transforms=[NF4LinearQuant4bit(), fusion], executors=(ex,))
    ju = thunder.jit(build(args), transforms=[NF4LinearQuant4bit()], executors=(ex,))
    tok = torch.randint(0, args.vocab_size, (1, 24))
    y, yu = jf(tok, torch.arange(24)), ju(tok, torch.arange(24))
    assert y.shape == (1, 1, args.vocab_size)
    names = _names(thunder.last_traces(jf)[-1])
    assert names.count("nf4_b200_attn_block") == args.n_layers and names.count("nf4_b200_mlp_block") == args.n_layers
    assert "nf4_b200_matmul" not in names and names.count("nf4_b200_norm_linear") == 1 and not fusion.declined
    torch.testing.assert_close(y.float(), yu.float(), rtol=3e-2, atol=3e-2)
    for name, buf in jf._model.named_buffers():
        if name.endswith("k_cache") or name.endswith("v_cache"):
            other = dict(ju._model.named_buffers())[name]
            torch.testing.assert_close(buf[:, :, :24].float(), other[:, :, :24].float(), rtol=3e-2, atol=3e-2)
            assert not buf[:, :, 24:].any()
    # the same module then decodes token by token on the fused blocks (a second trace for the new shapes)
    nxt = torch.randint(0, args.vocab_size, (1, 1))
    y1, y1u = jf(nxt, torch.tensor([24])), ju(nxt, torch.tensor([24]))
    assert "nf4_b200_attn_block" in _names(thunder.last_traces(jf)[-1])
    torch.testing.assert_close(y1.float(), y1u.float(), rtol=3e-2, atol=3e-2)


def test_many_sequences_single_token_attention_is_declined_cpu(cpu_backend):
    """A single-token step of more than 16 sequences: the attention kernel's limit; the MLP blocks still fuse."""
    args = tiny_args(max_batch=20, n_layers=1)
    fusion = NF4DecodeFusion()
    jf = thunder.jit(build(args), transforms=[NF4LinearQuant4bit(), fusion], executors=(get_nf4_executor(),))
    y = jf(torch.randint(0, args.vocab_size, (20, 1)), torch.tensor([0]))
    assert y.shape == (20, 1, args.vocab_size)
    names = _names(thunder.last_traces(jf)[-1])
    assert "nf4_b200_attn_block" not in names and names.count("nf4_b200_mlp_block") == 1
    assert fusion.declined and "16 sequences" in fusion.declined[0]


def test_pinned_members_are_the_same_objects_cpu(cpu_backend):
    """PinModuleMembers: every parameter and buffer the other transforms left alone becomes an override of itself
    (the same tensor object, so in-place updates stay visible), quantized members keep their overrides, the state
    dict is unchanged and the module decodes the same logits."""
    from nf4_b200.thunder_decode import PinModuleMembers

    args = tiny_args()
    ex = get_nf4_executor()
    plain = thunder.jit(build(args), transforms=[NF4LinearQuant4bit(), NF4DecodeFusion()], executors=(ex,))
    pinned = thunder.jit(build(args), transforms=[NF4LinearQuant4bit(), NF4DecodeFusion(), PinModuleMembers()], executors=(ex,))
    inner = pinned._model
    for name, p in inner.named_parameters(remove_duplicate=False):
        assert name in pinned._overrides_parameters
        if not name.endswith(("wq.weight", "wk.weight", "wv.weight", "wo.weight", "w1.weight", "w2.weight", "w3.weight", "output.weight")):
            assert pinned._overrides_parameters[name] is p, name
    for name, b in inner.named_buffers(remove_duplicate=False):
        assert pinned._overrides_buffers[name] is b, name
    assert pinned.get_parameter("layers.0.attention.wq.weight").dtype == torch.uint8      # the quantized override won
    for k, v in plain.state_dict().items():
        assert torch.equal(pinned.state_dict()[k], v), k
    torch.testing.assert_close(_decode(pinned, 3, 2, args.vocab_size), _decode(plain, 3, 2, args.vocab_size), rtol=0, atol=0)


def test_other_rope_base_is_declined_cpu(cpu_backend):
    args = tiny_args()
    fusion = NF4DecodeFusion(rope_theta=10000.0)          # the module's tables use 500000
    jf = thunder.jit(build(args), transforms=[NF4LinearQuant4bit(), fusion], executors=(get_nf4_executor(),))
    _decode(jf, 1, 2, args.vocab_size)
    names = _names(thunder.last_traces(jf)[-1])
    assert "nf4_b200_attn_block" not in names and names.count("nf4_b200_mlp_block") == args.n_layers
    assert any("rope tables" in d for d in fusion.declined)


# ------------------------------------------------------------------------------------------ GPU

@pytest.mark.gpu
@pytest.mark.parametrize("B", [1, 4])
def test_fused_decode_on_kernels_matches_oracle_backend(monkeypatch, B):
    """Jitted + fused + CUDA-graphed decode on the GPU against the unfused module on the CPU oracle."""
    from thunder.transforms.cudagraph import CUDAGraphTransform

    from nf4_b200 import _lib

    args = tiny_args(dim=512, n_heads=4, n_kv_heads=2, hidden_dim=1024, vocab_size=2048, max_seq_len=64, max_batch=B)
    ex = get_nf4_executor()
    fusion = NF4DecodeFusion()
    jg = thunder.jit(build(args, "cuda"), transforms=[NF4LinearQuant4bit(), fusion, CUDAGraphTransform()], executors=(ex,))
    got = _decode(jg, 6, B, args.vocab_size)
    assert fusion.fused["attn"] == args.n_layers and not fusion.declined
    names = _names(thunder.last_traces(jg)[-1])
    assert any("CUDAGraph" in n for n in names)
    # the embedding lookup was claimed by this executor too (bf16 table on CUDA), inside the captured region
    region = [b for b in thunder.last_traces(jg)[-1].bound_symbols if "CUDAGraph" in b.sym.name][0]
    assert "nf4_b200_embedding" in [s.sym.name for s in region.subsymbols]
    assert _lib.device_error()[0] == 0
    monkeypatch.setattr(functional, "quantize_4bit", _oracle_quantize_4bit)
    monkeypatch.setattr(functional, "linear_nf4", _oracle_linear_nf4)
    monkeypatch.setattr(NF4LinearQuant4bit, "quantize_weight", lambda self, w: functional.quantize_4bit(w, quant_type="nf4"))
    jc = thunder.jit(build(args, "cpu"), transforms=[NF4LinearQuant4bit()], executors=(ex,))
    want = _decode(jc, 6, B, args.vocab_size)
    torch.testing.assert_close(got, want, rtol=5e-2, atol=5e-2)
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.9


@pytest.mark.gpu
def test_greedy_step_claims_embedding_and_argmax_gpu():
    """GreedyStep (model + argmax) jitted by compile_decoder: token embedding and greedy argmax run on this
    library's kernels (claimed through register_implementation + checker), and the sampled ids equal torch's
    argmax over the logits of the same module without the final op."""
    from nf4_b200.thunder_decode import GreedyStep, compile_decoder

    args = tiny_args(dim=512, n_heads=4, n_kv_heads=2, hidden_dim=1024, vocab_size=2048, max_seq_len=64, max_batch=2)
    js = compile_decoder(GreedyStep(build(args, "cuda")))
    jl = compile_decoder(build(args, "cuda"))
    g = torch.Generator().manual_seed(5)
    for p in range(4):
        tok = torch.randint(0, args.vocab_size, (2, 1), generator=g).cuda()
        pos = torch.tensor([p], device="cuda")
        ids = js(tok, pos).clone()
        logits = jl(tok, pos)
        assert ids.shape == (2, 1) and ids.dtype == torch.int64
        assert torch.equal(ids, logits[:, -1, :].float().argmax(-1, keepdim=True))
    region = [b for b in thunder.last_traces(js)[-1].bound_symbols if "CUDAGraph" in b.sym.name][0]
    inner = [s.sym.name for s in region.subsymbols]
    assert "nf4_b200_embedding" in inner and "nf4_b200_argmax" in inner


@pytest.mark.gpu
def test_fused_prefill_on_kernels_matches_oracle_backend(monkeypatch):
    """A 40-token prompt for 2 sequences through the fused blocks on the GPU (RMSNorm, rotary + cache write and
    SiLU * up as single launches, the linears on the dequant-GEMM, torch's fused attention over the cache), then
    three single-token steps from that cache -- against the unfused module on the CPU oracle."""
    from nf4_b200 import _lib

    B, T = 2, 40
    args = tiny_args(dim=512, n_heads=4, n_kv_heads=2, hidden_dim=1024, vocab_size=2048, max_seq_len=64, max_batch=B)
    ex = get_nf4_executor()
    fusion = NF4DecodeFusion()
    jg = thunder.jit(build(args, "cuda"), transforms=[NF4LinearQuant4bit(), fusion], executors=(ex,))
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, args.vocab_size, (B, T), generator=g)
    steps = [torch.randint(0, args.vocab_size, (B, 1), generator=g) for _ in range(3)]

    def run(jm, dev):
        outs = [jm(prompt.to(dev), torch.arange(T, device=dev)).float().cpu()]
        for i, tok in enumerate(steps):
            outs.append(jm(tok.to(dev), torch.tensor([T + i], device=dev)).float().cpu())
        return torch.stack(outs)

    got = run(jg, "cuda")
    assert fusion.fused["attn"] == 2 * args.n_layers and fusion.fused["mlp"] == 2 * args.n_layers and not fusion.declined
    assert _lib.device_error()[0] == 0
    caches = {n: b.float().cpu() for n, b in jg._model.named_buffers() if n.endswith("_cache")}
    monkeypatch.setattr(functional, "quantize_4bit", _oracle_quantize_4bit)
    monkeypatch.setattr(functional, "linear_nf4", _oracle_linear_nf4)
    monkeypatch.setattr(NF4LinearQuant4bit, "quantize_weight", lambda self, w: functional.quantize_4bit(w, quant_type="nf4"))
    jc = thunder.jit(build(args, "cpu"), transforms=[NF4LinearQuant4bit()], executors=(ex,))
    want = run(jc, "cpu")
    torch.testing.assert_close(got, want, rtol=5e-2, atol=5e-2)
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.9
    for n, b in jc._model.named_buffers():
        if n.endswith("_cache"):
            torch.testing.assert_close(caches[n], b.float(), rtol=5e-2, atol=5e-2)
            assert not caches[n][:, :, T + 3:].any()


@pytest.mark.gpu
def test_rope_prefill_kernel_matches_the_single_token_kernel():
    """The prompt form of the rotary embedding writes the same cache rows (bit for bit) as feeding the tokens one
    by one through nf4_b200_rope_append, and returns the same rotated queries in attention layout."""
    import ctypes

    from nf4_b200 import _lib

    lib = _lib.load()
    B, T, Hq, Hkv, Dh, S = 3, 37, 8, 2, 128, 48
    g = torch.Generator(device="cuda").manual_seed(4)
    qkv = torch.randn((B, T, (Hq + 2 * Hkv) * Dh), device="cuda", generator=g).to(torch.bfloat16)
    pos = torch.randperm(S, device="cuda", generator=g)[:T].to(torch.int32)
    kc, vc = (torch.zeros((B, Hkv, S, Dh), device="cuda", dtype=torch.bfloat16) for _ in range(2))
    q4 = functional.rope_prefill(qkv, pos, kc, vc, Hq, Hkv, 5e5)
    kr, vr = torch.zeros_like(kc), torch.zeros_like(vc)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for t in range(T):
        q1 = torch.empty((B, Hq * Dh), device="cuda", dtype=torch.bfloat16)
        row = qkv[:, t].contiguous()
        p = pos[t].expand(B).contiguous()
        _lib.check(lib.nf4_b200_rope_append(row.data_ptr(), p.data_ptr(), q1.data_ptr(), kr.data_ptr(), vr.data_ptr(), B, Hq, Hkv, Dh,
                                            S, 5e5, st), "rope_append")
        assert torch.equal(q4[:, :, t], q1.view(B, Hq, Dh))
    assert torch.equal(kc, kr) and torch.equal(vc, vr)
    assert _lib.device_error()[0] == 0
