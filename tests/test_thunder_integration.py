"""Thunder-level behaviour of the NF4 transform / executor / plugin.

CPU tests drive the real trace rewriting with the CPU oracle standing in for the CUDA kernels
(substituted by monkeypatching, test-only); GPU tests run the same models on the kernels.  The
cases mirror the reference's own tests for this path (thunder/tests/test_transforms.py:116-344,
thunder/tests/test_transformer_engine_executor.py:722-760)."""

import numpy as np
import pytest
import torch

import oracle
from helpers import bf16_bits, bits_to_bf16

thunder_support = pytest.importorskip("nf4_b200.thunder_support")
if not thunder_support.thunder_available():
    pytest.skip("thunder is not importable (no baseline/_ref)", allow_module_level=True)

import thunder  # noqa: E402

from nf4_b200 import functional  # noqa: E402
from nf4_b200.codebook import NF4_LEVELS  # noqa: E402
from nf4_b200.thunder_executor import (NF4LinearQuant4bit, QuantizeNF4, get_nf4_executor,  # noqa: E402
                                       install_as_bitsandbytes, register_plugin)

CODE = np.array(NF4_LEVELS, np.float32)


def _oracle_quantize_4bit(A, absmax=None, out=None, blocksize=64, compress_statistics=False, quant_type="nf4",
                          quant_storage=torch.uint8):
    a = A.detach().cpu().contiguous()
    src = bf16_bits(a) if a.dtype == torch.bfloat16 else a.float().numpy()
    packed, am = oracle.quantize(src, CODE, blocksize)
    state = functional.QuantState(absmax=torch.from_numpy(am).to(A.device), shape=A.shape, dtype=A.dtype,
                                  blocksize=blocksize, code=torch.tensor(NF4_LEVELS, dtype=torch.float32, device=A.device))
    return torch.from_numpy(packed).to(A.device), state


def _oracle_linear_nf4(x, packed, bias, absmax, code, blocksize, shape, out=None):
    N, K = int(shape[0]), int(shape[1])
    p, a, c = packed.cpu().numpy(), absmax.cpu().numpy(), code.cpu().numpy()
    x2 = x.detach().cpu().reshape(-1, K)
    if x.dtype == torch.bfloat16:
        y = oracle.linear_bf16(bf16_bits(x2), p, a, c, N, K, blocksize, None if bias is None else bf16_bits(bias.cpu()),
                               mode=oracle.GEMV_MODE)
        y = bits_to_bf16(y)
    else:
        y = torch.from_numpy(oracle.linear_f32(x2.float().numpy(), p, a, c, N, K, blocksize,
                                               None if bias is None else bias.float().cpu().numpy())).to(x.dtype)
    return y.reshape(*x.shape[:-1], N).to(x.device)


@pytest.fixture
def cpu_backend(monkeypatch):
    """Oracle in place of the kernels, and no forced move of weights to CUDA."""
    monkeypatch.setattr(functional, "quantize_4bit", _oracle_quantize_4bit)
    monkeypatch.setattr(functional, "linear_nf4", _oracle_linear_nf4)
    monkeypatch.setattr(NF4LinearQuant4bit, "quantize_weight",
                        lambda self, w: functional.quantize_4bit(torch.zeros_like(w, device="cpu") if w.device.type == "meta" else w,
                                                                 quant_type="nf4"))


def _mlp(dtype=torch.float32, device="cpu"):
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(512, 1024), torch.nn.GELU(), torch.nn.Linear(1024, 512)).to(device, dtype).eval().requires_grad_(False)


def _check_mlp(device, dtype):
    m = _mlp(dtype, device)
    x = torch.randn(1, 512, device=device, dtype=dtype)
    ex = get_nf4_executor()
    jm = thunder.jit(m, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    got = jm(x)
    torch.testing.assert_close(got.float(), m(x).float(), atol=2e-1, rtol=2e-1)   # tolerance of the reference's test
    # the final trace calls the new symbol once per Linear, with the reference's argument layout
    trc = thunder.last_traces(jm)[-1]
    calls = [b for b in trc.bound_symbols if b.sym.name == "nf4_b200_matmul"]
    assert len(calls) == 2
    xarg, w, b, absmax, code, blocksize, dt, shape = calls[0].args
    assert blocksize == 64 and tuple(shape) == (1024, 512) and dt == dtype
    assert tuple(w.shape) == (1024 * 512 // 2, 1) and tuple(absmax.shape) == (1024 * 512 // 64,) and tuple(code.shape) == (16,)
    assert "quant pass" in str([t.get_provenance() for t in thunder.last_traces(jm)])
    # proxies in prologue/computation agree with the runtime tensors (test_transforms.py:220-230)
    sd = jm.state_dict()
    assert set(sd) == {"0.weight", "0.weight.absmax", "0.weight.code", "0.bias", "2.weight", "2.weight.absmax", "2.weight.code", "2.bias"}
    assert sd["0.weight"].dtype == torch.uint8 and sd["0.weight.absmax"].dtype == torch.float32
    cd = thunder.compile_data(jm)
    assert jm._overrides_parameters["0.weight"].device.type == device
    for a in trc.args:
        if a.name.endswith("_absmax"):
            assert a.dtype == thunder.dtypes.float32
    # a second jitted copy that receives the ORIGINAL weights reproduces the first exactly
    # (test_transformer_engine_executor.py:750-760)
    m2 = _mlp(dtype, device)
    jm2 = thunder.jit(m2, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    jm2.load_original_state_dict(m.state_dict())
    torch.testing.assert_close(jm2(x), got)
    for k, v in jm.state_dict().items():
        assert torch.equal(v, jm2.state_dict()[k]), k
    return jm


def test_mlp_cpu(cpu_backend):
    _check_mlp("cpu", torch.float32)
    _check_mlp("cpu", torch.bfloat16)


def test_tied_weights_and_tiny_linear_cpu(cpu_backend):
    """Linear(2,2) with a tied copy: numel 4 < blocksize, shared names preserved
    (thunder/tests/test_transforms.py:293-344)."""
    m0 = torch.nn.Linear(2, 2)
    m4 = torch.nn.Linear(2, 2)
    m4.weight, m4.bias = m0.weight, m0.bias
    torch.manual_seed(1234)
    m = torch.nn.Sequential(m0, torch.nn.GELU(), torch.nn.Linear(2, 2), torch.nn.GELU(), m4).eval().requires_grad_(False)
    x = torch.randn(3, 2)
    jm = thunder.jit(m, transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    y = jm(x)
    assert y.shape == (3, 2)
    assert jm._get_shared_names()["0.weight"] == {"0.weight", "4.weight"}
    assert jm._overrides_parameters["0.weight"] is jm._overrides_parameters["4.weight"]
    assert jm._overrides_parameters["0.weight"].shape == (2, 1) and jm._overrides_parameters["0.weight.absmax"].shape == (1,)
    # against the dequantised weights
    def deq(name):
        p, a = jm._overrides_parameters[name].numpy(), jm._overrides_parameters[name + ".absmax"].numpy()
        return torch.from_numpy(oracle.dequantize(p, a, CODE, 4, 64, out="f32")).view(2, 2)
    h = torch.nn.functional.gelu(x @ deq("0.weight").t() + m0.bias)
    h = torch.nn.functional.gelu(h @ deq("2.weight").t() + m[2].bias)
    torch.testing.assert_close(y, h @ deq("4.weight").t() + m0.bias, atol=1e-4, rtol=1e-4)


def test_plugin_and_alias_routes_cpu(cpu_backend):
    import thunder.plugins

    register_plugin("quantize-nf4-b200")
    assert thunder.plugins.get_plugin("quantize-nf4-b200") is QuantizeNF4
    pl = QuantizeNF4()
    assert isinstance(pl.setup_transforms()[0], NF4LinearQuant4bit) and pl.setup_executors()[0] is get_nf4_executor()
    # the reference's own transform, unmodified, on this package under the name it imports
    mod = install_as_bitsandbytes()
    assert mod.functional.QuantState is functional.QuantState
    import thunder.transforms.quantization as refq

    class RefOnCpu(refq.BitsAndBytesLinearQuant4bit):
        def quantize_weight(self, w):                 # the reference forces .to("cuda") here
            return refq.bitsandbytes.functional.quantize_4bit(w, quant_type="nf4")

    m = _mlp(torch.bfloat16)
    x = torch.randn(2, 512, dtype=torch.bfloat16)
    jref = thunder.jit(m, transforms=[RefOnCpu()], executors=(refq.get_bitsandbytes_executor(),))
    jours = thunder.jit(_mlp(torch.bfloat16), transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    torch.testing.assert_close(jref(x), jours(x), rtol=0, atol=0)
    for k, v in jref.state_dict().items():
        assert torch.equal(v, jours.state_dict()[k]), k


def test_llama_shaped_module_cpu(cpu_backend):
    """The in-repo Llama definition of the reference: 7 quantized linears per layer + the output head,
    the embedding stays bf16 (thunder/tests/llama2_model.py:129-290)."""
    lm = pytest.importorskip("thunder.tests.llama2_model")
    args = lm.ModelArgs(dim=128, n_layers=2, n_heads=2, n_kv_heads=1, vocab_size=256, hidden_dim=256, multiple_of=64, max_seq_len=16)
    torch.manual_seed(0)
    model = lm.Transformer(args).to(torch.bfloat16).eval().requires_grad_(False)
    tokens = torch.randint(0, 256, (1, 8))
    want = model(tokens)
    jm = thunder.jit(model, transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    got = jm(tokens)
    got0 = got[0] if isinstance(got, tuple) else got
    want0 = want[0] if isinstance(want, tuple) else want
    trc = thunder.last_traces(jm)[-1]
    n_calls = sum(1 for b in trc.bound_symbols if b.sym.name == "nf4_b200_matmul")
    assert n_calls == 7 * args.n_layers + 1
    assert jm.state_dict()["output.weight"].dtype == torch.uint8
    assert jm.state_dict()["tok_embeddings.weight"].dtype == torch.bfloat16
    assert torch.isfinite(got0.float()).all()
    assert (got0.float() - want0.float()).abs().max() < 1.0    # 4-bit weights: close to, not equal to, the bf16 model


# ------------------------------------------------------------------------------------- GPU

@pytest.mark.gpu
def test_mlp_gpu():
    _check_mlp("cuda", torch.bfloat16)
    _check_mlp("cuda", torch.float32)


@pytest.mark.gpu
def test_weights_on_host_are_quantized_on_device_and_returned():
    """A CPU model is quantized on the GPU and its packed tensors come back to the CPU
    (quantization.py:53-63, 87-89); packed bytes equal the oracle's."""
    m = _mlp(torch.bfloat16, "cpu")
    jm = thunder.jit(m, transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    sd = jm.state_dict()
    assert sd["0.weight"].device.type == "cpu"
    p_ref, a_ref = oracle.quantize(bf16_bits(m[0].weight.detach()), CODE, 64)
    assert np.array_equal(sd["0.weight"].numpy(), p_ref) and np.array_equal(sd["0.weight.absmax"].numpy(), a_ref)


@pytest.mark.gpu
def test_llama_shaped_module_gpu_matches_oracle_backend(monkeypatch):
    lm = pytest.importorskip("thunder.tests.llama2_model")
    args = lm.ModelArgs(dim=256, n_layers=2, n_heads=2, n_kv_heads=1, vocab_size=512, hidden_dim=512, multiple_of=64, max_seq_len=32)
    torch.manual_seed(0)
    model = lm.Transformer(args).to(torch.bfloat16).eval().requires_grad_(False)
    tokens = torch.randint(0, 512, (1, 4))
    jm = thunder.jit(model.cuda(), transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    got = jm(tokens.cuda())
    got0 = (got[0] if isinstance(got, tuple) else got).float().cpu()
    # same model through the oracle backend on the CPU
    monkeypatch.setattr(functional, "quantize_4bit", _oracle_quantize_4bit)
    monkeypatch.setattr(functional, "linear_nf4", _oracle_linear_nf4)
    monkeypatch.setattr(NF4LinearQuant4bit, "quantize_weight", lambda self, w: functional.quantize_4bit(w, quant_type="nf4"))
    jc = thunder.jit(model.cpu(), transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    want = jc(tokens)
    want0 = (want[0] if isinstance(want, tuple) else want).float()
    torch.testing.assert_close(got0, want0, rtol=5e-2, atol=5e-2)


def _meta_mlp(dtype):
    with torch.device("meta"):
        return torch.nn.Sequential(torch.nn.Linear(512, 1024), torch.nn.GELU(), torch.nn.Linear(1024, 512)).to(dtype).eval().requires_grad_(False)


def test_materialization_routes_cpu(cpu_backend):
    """The three ways the reference builds a quantized module give the same parameters and outputs
    (thunder/tests/test_transforms.py:116-186): from real weights; from a meta-device module filled from the
    ORIGINAL state dict (quantized while loading, submodule by submodule); from a meta-device module
    filled from the TRANSFORMED (already quantized) state dict."""
    from thunder.transforms import MaterializationTransform

    ex = get_nf4_executor()
    dtype = torch.bfloat16
    ref = _mlp(dtype)
    jm_ref = thunder.jit(ref, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    init_orig = MaterializationTransform.init_from_original_state_dict(ref.state_dict())
    jm = thunder.jit(_meta_mlp(dtype), transforms=[NF4LinearQuant4bit(), MaterializationTransform("cpu", init=init_orig)],
                     executors=(ex,))
    init_tr = MaterializationTransform.init_from_transformed_state_dict(jm_ref.state_dict())
    jm2 = thunder.jit(_meta_mlp(dtype), transforms=[NF4LinearQuant4bit(), MaterializationTransform("cpu", init=init_tr)],
                      executors=(ex,))
    x = torch.randn(2, 512, dtype=dtype)
    expected = jm_ref(x)
    assert torch.equal(jm(x), expected) and torch.equal(jm2(x), expected)
    for n, p in jm_ref.named_parameters():
        assert torch.equal(jm.get_parameter(n), p), n
        assert torch.equal(jm2.get_parameter(n), p), n
        assert jm.get_parameter(n).device.type == "cpu"
    assert set(jm.state_dict()) == set(jm_ref.state_dict())


def test_materialization_from_module_init_with_tied_weights_cpu(cpu_backend):
    """Meta-device module materialised by re-running the modules' own initialisers, with a tied Linear(2, 2)
    (numel 4 < blocksize) -- thunder/tests/test_transforms.py:293-344."""
    from thunder.transforms import MaterializationTransform

    def get_model():
        m0 = torch.nn.Linear(2, 2)
        with torch.device("meta"):      # not to change the rng state
            m4 = torch.nn.Linear(2, 2)
        m4.weight, m4.bias = m0.weight, m0.bias
        return torch.nn.Sequential(m0, torch.nn.GELU(), torch.nn.Linear(2, 2), torch.nn.GELU(), m4).eval().requires_grad_(False)

    ex = get_nf4_executor()
    torch.manual_seed(1234)
    m_ref = get_model()
    inp = torch.randn(3, 2)
    jm_ref = thunder.jit(m_ref, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    torch.manual_seed(1234)
    with torch.device("meta"):
        m = get_model()
    jm = thunder.jit(m, transforms=[NF4LinearQuant4bit(),
                                    MaterializationTransform("cpu", init=MaterializationTransform.init_from_original_module_init())],
                     executors=(ex,))
    torch.testing.assert_close(jm(inp), jm_ref(inp))
    assert jm_ref._get_shared_names()["0.weight"] == {"0.weight", "4.weight"}
    assert jm._get_shared_names()["0.weight"] == {"0.weight", "4.weight"}


@pytest.mark.gpu
def test_materialization_routes_gpu():
    """The same three routes on the kernels: a meta-device module is materialised on the GPU and its
    weights are quantized there, shard by shard of the state dict (thunder/tests/test_transforms.py:116-186)."""
    from thunder.transforms import MaterializationTransform

    ex = get_nf4_executor()
    dtype = torch.bfloat16
    ref = _mlp(dtype, "cuda")
    jm_ref = thunder.jit(ref, transforms=[NF4LinearQuant4bit()], executors=(ex,))

    def meta():
        m = _meta_mlp(dtype)
        for p in m.parameters():
            p._thunder_device = torch.device("cuda")
        return m

    init_orig = MaterializationTransform.init_from_original_state_dict(ref.state_dict())
    jm = thunder.jit(meta(), transforms=[NF4LinearQuant4bit(), MaterializationTransform("cuda", init=init_orig)], executors=(ex,))
    init_tr = MaterializationTransform.init_from_transformed_state_dict(jm_ref.state_dict())
    jm2 = thunder.jit(meta(), transforms=[NF4LinearQuant4bit(), MaterializationTransform("cuda", init=init_tr)], executors=(ex,))
    x = torch.randn(2, 512, dtype=dtype, device="cuda")
    expected = jm_ref(x)
    assert torch.equal(jm(x), expected) and torch.equal(jm2(x), expected)
    for n, p in jm_ref.named_parameters():
        assert torch.equal(jm.get_parameter(n), p), n
        assert torch.equal(jm2.get_parameter(n), p), n
        assert jm.get_parameter(n).device.type == "cuda"
    torch.testing.assert_close(expected.float(), ref(x).float(), atol=2e-1, rtol=2e-1)


@pytest.mark.gpu
def test_cuda_graph_transform_gpu():
    """The quantized linears inside Thunder's CUDA-graph transform (thunder/transforms/cudagraph.py:229-387,
    what the reduce-overhead plugin installs): the op allocates nothing but its output, launches on the
    current stream and keeps no per-call host state, so regions containing it capture and replay.  One row
    (fused GEMV) and 40 rows (tensor-core GEMM) of activations."""
    from thunder.transforms.cudagraph import CUDAGraphTransform

    ex = get_nf4_executor()
    m = _mlp(torch.bfloat16, "cuda")
    jm_plain = thunder.jit(m, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    jm_graph = thunder.jit(m, transforms=[NF4LinearQuant4bit(), CUDAGraphTransform()], executors=(ex,))
    g = torch.Generator(device="cuda").manual_seed(3)
    for rows in (1, 40):
        for _ in range(3):      # first call captures, later calls replay with new input values
            x = torch.randn(rows, 512, device="cuda", dtype=torch.bfloat16, generator=g)
            y = jm_graph(x)
            torch.testing.assert_close(y, jm_plain(x), rtol=1.6e-2, atol=1e-2)
            # and against a third party that shares no kernel with either: the oracle's linears around torch's GELU
            h = x.cpu()
            for i in (0, 2):
                h = _oracle_linear_nf4(h, jm_graph.get_parameter(f"{i}.weight"), m[i].bias.detach().cpu(),
                                       jm_graph.get_parameter(f"{i}.weight.absmax"), jm_graph.get_parameter(f"{i}.weight.code"),
                                       64, m[i].weight.shape)
                if i == 0:
                    h = torch.nn.functional.gelu(h.float()).to(torch.bfloat16)
            torch.testing.assert_close(y.float().cpu(), h.float(), rtol=3e-2, atol=3e-2)
    trc = thunder.last_traces(jm_graph)[-1]
    assert any("CUDAGraph" in b.sym.name for b in trc.bound_symbols), [b.sym.name for b in trc.bound_symbols]
    from nf4_b200 import _lib
    assert _lib.device_error()[0] == 0


# ------------------------------------------------------------------------------------- gradients

def _oracle_input_grad(g, packed, absmax, code, blocksize, shape):
    N, K = int(shape[0]), int(shape[1])
    w = torch.from_numpy(oracle.dequantize(packed.cpu().numpy().reshape(-1), absmax.cpu().numpy(), code.cpu().numpy(), N * K,
                                           int(blocksize), out="f32")).view(N, K)
    return (g.detach().float().cpu() @ w).to(g.dtype).to(g.device)


def _check_input_gradient(device, dtype):
    """y = model(x) through the quantized linears, loss = sum(y * r): x.grad against the gradient of the same
    model with the DEQUANTIZED weights in fp32 (the weights themselves are frozen and get no gradient)."""
    m = _mlp(dtype, device)
    ex = get_nf4_executor()
    jm = thunder.jit(m, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    g = torch.Generator().manual_seed(11)
    x = torch.randn((4, 512), generator=g).to(device=device, dtype=dtype).requires_grad_(True)
    r = torch.randn((4, 512), generator=g).to(device=device, dtype=dtype)
    y = jm(x)
    (y * r).sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape
    names = [b.sym.name for t in thunder.last_backward_traces(jm)[-1:] for b in t.bound_symbols]
    assert names.count("nf4_b200_matmul_bwd") == 2, names

    def deq(i):
        p = jm.get_parameter(f"{i}.weight").cpu().numpy().reshape(-1)
        a = jm.get_parameter(f"{i}.weight.absmax").cpu().numpy()
        n, k = m[i].weight.shape
        return torch.from_numpy(oracle.dequantize(p, a, CODE, n * k, 64, out="f32")).view(n, k)

    x32 = x.detach().float().cpu().requires_grad_(True)
    h = torch.nn.functional.gelu(x32 @ deq(0).t() + m[0].bias.float().cpu())
    y32 = h @ deq(2).t() + m[2].bias.float().cpu()
    (y32 * r.float().cpu()).sum().backward()
    tol = dict(rtol=1e-3, atol=1e-3) if dtype == torch.float32 else dict(rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(x.grad.float().cpu(), x32.grad, **tol)
    torch.testing.assert_close(y.detach().float().cpu(), y32.detach(), **tol)


def test_input_gradient_cpu(cpu_backend, monkeypatch):
    monkeypatch.setattr(functional, "linear_nf4_input_grad", _oracle_input_grad)
    _check_input_gradient("cpu", torch.float32)


def test_qlora_composition_cpu(cpu_backend, monkeypatch):
    """The reference's LoRA transform (thunder/transforms/qlora.py:15-238) in front of the NF4 transform: the
    adapters' matmuls stay in 32 bits, the wrapped linear runs on the quantized weight, and the gradient of the
    input flows back through both.  (The reference creates the adapters with requires_grad=False and checks that
    in its prologue, so the quantity that can be differentiated through the stock transform is the input.)"""
    from thunder.transforms import LORATransform

    monkeypatch.setattr(functional, "linear_nf4_input_grad", _oracle_input_grad)
    torch.manual_seed(0)     # square layers, as in the reference's own LoRA test (thunder/tests/test_transforms.py:347-394)
    m = torch.nn.Sequential(torch.nn.Linear(512, 512), torch.nn.GELU(), torch.nn.Linear(512, 512)).eval().requires_grad_(False)

    class SeededLora(LORATransform):
        def init_lora_linear(self, lora_a, lora_b):          # the stock init zeroes lora_b: the adapters would be inert
            g = torch.Generator().manual_seed(lora_a.numel())
            with torch.no_grad():
                lora_a.copy_(torch.randn(lora_a.shape, generator=g) * 0.05)
                lora_b.copy_(torch.randn(lora_b.shape, generator=g) * 0.05)

    lora = SeededLora(r=8, lora_alpha=16)
    jm = thunder.jit(m, transforms=[lora, NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    x = torch.randn(3, 512).requires_grad_(True)
    y = jm(x)
    names = [b.sym.name for b in thunder.last_traces(jm)[-1].bound_symbols]
    assert names.count("nf4_b200_matmul") == 2
    assert jm.get_parameter("0.weight").dtype == torch.uint8 and jm.get_parameter("0.weight.lora_a").shape == (8, 512)
    y.sum().backward()
    bwd = [b.sym.name for b in thunder.last_backward_traces(jm)[-1].bound_symbols]
    assert bwd.count("nf4_b200_matmul_bwd") == 2

    # the same function in plain torch on the dequantised weights
    def deq(i):
        p = jm.get_parameter(f"{i}.weight").numpy().reshape(-1)
        a = jm.get_parameter(f"{i}.weight.absmax").numpy()
        n, k = m[i].weight.shape
        return torch.from_numpy(oracle.dequantize(p, a, CODE, n * k, 64, out="f32")).view(n, k)

    A0, B0, A2, B2 = (jm.get_parameter(n).detach() for n in ("0.weight.lora_a", "0.weight.lora_b", "2.weight.lora_a", "2.weight.lora_b"))
    x2 = x.detach().clone().requires_grad_(True)
    h = torch.nn.functional.gelu(x2 @ deq(0).t() + m[0].bias + (x2 @ A0.t() @ B0.t()) * lora.scaling)
    y_ref = h @ deq(2).t() + m[2].bias + (h @ A2.t() @ B2.t()) * lora.scaling
    y_ref.sum().backward()
    torch.testing.assert_close(y, y_ref, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-3, atol=1e-3)


@pytest.mark.gpu
def test_input_gradient_gpu():
    _check_input_gradient("cuda", torch.bfloat16)
    _check_input_gradient("cuda", torch.float32)


def test_plugin_route_through_thunder_compile_cpu(cpu_backend):
    """`thunder.compile(model, recipe=..., plugins="quantize-int4")` with the plugin name re-bound to this
    package (thunder/plugins/quantization.py:4-37 is the reference's plugin; thunder/core/recipe.py:141-165 puts a
    plugin's transforms and executors in front of the recipe's own).  The default recipe asks for nvFuser and its
    alternative for Inductor; this environment has neither a usable one, so the recipe is the base recipe
    with the fusion backend left out (BaseRecipe is documented as the template to extend): PrunePrologueChecks
    plus the always-on torch / python executors behind the plugin's."""
    import thunder.plugins
    from thunder.recipes import BaseRecipe

    class NoFuserRecipe(BaseRecipe):
        def setup_fuser(self):
            self.fuser = None

    previous = thunder.plugins.get_plugin("quantize-int4")
    register_plugin()                       # "quantize-int4" -> QuantizeNF4
    try:
        assert thunder.plugins.get_plugin("quantize-int4") is QuantizeNF4
        m = _mlp(torch.bfloat16)
        x = torch.randn(2, 512, dtype=torch.bfloat16)
        jm = thunder.compile(m, recipe=NoFuserRecipe(fuser="torch.compile"), plugins="quantize-int4")
        y = jm(x)
        names = [b.sym.name for b in thunder.last_traces(jm)[-1].bound_symbols]
        assert names.count("nf4_b200_matmul") == 2
        assert jm.state_dict()["0.weight"].dtype == torch.uint8
        direct = thunder.jit(_mlp(torch.bfloat16), transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
        torch.testing.assert_close(y, direct(x), rtol=0, atol=0)
    finally:
        if previous is not None:
            thunder.plugins.register_plugin("quantize-int4", previous)


@pytest.mark.gpu
def test_nvtx_ranges_wrap_the_nf4_symbol_gpu():
    """thunder.dev_utils.nvtx_profile_transform.NvtxProfileTransform (nvtx_profile_transform.py:26-76) composes with
    the executor: every nf4_b200_matmul call of the execution trace sits between a range push that names it and
    a pop, and the module still computes the same values."""
    from thunder.dev_utils.nvtx_profile_transform import NvtxProfileTransform

    ex = get_nf4_executor()
    m = _mlp(torch.bfloat16, "cuda")
    jm = thunder.jit(m, transforms=[NF4LinearQuant4bit(), NvtxProfileTransform()], executors=(ex,))
    plain = thunder.jit(m, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    x = torch.randn(2, 512, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(jm(x), plain(x))
    bs = thunder.last_traces(jm)[-1].bound_symbols
    at = [i for i, b in enumerate(bs) if b.sym.name == "nf4_b200_matmul"]
    assert len(at) == 2
    for i in at:
        assert bs[i - 1].sym.name == "nvtx_range_push" and "nf4_b200_matmul" in bs[i - 1].args[0]
        assert bs[i + 1].sym.name == "nvtx_range_pop"
