"""Streaming quantize-on-load (nf4_b200.loader): a checkpoint arrives as an iterator of (name, tensor) and is
quantized submodule by submodule into a meta-device module materialised by the reference's
MaterializationTransform (thunder/transforms/materialization.py:92-172)."""

import pytest
import torch

from test_thunder_integration import _oracle_linear_nf4, _oracle_quantize_4bit

thunder_support = pytest.importorskip("nf4_b200.thunder_support")
if not thunder_support.thunder_available():
    pytest.skip("thunder is not importable (no baseline/_ref)", allow_module_level=True)

import thunder  # noqa: E402
from thunder.transforms import MaterializationTransform  # noqa: E402

from nf4_b200 import functional  # noqa: E402
from nf4_b200.llama import LlamaArgs, LlamaDecoder  # noqa: E402
from nf4_b200.loader import init_from_tensor_stream, seeded_tensors, stream_load  # noqa: E402
from nf4_b200.thunder_executor import NF4LinearQuant4bit, get_nf4_executor  # noqa: E402


@pytest.fixture
def cpu_backend(monkeypatch):
    monkeypatch.setattr(functional, "quantize_4bit", _oracle_quantize_4bit)
    monkeypatch.setattr(functional, "linear_nf4", _oracle_linear_nf4)
    monkeypatch.setattr(NF4LinearQuant4bit, "quantize_weight",
                        lambda self, w: functional.quantize_4bit(torch.zeros_like(w, device="cpu") if w.device.type == "meta" else w,
                                                                 quant_type="nf4"))


def _args(**kw):
    base = dict(dim=256, n_layers=2, n_heads=2, n_kv_heads=1, vocab_size=512, hidden_dim=512, max_seq_len=32, max_batch=1)
    base.update(kw)
    return LlamaArgs(**base)


def test_stream_into_meta_module_equals_loading_the_whole_state_dict_cpu(cpu_backend):
    args = _args()
    ex = get_nf4_executor()
    real = LlamaDecoder(args).to(torch.bfloat16).eval().requires_grad_(False)
    with torch.no_grad():
        for n, t in seeded_tensors(real, 5, device="cpu"):
            real.get_parameter(n).copy_(t)
    real.reset_rope_tables()
    j_real = thunder.jit(real, transforms=[NF4LinearQuant4bit()], executors=(ex,))
    with torch.device("meta"):
        meta = LlamaDecoder(args).to(torch.bfloat16).eval().requires_grad_(False)
    stats = {}
    seen = []

    def stream():
        for n, t in seeded_tensors(meta, 5, device="cpu"):
            seen.append(n)
            yield n, t

    j_meta = thunder.jit(meta, executors=(ex,),
                         transforms=[NF4LinearQuant4bit(), MaterializationTransform("cpu", init=init_from_tensor_stream(stream(), stats))])
    sd_real, sd_meta = j_real.state_dict(), j_meta.state_dict()
    assert list(sd_real) == list(sd_meta)
    for k in sd_real:
        assert torch.equal(sd_real[k], sd_meta[k]), k
    assert stats["tensors"] == len(seen) == len(list(real.named_parameters()))
    # one submodule's tensors at a time: never more than the largest single tensor is held
    largest = max(p.numel() * p.element_size() for p in real.parameters())
    assert stats["max_pending_bytes"] == largest
    tok, pos = torch.randint(0, args.vocab_size, (1, 3)), torch.arange(3)
    assert torch.equal(j_real(tok, pos), j_meta(tok, pos))
    # rotary tables and caches (not in the checkpoint) were initialised by the modules themselves
    assert torch.equal(j_meta.get_buffer("freqs_cos"), real.freqs_cos)
    assert j_meta.get_buffer("layers.0.attention.k_cache").shape == real.layers[0].attention.k_cache.shape


def test_stream_errors_cpu(cpu_backend):
    args = _args(n_layers=1)
    m = LlamaDecoder(args).to(torch.bfloat16).eval().requires_grad_(False)
    jm = thunder.jit(m, transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))
    with pytest.raises(KeyError, match="no entry"):
        stream_load(jm, [("layers.0.nope.weight", torch.zeros(1))])
    some = list(seeded_tensors(m, 1, device="cpu"))[:3]
    with pytest.raises(KeyError, match="never arrived"):
        stream_load(jm, some)


@pytest.mark.gpu
def test_peak_device_memory_is_the_quantized_model_plus_one_tensor():
    """Two layers of the 70B shape (d 8192, 64/8 heads, ffn 28672): 3.4 GB in bf16, 0.96 GB quantized.  Streamed
    from the seeded generator into a meta-device module, the device never holds more than the quantized
    model, the caches, and about one 16-bit tensor (plus the generator's fp32 chunks)."""
    args = LlamaArgs(dim=8192, n_layers=2, n_heads=64, n_kv_heads=8, vocab_size=8192, hidden_dim=28672, max_seq_len=64, max_batch=1)
    with torch.device("meta"):
        meta = LlamaDecoder(args).to(torch.bfloat16).eval().requires_grad_(False)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    stats = {}
    jm = thunder.jit(meta, executors=(get_nf4_executor(),),
                     transforms=[NF4LinearQuant4bit(), MaterializationTransform("cuda", init=init_from_tensor_stream(seeded_tensors(meta, 1), stats))])
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    held = torch.cuda.memory_allocated() - base
    n_w = sum(p.numel() for n, p in meta.named_parameters() if p.dim() == 2 and "tok_embeddings" not in n)
    quantized = n_w // 2 + n_w // 16
    bf16_model = sum(p.numel() * 2 for p in meta.parameters())
    largest = 28672 * 8192
    assert held < quantized + 2 * args.vocab_size * args.dim + 64 * 2 ** 20          # packed + absmax + embedding + buffers
    assert peak < held + largest * 2 + 3 * (1 << 25) * 4 + 64 * 2 ** 20               # + one bf16 tensor and the generator's fp32 chunks
    assert peak < bf16_model / 2
    assert stats["max_pending_bytes"] == largest * 2
    # and it decodes
    y = jm(torch.randint(0, args.vocab_size, (1, 1), device="cuda"), torch.tensor([0], device="cuda"))
    assert y.shape == (1, 1, args.vocab_size) and torch.isfinite(y.float()).all()
    assert jm.get_parameter("layers.1.feed_forward.w1.weight").dtype == torch.uint8
