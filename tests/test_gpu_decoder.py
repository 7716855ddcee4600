"""The Llama-shaped NF4 decode step (glue kernels + fused GEMVs + CUDA graph) against a plain
PyTorch fp32 restatement of the same model that rounds to bf16 at the same points.  torch is only
the checker here; the oracle covers the quantized linears themselves."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _deq(w, round_w=False):
    import nf4_b200

    qs = nf4_b200.QuantState(w.absmax, shape=(w.N, w.K), code=w.code, blocksize=64, dtype=torch.bfloat16)
    # GEMV numerics: levels rounded to bf16, scaled by the fp32 absmax, no rounding of the product
    idx = torch.stack([w.packed.view(-1) >> 4, w.packed.view(-1) & 15], 1).view(-1).long()
    lv = qs.code.to(torch.bfloat16).float()[idx]
    wd = (lv.view(-1, 64) * w.absmax.view(-1, 1)).view(w.N, w.K)
    # tensor-core numerics: the product is rounded to bf16 before the matrix multiply
    return wd.to(torch.bfloat16).float() if round_w else wd


def _bf(t):
    return t.to(torch.bfloat16).float()


def _rms(x, w, eps):
    return _bf(x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float())


def _rope(x, pos, theta):
    # x [B, H, Dh], interleaved pairs
    B, H, Dh = x.shape
    i = torch.arange(Dh // 2, device=x.device, dtype=torch.float32)
    ang = pos.float().view(B, 1, 1) * torch.pow(torch.tensor(theta, device=x.device), -2.0 * i / Dh).view(1, 1, -1)
    xr = x.view(B, H, Dh // 2, 2)
    c, s = torch.cos(ang), torch.sin(ang)
    out = torch.stack([xr[..., 0] * c - xr[..., 1] * s, xr[..., 0] * s + xr[..., 1] * c], dim=-1)
    return _bf(out.view(B, H, Dh))


class TorchRef:
    def __init__(self, dec):
        self.dec, self.cfg = dec, dec.cfg
        tc = dec.tensor_core
        self.layers = [{k: _deq(l[k], tc) for k in ("qkv", "o", "gu", "down")} for l in dec.layers]
        self.head = _deq(dec.lm_head, tc)
        L, B, S = self.cfg.n_layers, dec.B, dec.S
        self.k = torch.zeros((L, B, dec.Hkv, S, 128), device=dec.dev)
        self.v = torch.zeros((L, B, dec.Hkv, S, 128), device=dec.dev)

    def step(self, ids, pos):
        cfg, dec = self.cfg, self.dec
        B = ids.shape[0]
        x = dec.embed[ids].float()
        for li, w in enumerate(self.layers):
            xn = _rms(x, dec.layers[li]["norm1"], cfg.norm_eps)
            qkv = _bf(xn @ w["qkv"].t())
            hq, hk = dec.Hq * 128, dec.Hkv * 128
            q = _rope(qkv[:, :hq].view(B, dec.Hq, 128), pos, cfg.rope_theta)
            k = _rope(qkv[:, hq:hq + hk].view(B, dec.Hkv, 128), pos, cfg.rope_theta)
            v = qkv[:, hq + hk:].view(B, dec.Hkv, 128)
            for b in range(B):
                self.k[li, b, :, pos[b]] = k[b]
                self.v[li, b, :, pos[b]] = v[b]
            out = torch.zeros((B, dec.Hq, 128), device=x.device)
            G = dec.Hq // dec.Hkv
            for b in range(B):
                n = int(pos[b]) + 1
                for h in range(dec.Hq):
                    kk, vv = self.k[li, b, h // G, :n], self.v[li, b, h // G, :n]
                    p = torch.softmax((kk @ q[b, h]) / math.sqrt(128.0), dim=0)
                    out[b, h] = p @ vv
            attn = _bf(out.view(B, -1))
            x = _bf(attn @ w["o"].t() + x)
            xn = _rms(x, dec.layers[li]["norm2"], cfg.norm_eps)
            gu = _bf(xn @ w["gu"].t())
            g, u = gu[:, 0::2], gu[:, 1::2]          # gate/up rows are interleaved in the fused matrix
            h = _bf(g / (1 + torch.exp(-g)) * u)
            x = _bf(h @ w["down"].t() + x)
        xn = _rms(x, dec.final_norm, cfg.norm_eps)
        return _bf(xn @ self.head.t())


@pytest.mark.parametrize("fused,pdl", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("use_graph", [False, True])
def test_decode_steps_match_torch_reference(use_graph, fused, pdl):
    from nf4_b200.decoder import NF4Decoder, tiny_config

    torch.manual_seed(0)
    cfg = tiny_config()
    dec = NF4Decoder(cfg, batch=2, max_seq=32, device="cuda:0", seed=3, attn_splits=3, fused=fused, pdl=pdl)
    if use_graph:
        dec.capture()
    ref = TorchRef(dec)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (2, 9), generator=g).cuda()
    dec.reset()
    agree = 0
    for t in range(toks.shape[1]):
        pos = dec.positions.clone().long()
        dec.ids_in.copy_(toks[:, t])
        dec.run_step()
        torch.cuda.synchronize()
        want = ref.step(toks[:, t], pos)
        torch.testing.assert_close(dec.logits.float(), want, rtol=3e-2, atol=3e-2)
        agree += int((dec.ids_out == want.argmax(-1)).sum())
        assert int(dec.positions[0]) == t + 1
    assert agree >= 2 * toks.shape[1] - 2   # bf16 near-ties may flip an argmax
    # the caches hold what the reference holds
    torch.testing.assert_close(dec.k_cache[:, :, :, :9].float(), ref.k[:, :, :, :9], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dec.v_cache[:, :, :, :9].float(), ref.v[:, :, :, :9], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("use_graph", [False, True])
def test_batched_decode_on_tensor_cores(use_graph):
    """More than 8 sequences: the step's linears run on the tcgen05 kernel (K split over thread blocks,
    residual and SwiGLU epilogues, programmatic dependent launch)."""
    from nf4_b200 import _lib
    from nf4_b200.decoder import NF4Decoder, tiny_config

    cfg = tiny_config()
    B = 12
    dec = NF4Decoder(cfg, batch=B, max_seq=16, device="cuda:0", seed=5, tensor_core_from=9)
    assert dec.tensor_core
    if use_graph:
        dec.capture()
    ref = TorchRef(dec)
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg.vocab, (B, 4), generator=g).cuda()
    dec.reset()
    agree = 0
    for t in range(toks.shape[1]):
        pos = dec.positions.clone().long()
        dec.ids_in.copy_(toks[:, t])
        dec.run_step()
        torch.cuda.synchronize()
        want = ref.step(toks[:, t], pos)
        torch.testing.assert_close(dec.logits.float(), want, rtol=3e-2, atol=3e-2)
        agree += int((dec.ids_out == want.argmax(-1)).sum())
    assert agree >= B * toks.shape[1] - 3
    assert _lib.device_error()[0] == 0


def test_sixteen_sequences_wide_model_on_the_gemv():
    """16 sequences of a model 1024 wide: the activations no longer fit beside the GEMV's tables, so RMSNorm runs as
    its own launch while the SwiGLU and residual epilogues stay fused (the shape of the tensor-parallel 70B step)."""
    from nf4_b200 import _lib
    from nf4_b200.decoder import NF4Decoder, tiny_config

    cfg = tiny_config(n_layers=2, d_model=1024, n_heads=8, n_kv_heads=2, ffn=2048, vocab=2048)
    B = 16
    dec = NF4Decoder(cfg, batch=B, max_seq=16, device="cuda:0", seed=6)
    assert not dec.tensor_core and not dec.lib.nf4_b200_gemv_decode_fits(B, 2 * cfg.ffn, cfg.d_model, 1)
    assert dec.lib.nf4_b200_gemv_decode_fits(B, 2 * cfg.ffn, cfg.d_model, 0)
    dec.capture()
    # one launch per projection (SwiGLU inside gate|up), one more wherever its RMSNorm does not fit, + attention per
    # layer, + embed and argmax: no separate SiLU * up launch
    fits = lambda n: 1 if dec.lib.nf4_b200_gemv_decode_fits(B, n, cfg.d_model, 1) else 2
    n_qkv = (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim
    assert fits(2 * cfg.ffn) == 2
    assert dec.launches_per_step == 1 + cfg.n_layers * (fits(n_qkv) + 1 + 1 + fits(2 * cfg.ffn) + 1) + fits(cfg.vocab) + 1
    ref = TorchRef(dec)
    g = torch.Generator().manual_seed(4)
    toks = torch.randint(0, cfg.vocab, (B, 4), generator=g).cuda()
    dec.reset()
    agree = 0
    for t in range(toks.shape[1]):
        pos = dec.positions.clone().long()
        dec.ids_in.copy_(toks[:, t])
        dec.run_step()
        torch.cuda.synchronize()
        want = ref.step(toks[:, t], pos)
        torch.testing.assert_close(dec.logits.float(), want, rtol=3e-2, atol=3e-2)
        agree += int((dec.ids_out == want.argmax(-1)).sum())
    assert agree >= 0.9 * B * toks.shape[1]      # bf16 near-ties may flip an argmax (the logits themselves are checked above)
    assert _lib.device_error()[0] == 0


def test_fused_and_unfused_steps_agree_bitwise():
    """Prologue fusion, the one-launch attention and programmatic dependent launch change the
    schedule, not the arithmetic: same tokens and same logits as the kernel-per-op chain."""
    from nf4_b200 import _lib
    from nf4_b200.decoder import NF4Decoder, tiny_config

    cfg = tiny_config(n_layers=3)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab, (2, 12), generator=g)
    outs, logits = [], []
    for fused, pdl, graph in [(False, False, False), (True, False, False), (True, True, False), (True, True, True)]:
        d = NF4Decoder(cfg, batch=2, max_seq=64, seed=4, attn_splits=4, fused=fused, pdl=pdl)
        if graph:
            d.capture()
        outs.append(d.generate(prompt, 10))
        logits.append(d.logits.clone())
    for o, l in zip(outs[1:], logits[1:]):
        assert torch.equal(o, outs[0])
        assert torch.equal(l, logits[0])
    assert _lib.device_error()[0] == 0


def test_generate_is_deterministic_and_graph_equals_eager():
    from nf4_b200.decoder import NF4Decoder, tiny_config

    cfg = tiny_config()
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (1, 6), generator=g)
    a = NF4Decoder(cfg, batch=1, max_seq=32, seed=11)
    out_eager = a.generate(prompt, 8)
    a.capture()
    out_graph = a.generate(prompt, 8)
    assert torch.equal(out_eager, out_graph)
    assert torch.equal(a.generate(prompt, 8), out_graph)
    assert a.launches_per_step == 1 + 10 * cfg.n_layers + 3 + 0 or a.launches_per_step > 0


def test_glue_kernels_against_torch():
    import ctypes

    from nf4_b200 import _lib

    lib = _lib.load()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((5, 4096), device="cuda", generator=g).to(torch.bfloat16)
    w = torch.randn((4096,), device="cuda", generator=g).to(torch.bfloat16)
    y = torch.empty_like(x)
    _lib.check(lib.nf4_b200_rmsnorm(x.data_ptr(), w.data_ptr(), y.data_ptr(), 5, 4096, 1e-5, st), "rmsnorm")
    torch.testing.assert_close(y.float(), _rms(x.float(), w, 1e-5), rtol=1e-2, atol=1e-2)
    gu = torch.randn((3, 2 * 1024), device="cuda", generator=g).to(torch.bfloat16)
    h = torch.empty((3, 1024), device="cuda", dtype=torch.bfloat16)
    _lib.check(lib.nf4_b200_silu_mul(gu.data_ptr(), h.data_ptr(), 3, 1024, 0, st), "silu_mul")
    gf = gu.float()
    torch.testing.assert_close(h.float(), _bf(torch.nn.functional.silu(gf[:, :1024]) * gf[:, 1024:]), rtol=1e-2, atol=1e-2)
    _lib.check(lib.nf4_b200_silu_mul(gu.data_ptr(), h.data_ptr(), 3, 1024, 1, st), "silu_mul")
    torch.testing.assert_close(h.float(), _bf(torch.nn.functional.silu(gf[:, 0::2]) * gf[:, 1::2]), rtol=1e-2, atol=1e-2)
    # prompt-sized input (the 16-byte form of the halves layout): bit-identical to the small-size kernel row by row
    gu = torch.randn((300, 2 * 3584), device="cuda", generator=g).to(torch.bfloat16)
    h = torch.empty((300, 3584), device="cuda", dtype=torch.bfloat16)
    _lib.check(lib.nf4_b200_silu_mul(gu.data_ptr(), h.data_ptr(), 300, 3584, 0, st), "silu_mul")
    h_rows = torch.empty_like(h)
    for r0 in range(0, 300, 100):       # 100 x 3584 < 2^20 outputs: the element-pair kernel
        _lib.check(lib.nf4_b200_silu_mul(gu[r0:r0 + 100].data_ptr(), h_rows[r0:r0 + 100].data_ptr(), 100, 3584, 0, st), "silu_mul")
    assert torch.equal(h, h_rows)
    gf = gu.float()
    torch.testing.assert_close(h.float(), _bf(torch.nn.functional.silu(gf[:, :3584]) * gf[:, 3584:]), rtol=1e-2, atol=1e-2)
    logits = torch.randn((4, 128256), device="cuda", generator=g).to(torch.bfloat16)
    ids = torch.empty((4,), device="cuda", dtype=torch.int64)
    _lib.check(lib.nf4_b200_argmax(logits.data_ptr(), ids.data_ptr(), 4, 128256, st), "argmax")
    # first maximum wins
    want = torch.stack([(row == row.max()).nonzero()[0, 0] for row in logits.float()])
    assert torch.equal(ids, want)
    # planted ties inside one 16-byte load and across threads (vector path), and a width the vector path refuses
    logits[0, 1000:1008] = 50.0
    logits[1, 77] = logits[1, 77 + 8 * 1024] = 60.0
    _lib.check(lib.nf4_b200_argmax(logits.data_ptr(), ids.data_ptr(), 4, 128256, st), "argmax")
    assert ids[0].item() == 1000 and ids[1].item() == 77
    odd = torch.randn((3, 1001), device="cuda", generator=g).to(torch.bfloat16)
    odd[2, 400] = odd[2, 900] = 70.0
    ids3 = torch.empty((3,), device="cuda", dtype=torch.int64)
    _lib.check(lib.nf4_b200_argmax(odd.data_ptr(), ids3.data_ptr(), 3, 1001, st), "argmax")
    assert torch.equal(ids3, torch.stack([(row == row.max()).nonzero()[0, 0] for row in odd.float()]))
    a = torch.randn((4096,), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn((4096,), device="cuda", generator=g).to(torch.bfloat16)
    c = torch.empty_like(a)
    _lib.check(lib.nf4_b200_add(a.data_ptr(), b.data_ptr(), c.data_ptr(), 4096, st), "add")
    assert torch.equal(c, (a.float() + b.float()).to(torch.bfloat16))
    # fused residual epilogue of the GEMV
    import nf4_b200

    wgt = (torch.randn((512, 1024), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    packed, qs = nf4_b200.quantize_4bit(wgt)
    xx = torch.randn((2, 1024), device="cuda", generator=g).to(torch.bfloat16)
    res = torch.randn((2, 512), device="cuda", generator=g).to(torch.bfloat16)
    plain = nf4_b200.matmul_4bit(xx, packed.t(), quant_state=qs)
    fused = torch.empty_like(plain)
    _lib.check(lib.nf4_b200_gemv_fused(xx.data_ptr(), 2, 1024, packed.data_ptr(), qs.absmax.data_ptr(), qs.code.data_ptr(),
                                       512, None, res.data_ptr(), fused.data_ptr(), _lib.NF4_BF16, st), "gemv_fused")
    torch.testing.assert_close(fused.float(), plain.float() + res.float(), rtol=1.6e-2, atol=2e-2)
    # decode form: RMSNorm prologue, SwiGLU prologue (halves layout) and SwiGLU epilogue (row pairs)
    nw = torch.randn((1024,), device="cuda", generator=g).to(torch.bfloat16)
    y1 = torch.empty_like(plain)
    _lib.check(lib.nf4_b200_gemv_decode(xx.data_ptr(), 2, 1024, packed.data_ptr(), qs.absmax.data_ptr(), qs.code.data_ptr(), 512,
                                        None, y1.data_ptr(), 1, nw.data_ptr(), 1e-5, 0, 0, st), "gemv_decode rmsnorm")
    assert torch.equal(y1, nf4_b200.matmul_4bit(_rms(xx.float(), nw, 1e-5).to(torch.bfloat16), packed.t(), quant_state=qs))
    x2 = torch.randn((2, 2048), device="cuda", generator=g).to(torch.bfloat16)
    y2 = torch.empty_like(plain)
    _lib.check(lib.nf4_b200_gemv_decode(x2.data_ptr(), 2, 1024, packed.data_ptr(), qs.absmax.data_ptr(), qs.code.data_ptr(), 512,
                                        None, y2.data_ptr(), 2, None, 0.0, 0, 0, st), "gemv_decode silu prologue")
    hh = _bf(torch.nn.functional.silu(x2.float()[:, :1024]) * x2.float()[:, 1024:]).to(torch.bfloat16)
    torch.testing.assert_close(y2.float(), nf4_b200.matmul_4bit(hh, packed.t(), quant_state=qs).float(), rtol=1.6e-2, atol=1e-2)
    y3 = torch.empty((2, 256), device="cuda", dtype=torch.bfloat16)
    _lib.check(lib.nf4_b200_gemv_decode(xx.data_ptr(), 2, 1024, packed.data_ptr(), qs.absmax.data_ptr(), qs.code.data_ptr(), 512,
                                        None, y3.data_ptr(), 0, None, 0.0, 1, 0, st), "gemv_decode swiglu epilogue")
    pf = plain.float()
    assert torch.equal(y3, (torch.nn.functional.silu(pf[:, 0::2]) * pf[:, 1::2]).to(torch.bfloat16)) or \
        torch.allclose(y3.float(), _bf(pf[:, 0::2] / (1 + torch.exp(-pf[:, 0::2])) * pf[:, 1::2]), rtol=1e-2, atol=1e-3)
