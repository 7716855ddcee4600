"""Shared helpers of the tests: seeded synthetic inputs and torch<->numpy bit views."""

import hashlib

import numpy as np
import torch


def seeded_weight(shape, seed, std=0.02, dtype=torch.bfloat16):
    """W ~ N(0, std) drawn on the CPU generator from `seed`, rounded to dtype."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(dtype)


def seeded_act(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.bfloat16
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(torch.bfloat16)


def sha256(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# ---------------------------------------------------------------------------------------------------
# CPU checkers of the decode-step kernels (test-only stand-ins with the same signatures as
# nf4_b200.functional.gemv_decode / attn_decode_fused / silu_mul): the quantized product comes from the
# oracle, the glue is plain torch in fp32 with bf16 roundings where the kernels round.
# ---------------------------------------------------------------------------------------------------

def _bf(t):
    return t.to(torch.bfloat16).float()


def cpu_gemv_decode(x, packed, absmax, code, N, K, *, prologue=0, norm_w=None, eps=0.0, epilogue=0, residual=None, out=None,
                    pdl=False, next_weight=None):
    import oracle

    in_cols = 2 * K if prologue == 2 else K
    x2 = x.detach().reshape(-1, in_cols).float().cpu()
    if prologue == 1:
        x2 = _bf(x2 * torch.rsqrt((x2 * x2).mean(-1, keepdim=True) + eps) * norm_w.float().cpu())
    elif prologue == 2:
        g, u = x2[:, :K], x2[:, K:]
        x2 = _bf(g / (1.0 + torch.exp(-g)) * u)
    y = oracle.linear_bf16(bf16_bits(x2.to(torch.bfloat16)), packed.cpu().numpy().reshape(-1), absmax.cpu().numpy(),
                           code.cpu().numpy(), N, K, 64, None, mode=oracle.GEMV_MODE)
    y = bits_to_bf16(y).float()
    if epilogue == 1:
        g, u = y[:, 0::2], y[:, 1::2]
        y = g / (1.0 + torch.exp(-g)) * u
    elif epilogue == 2:
        g, u = y[:, : N // 2], y[:, N // 2:]
        y = g / (1.0 + torch.exp(-g)) * u
    elif residual is not None:
        # the kernel adds the residual to the fp32 sum and rounds once; y here was rounded first, which
        # stays inside the tolerance the fused and unfused forms are compared at
        y = y + residual.detach().reshape(y.shape).float().cpu()
    n_out = N // 2 if epilogue else N
    return y.to(torch.bfloat16).reshape(*x.shape[:-1], n_out).to(x.device)


def cpu_silu_mul(gate_up, F, interleaved):
    g2 = gate_up.detach().reshape(-1, 2 * F).float()
    g, u = (g2[:, 0::2], g2[:, 1::2]) if interleaved else (g2[:, :F], g2[:, F:])
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype).reshape(*gate_up.shape[:-1], F)


def cpu_attn_decode_fused(qkv, positions, k_cache, v_cache, Hq, Hkv, theta, *, pdl=False, out=None):
    B, Dh = qkv.shape[0], 128
    q = qkv[:, : Hq * Dh].float().view(B, Hq, Dh)
    k = qkv[:, Hq * Dh: (Hq + Hkv) * Dh].float().view(B, Hkv, Dh)
    v = qkv[:, (Hq + Hkv) * Dh:].view(B, Hkv, Dh)
    i = torch.arange(Dh // 2, dtype=torch.float32)
    ang = positions.float().view(B, 1, 1) * torch.pow(torch.tensor(float(theta)), -2.0 * i / Dh).view(1, 1, -1)
    c, s = torch.cos(ang), torch.sin(ang)

    def rot(t):
        tr = t.view(*t.shape[:-1], Dh // 2, 2)
        return _bf(torch.stack([tr[..., 0] * c - tr[..., 1] * s, tr[..., 0] * s + tr[..., 1] * c], dim=-1).flatten(-2))

    q, k = rot(q), rot(k)
    res = torch.empty((B, Hq * Dh), dtype=torch.float32)
    rep = Hq // Hkv
    for b in range(B):
        p = int(positions[b])
        k_cache[b, :, p] = k[b].to(k_cache.dtype)
        v_cache[b, :, p] = v[b]
        kk = k_cache[b, :, : p + 1].float().repeat_interleave(rep, dim=0)      # [Hq, L, Dh]
        vv = v_cache[b, :, : p + 1].float().repeat_interleave(rep, dim=0)
        sc = torch.einsum("hd,hld->hl", q[b], kk) / (Dh ** 0.5)
        res[b] = torch.einsum("hl,hld->hd", torch.softmax(sc, dim=-1), vv).reshape(-1)
    return res.to(qkv.dtype)


def cpu_rms_norm_rows(x, weight, eps):
    xf = x.detach().float()
    return (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def cpu_rope_prefill(qkv, positions, k_cache, v_cache, Hq, Hkv, theta):
    """qkv [B, T, (Hq+2*Hkv)*Dh] -> rotated q [B, Hq, T, Dh]; rotated k and v written to cache rows positions[t]."""
    B, T, Dh = qkv.shape[0], qkv.shape[1], k_cache.shape[-1]
    parts = qkv.float().view(B, T, Hq + 2 * Hkv, Dh)
    i = torch.arange(Dh // 2, dtype=torch.float32)
    ang = positions.float().view(1, T, 1, 1) * torch.pow(torch.tensor(float(theta)), -2.0 * i / Dh).view(1, 1, 1, -1)
    c, s = torch.cos(ang), torch.sin(ang)

    def rot(t):
        tr = t.reshape(*t.shape[:-1], Dh // 2, 2)
        return _bf(torch.stack([tr[..., 0] * c - tr[..., 1] * s, tr[..., 0] * s + tr[..., 1] * c], dim=-1).flatten(-2))

    q, k, v = rot(parts[:, :, :Hq]), rot(parts[:, :, Hq:Hq + Hkv]), parts[:, :, Hq + Hkv:]
    idx = positions.long()
    k_cache[:, :, idx] = k.transpose(1, 2).to(k_cache.dtype)
    v_cache[:, :, idx] = v.transpose(1, 2).to(v_cache.dtype)
    return q.transpose(1, 2).contiguous().to(qkv.dtype)
