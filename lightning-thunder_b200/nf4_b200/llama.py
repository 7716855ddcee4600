"""A Llama-shaped decoder as a plain torch.nn.Module with its KV cache held in buffers -- the model
the benchmark configurations describe (RMSNorm, rotary embedding on interleaved pairs, grouped-query
attention, SwiGLU MLP, untied output head), written after the reference's in-repo definition
(thunder/tests/llama2_model.py:129-290: same submodule names `attention.wq/wk/wv/wo`,
`feed_forward.w1/w2/w3`, `attention_norm`, `ffn_norm`, `tok_embeddings`, `norm`, `output`) and
extended by what decoding needs: `forward(tokens, input_pos)` writes the new keys and values into
the cache at `input_pos` and attends over the cache under a position mask, so one module serves
prefill (T tokens at positions 0..T-1) and decode (one token at position p).

Nothing here knows about quantization: `thunder.jit(model, transforms=[NF4LinearQuant4bit(), ...])`
replaces every nn.Linear by the NF4 kernels exactly as it does for the reference's own models.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class LlamaArgs:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    vocab_size: int = 128256
    hidden_dim: int = 14336
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq_len: int = 1024
    max_batch: int = 1


def llama3_8b_args(**kw) -> LlamaArgs:
    return LlamaArgs(**kw)


def llama3_70b_args(**kw) -> LlamaArgs:
    return LlamaArgs(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, hidden_dim=28672, **kw)


class RMSNorm(nn.Module):
    """x * rsqrt(mean(x^2) + eps) * weight, computed in fp32 and rounded once to x's type
    (thunder/tests/llama2_model.py:25-37 rounds the normalised value before the weight multiply; the
    single rounding here is what torch.nn.functional.rms_norm does)."""

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.dim = dim
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return F.rms_norm(x, (self.dim,), self.weight, self.eps)


def rope_tables(head_dim: int, end: int, theta: float):
    """cos / sin of position * theta^(-2i/head_dim), fp32 [end, head_dim/2] (llama2_model.py:40-47)."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    ang = torch.outer(torch.arange(end).float(), freqs)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotates the (2i, 2i+1) pairs of x [B, T, H, Dh] by the angles of cos/sin [T, Dh/2]
    (llama2_model.py:58-82)."""
    B, T, H, Dh = x.shape
    xf = x.float().reshape(B, T, H, Dh // 2, 2)
    xr, xi = xf[..., 0], xf[..., 1]
    c = cos.view(1, T, 1, Dh // 2)
    s = sin.view(1, T, 1, Dh // 2)
    out = torch.stack([xr * c - xi * s, xr * s + xi * c], dim=-1).flatten(3)
    return out.type_as(x)


class Attention(nn.Module):
    def __init__(self, args: LlamaArgs):
        super().__init__()
        self.n_heads = args.n_heads
        self.n_kv_heads = args.n_kv_heads
        self.n_rep = args.n_heads // args.n_kv_heads
        self.head_dim = args.dim // args.n_heads
        self.wq = nn.Linear(args.dim, args.n_heads * self.head_dim, bias=False)
        self.wk = nn.Linear(args.dim, args.n_kv_heads * self.head_dim, bias=False)
        self.wv = nn.Linear(args.dim, args.n_kv_heads * self.head_dim, bias=False)
        self.wo = nn.Linear(args.n_heads * self.head_dim, args.dim, bias=False)
        shape = (args.max_batch, args.n_kv_heads, args.max_seq_len, self.head_dim)
        self.register_buffer("k_cache", torch.zeros(shape), persistent=False)
        self.register_buffer("v_cache", torch.zeros(shape), persistent=False)

    def reset_parameters(self) -> None:
        """(Re)initialises what the state dict does not carry: an empty cache."""
        self.k_cache.zero_()
        self.v_cache.zero_()

    def forward(self, x, cos, sin, input_pos, mask):
        B, T, _ = x.shape
        assert B == self.k_cache.shape[0], "the batch must fill the KV cache (max_batch)"
        q = self.wq(x).view(B, T, self.n_heads, self.head_dim)
        k = self.wk(x).view(B, T, self.n_kv_heads, self.head_dim)
        v = self.wv(x).view(B, T, self.n_kv_heads, self.head_dim)
        q = apply_rope(q, cos, sin)
        k = apply_rope(k, cos, sin)
        # the cache keeps [B, Hkv, S, Dh]; rows input_pos are (over)written, the rest is history
        keys = self.k_cache.index_copy_(2, input_pos, k.transpose(1, 2))
        values = self.v_cache.index_copy_(2, input_pos, v.transpose(1, 2))
        q = q.transpose(1, 2)
        if self.n_rep > 1:
            S = keys.shape[2]
            keys = keys[:, :, None, :, :].expand(B, self.n_kv_heads, self.n_rep, S, self.head_dim).reshape(
                B, self.n_heads, S, self.head_dim)
            values = values[:, :, None, :, :].expand(B, self.n_kv_heads, self.n_rep, S, self.head_dim).reshape(
                B, self.n_heads, S, self.head_dim)
        y = F.scaled_dot_product_attention(q, keys, values, attn_mask=mask, dropout_p=0.0, is_causal=False)
        y = y.transpose(1, 2).reshape(B, T, self.n_heads * self.head_dim)
        return self.wo(y)


class FeedForward(nn.Module):
    def __init__(self, args: LlamaArgs):
        super().__init__()
        self.w1 = nn.Linear(args.dim, args.hidden_dim, bias=False)
        self.w2 = nn.Linear(args.hidden_dim, args.dim, bias=False)
        self.w3 = nn.Linear(args.dim, args.hidden_dim, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))


class TransformerBlock(nn.Module):
    def __init__(self, layer_id: int, args: LlamaArgs):
        super().__init__()
        self.layer_id = layer_id
        self.attention = Attention(args)
        self.feed_forward = FeedForward(args)
        self.attention_norm = RMSNorm(args.dim, args.norm_eps)
        self.ffn_norm = RMSNorm(args.dim, args.norm_eps)

    def forward(self, x, cos, sin, input_pos, mask):
        h = x + self.attention(self.attention_norm(x), cos, sin, input_pos, mask)
        return h + self.feed_forward(self.ffn_norm(h))


class LlamaDecoder(nn.Module):
    def __init__(self, args: LlamaArgs):
        super().__init__()
        self.args = args
        self.tok_embeddings = nn.Embedding(args.vocab_size, args.dim)
        self.layers = nn.ModuleList(TransformerBlock(i, args) for i in range(args.n_layers))
        self.norm = RMSNorm(args.dim, args.norm_eps)
        self.output = nn.Linear(args.dim, args.vocab_size, bias=False)
        cos, sin = rope_tables(args.dim // args.n_heads, args.max_seq_len, args.rope_theta)
        self.register_buffer("freqs_cos", cos, persistent=False)
        self.register_buffer("freqs_sin", sin, persistent=False)

    def forward(self, tokens: torch.Tensor, input_pos: torch.Tensor) -> torch.Tensor:
        """tokens [B, T] int64, input_pos [T] int64 (the cache rows these tokens occupy).  Returns the
        logits of the last token, [B, 1, vocab]."""
        S = self.args.max_seq_len
        h = self.tok_embeddings(tokens)
        cos = self.freqs_cos[input_pos]
        sin = self.freqs_sin[input_pos]
        # query t sees cache rows 0..input_pos[t]
        mask = torch.arange(S, device=tokens.device)[None, :] <= input_pos[:, None]
        for layer in self.layers:
            h = layer(h, cos, sin, input_pos, mask)
        h = self.norm(h[:, -1:, :])
        return self.output(h)

    def _apply(self, fn, recurse=True):
        """`.to(dtype)` converts floating-point buffers too; the rotary tables stay fp32 whatever the model's type."""
        super()._apply(fn, recurse)
        if self.freqs_cos.dtype != torch.float32:
            dev = self.freqs_cos.device
            if dev.type == "meta":
                self.freqs_cos = torch.empty(self.freqs_cos.shape, dtype=torch.float32, device=dev)
                self.freqs_sin = torch.empty(self.freqs_sin.shape, dtype=torch.float32, device=dev)
            else:
                cos, sin = rope_tables(self.args.dim // self.args.n_heads, self.args.max_seq_len, self.args.rope_theta)
                self.freqs_cos, self.freqs_sin = cos.to(dev), sin.to(dev)
        return self

    def reset_parameters(self) -> None:
        """(Re)initialises what the state dict does not carry: the rotary tables."""
        cos, sin = rope_tables(self.args.dim // self.args.n_heads, self.args.max_seq_len, self.args.rope_theta)
        self.freqs_cos.copy_(cos)
        self.freqs_sin.copy_(sin)

    def reset_rope_tables(self) -> None:
        """Rebuilds the cos/sin tables in fp32 on the module's device (`.to(dtype)` rounds buffers too)."""
        cos, sin = rope_tables(self.args.dim // self.args.n_heads, self.args.max_seq_len, self.args.rope_theta)
        self.freqs_cos = cos.to(self.freqs_cos.device)
        self.freqs_sin = sin.to(self.freqs_sin.device)

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """Seeded N(0, std) for every Linear and the embedding (the benchmark configurations are
        random-init), one generator per tensor so a tensor's values do not depend on the others."""
        for i, (name, p) in enumerate(self.named_parameters()):
            if p.dim() < 2:
                continue
            g = torch.Generator(device=p.device).manual_seed(seed * 1000003 + i)
            p.copy_((torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32) * std).to(p.dtype))
