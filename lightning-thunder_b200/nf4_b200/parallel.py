"""Tensor-parallel sharding arithmetic of the NF4 decoder (device-agnostic; the decode engine and the
CPU multi-process tests share it).

Column-parallel projections (Q, K, V, gate, up, output head) are split by rows of the row-major weight,
row-parallel ones (attention output, down) by columns, in contiguous chunks of size dim/tp indexed by
rank -- the chunking of thunder/distributed/__init__.py:535-546 (`narrow(dim, chunk * rank, chunk)`).
Each rank quantizes only its shard; K/tp stays a multiple of the 64-element quantization block, so no
block straddles two ranks and the shard's codes equal the corresponding codes of the full matrix.
Partial outputs of a row-parallel projection meet in one all-reduce (sum), as in
thunder/distributed/tensor_parallel/row_wise.py:53-80.
"""

from __future__ import annotations

import torch

BLOCK = 64


def check_shardable(n_heads: int, n_kv_heads: int, head_dim: int, ffn: int, vocab: int, tp: int) -> None:
    """Raises ValueError unless every projection splits evenly and no quantization block straddles ranks."""
    if tp < 1:
        raise ValueError(f"tp={tp}")
    if n_heads % tp or n_kv_heads % tp:
        raise ValueError(f"heads ({n_heads} query, {n_kv_heads} key/value) do not divide by tp={tp}")
    if ffn % (BLOCK * tp):
        raise ValueError(f"ffn={ffn}: ffn/tp must be a multiple of the {BLOCK}-element quantization block")
    if (n_heads // tp * head_dim) % BLOCK:
        raise ValueError("the attention-output shard's K must be a multiple of the quantization block")
    if vocab % tp:
        raise ValueError(f"vocab={vocab} does not divide by tp={tp}")


def shard_rows(w: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """Column-parallel: rows [rank * N/tp, (rank + 1) * N/tp) of w [N, K]."""
    chunk = w.shape[0] // tp
    return w.narrow(0, chunk * rank, chunk)


def shard_cols(w: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """Row-parallel: columns [rank * K/tp, (rank + 1) * K/tp) of w [N, K], contiguous."""
    chunk = w.shape[1] // tp
    if chunk % BLOCK:
        raise ValueError(f"K/tp = {chunk} is not a multiple of {BLOCK}: a quantization block would straddle ranks")
    return w.narrow(1, chunk * rank, chunk).contiguous()


def shard_qkv(wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """This rank's heads of Q, K and V stacked into one matrix (rows of whole heads, so the bytes of a
    separate quantization of the three shards and of the stack are the same)."""
    return torch.cat([shard_rows(wq, rank, tp), shard_rows(wk, rank, tp), shard_rows(wv, rank, tp)], dim=0)


def shard_gate_up(wg: torch.Tensor, wu: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """This rank's gate and up rows interleaved (gate_0, up_0, gate_1, up_1, ...), the layout the SwiGLU
    epilogue of the linear kernels reads."""
    g, u = shard_rows(wg, rank, tp), shard_rows(wu, rank, tp)
    return torch.stack([g, u], dim=1).reshape(2 * g.shape[0], g.shape[1])


def local_candidates(logits: torch.Tensor, local_ids: torch.Tensor, rank: int, vocab_per_rank: int) -> torch.Tensor:
    """[B, 2] fp32: (best local logit, its GLOBAL token id) of a rank that owns a vocabulary slice."""
    cand = torch.empty((logits.shape[0], 2), dtype=torch.float32, device=logits.device)
    cand[:, 0] = logits.gather(1, local_ids.view(-1, 1)).view(-1).float()
    cand[:, 1] = (local_ids + rank * vocab_per_rank).float()
    return cand


def merge_candidates(cand_all: torch.Tensor) -> torch.Tensor:
    """cand_all [tp, B, 2] gathered from all ranks -> [B] int64 winning token ids; on equal logits the
    lowest rank (= lowest token id range) wins, which is what a single argmax over the full vocabulary gives."""
    best = cand_all[:, :, 0].argmax(dim=0)
    return cand_all[:, :, 1].gather(0, best.view(1, -1)).view(-1).long()
