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
