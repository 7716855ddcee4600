"""The NF4 decode path through Thunder's own API: `compile_decoder(model)` is
`thunder.jit(model, transforms=[...], executors=[...])` with the transform stack a serving loop wants,
and `generate` is the prefill + token-by-token loop of the reference's inference benchmark
(thunder/benchmarks/benchmark_inference.py:440-529: the whole prompt in one call, then one call per
token with the sampled id fed back).

Transform stack, in order:
  NF4LinearQuant4bit      every nn.Linear -> NF4 weights + the `nf4_b200_matmul` symbol   (the drop-in for
                          thunder.transforms.quantization.BitsAndBytesLinearQuant4bit)
  NF4DecodeFusion         single-token traces: attention / MLP blocks -> fused kernels     (nf4_b200.fusion)
  PinModuleMembers        untouched parameters / buffers become overrides of themselves: the prologue's per-call
                          fetch of every member is a dictionary hit
  PrunePrologueChecks     drops the per-call re-validation of module members               (thunder/transforms/
                          prune_prologue_checks.py, what thunder/recipes/base.py:103-112 installs)
  CUDAGraphTransform      the computation replays as one CUDA graph                        (thunder/transforms/
                          cudagraph.py:229-387, what the reduce-overhead plugin installs; subclassed here only
                          to make the per-call graph lookup cheaper, see _graph_transform)
"""

from __future__ import annotations

import torch
from torch import nn

from .fusion import NF4DecodeFusion
from .thunder_executor import NF4LinearQuant4bit, get_nf4_executor, thunder

from thunder.core.transform_common import Transform  # noqa: E402


def _graph_transform():
    """thunder.transforms.cudagraph.CUDAGraphTransform with a cheaper per-call path for modules with hundreds
    of parameters.  The stock runner (cudagraph.py:137-163) describes dtype, size and stride of EVERY argument on
    every call to find its graph; here only the arguments that are not static memory (the call's real inputs)
    are described -- parameters and buffers cannot change their metadata without a new trace -- and a static
    argument is only compared by identity (a replaced tensor is still copied into the captured one, as upstream)."""
    from thunder.transforms.cudagraph import CUDAGraphRunner, CUDAGraphTransform, to_arg_descriptor

    class Runner(CUDAGraphRunner):
        def make_cache_key(self, fn_name, *args):
            mask = self.make_static_inputs_mask(fn_name, *args)
            return (fn_name, len(args), to_arg_descriptor(*[a for a, m in zip(args, mask) if not m]))

        def call_cuda_graph(self, fn_name, *args):
            fn, _ = self.python_callables[fn_name]
            key = self.make_cache_key(fn_name, *args)
            entry = self.cuda_graph_cache.get(key)
            if entry is None:
                entry = self.build_cuda_graph(fn, args, self.make_static_inputs_mask(fn_name, *args))
                self.cuda_graph_cache[key] = entry
            graph, static_inputs, static_outputs = entry
            for static_input, arg in zip(static_inputs, args):
                if static_input is not arg and isinstance(static_input, torch.Tensor) and isinstance(arg, torch.Tensor):
                    static_input.copy_(arg)
            graph.replay()
            return static_outputs

    class _Transform(CUDAGraphTransform):
        def __init__(self, *, share_mem_pool: bool = False):
            super().__init__(share_mem_pool=share_mem_pool)
            self.cuda_graph_runner = Runner(share_mem_pool=share_mem_pool)

    return _Transform()


class PinModuleMembers(Transform):
    """Registers every parameter and buffer that the earlier transforms left alone as an override of itself
    (`ThunderModule._overrides_parameters` / `_overrides_buffers`, the mechanism of thunder/core/module.py:58-72).
    The prologue fetches each member on every call; an override is a dictionary hit, anything else goes through
    torch's `get_parameter` / `get_buffer`, which walk the dotted path module by module -- about 130 such walks
    per decode step for a 32-layer model (norm weights, KV caches, rotary tables).  Values are the same tensor
    objects, so in-place updates (the KV cache, `load_state_dict`) stay visible; place it after the transforms
    that replace members."""

    def transform_module(self, model) -> None:
        inner = model._model
        for name, p in inner.named_parameters(remove_duplicate=False):
            if p.device.type != "meta":
                model._overrides_parameters.setdefault(name, p)
        for name, b in inner.named_buffers(remove_duplicate=False):
            if b.device.type != "meta":
                model._overrides_buffers.setdefault(name, b)


class GreedyStep(nn.Module):
    """model(tokens, input_pos) followed by argmax over the vocabulary: returns the next token ids
    [B, 1] (int64), so a decode loop never brings logits to the host."""

    def __init__(self, model: nn.Module):
        super().__init__()
        self.model = model

    def forward(self, tokens: torch.Tensor, input_pos: torch.Tensor) -> torch.Tensor:
        logits = self.model(tokens, input_pos)
        return torch.argmax(logits[:, -1, :], dim=-1, keepdim=True)


def compile_decoder(model: nn.Module, *, fuse: bool = True, cuda_graph: bool = True, prune_checks: bool = True,
                    rope_theta: float | None = None, extra_transforms=(), **jit_kwargs):
    """thunder.jit of `model` on the NF4 executor.  Returns the ThunderModule; `.nf4_fusion` is the
    fusion pass (its `fused` / `declined` records say what was rewritten)."""
    from thunder.transforms.prune_prologue_checks import PrunePrologueChecks

    transforms = [NF4LinearQuant4bit()]
    fusion = None
    if fuse:
        if rope_theta is None:
            inner = getattr(model, "model", model)
            rope_theta = getattr(getattr(inner, "args", None), "rope_theta", None)
        fusion = NF4DecodeFusion(rope_theta=rope_theta)
        transforms.append(fusion)
    transforms += list(extra_transforms)
    if prune_checks:
        transforms.append(PinModuleMembers())
        transforms.append(PrunePrologueChecks())
    if cuda_graph:
        transforms.append(_graph_transform())
    jm = thunder.jit(model, transforms=transforms, executors=(get_nf4_executor(),), **jit_kwargs)
    jm.nf4_fusion = fusion
    return jm


@torch.no_grad()
def generate(jstep, prompt: torch.Tensor, n_new: int) -> torch.Tensor:
    """Greedy decoding with a jitted GreedyStep: one call for the prompt [B, T] (prefill), then one call
    per new token with the previous ids fed back on the device.  Returns [B, n_new] int64 (device)."""
    B, T = prompt.shape
    dev = prompt.device
    out = torch.empty((B, n_new), dtype=torch.int64, device=dev)
    tok = jstep(prompt, torch.arange(T, device=dev))
    out[:, :1] = tok
    pos = torch.tensor([T], device=dev)
    for t in range(1, n_new):
        tok = jstep(tok.clone(), pos)
        out[:, t:t + 1] = tok
        pos = pos + 1
    return out
