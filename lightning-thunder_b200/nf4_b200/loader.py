"""Streaming quantize-on-load: an unquantized checkpoint goes into a jitted, NF4-transformed module one
tensor at a time, so neither the device nor the host ever holds the model in 16 bits.

The reference already loads submodule by submodule: `ThunderModule.load_original_state_dict`
(thunder/core/module.py:137-190) runs every transform's `transform_state_dict_for_submodule` on one
submodule's entries and copies the result into the module's (address-stable) parameters, and
`MaterializationTransform.init_from_original_state_dict` (thunder/transforms/materialization.py:151-159)
uses it to fill a meta-device module.  Both take a complete state dict, though.  `stream_load` feeds the same
per-submodule hook from an ITERATOR of (name, tensor) pairs -- a lazily read checkpoint file, or the seeded
generator below -- and drops each tensor as soon as its submodule is loaded;
`init_from_tensor_stream` is the matching `init=` callable for `MaterializationTransform`:

    with torch.device("meta"):
        model = LlamaDecoder(args).to(torch.bfloat16)
    jm = thunder.jit(model, executors=[get_nf4_executor()],
                     transforms=[NF4LinearQuant4bit(),
                                 MaterializationTransform("cuda", init=init_from_tensor_stream(seeded_tensors(model, 1)))])

Peak device memory: the quantized model + the largest single 16-bit tensor (+ what the module's buffers need).
"""

from __future__ import annotations

from collections.abc import Iterable, Iterator

import torch


def _direct_entries(module: torch.nn.Module) -> set[str]:
    """Names of a module's own parameters and persistent buffers (what a state dict holds for it)."""
    names = {n for n, p in module.named_parameters(recurse=False) if p is not None}
    names |= {n for n, b in module.named_buffers(recurse=False) if b is not None and n not in module._non_persistent_buffers_set}
    return names


def stream_load(jm, tensors: Iterable[tuple[str, torch.Tensor]]) -> dict:
    """Loads original (untransformed) tensors into the ThunderModule `jm` as they arrive.  A submodule is
    transformed and copied in as soon as all of its own entries have been seen; its tensors are released right
    after.  Returns {"tensors": count, "bytes": total source bytes, "max_pending_bytes": most source bytes held
    at once}.  Raises KeyError for a name the module does not have and for entries that never arrived."""
    modules = dict(jm._model.named_modules())
    want = {name: _direct_entries(m) for name, m in modules.items()}
    shared = jm._get_shared_names()
    processed: set[str] = set()
    pending: dict[str, dict[str, torch.Tensor]] = {}
    done: set[str] = set()
    stats = {"tensors": 0, "bytes": 0, "max_pending_bytes": 0}
    held = 0
    for name, t in tensors:
        mod, _, leaf = name.rpartition(".")
        if mod not in want or leaf not in want[mod]:
            raise KeyError(f"stream_load: the module has no entry {name!r}")
        if mod in done:
            raise KeyError(f"stream_load: {name!r} arrived after its submodule had been loaded")
        part = pending.setdefault(mod, {})
        part[leaf] = t
        nbytes = t.numel() * t.element_size()
        held += nbytes
        stats["tensors"] += 1
        stats["bytes"] += nbytes
        stats["max_pending_bytes"] = max(stats["max_pending_bytes"], held)
        if set(part) == want[mod]:
            jm._transform_and_load_for_submodule(mod, part, shared, processed)
            held -= sum(v.numel() * v.element_size() for v in part.values())
            del pending[mod], part
            done.add(mod)
        del t
    # tied entries may legitimately be absent (their twin was loaded); everything else must have arrived
    missing = []
    for mod, names in want.items():
        if mod in done or not names:
            continue
        for leaf in names - set(pending.get(mod, {})):
            full = f"{mod}.{leaf}" if mod else leaf
            if not (shared.get(full, {full}) & processed):
                missing.append(full)
        if mod in pending and not [m for m in missing if m.startswith(mod)]:
            jm._transform_and_load_for_submodule(mod, pending.pop(mod), shared, processed)
    if missing:
        raise KeyError(f"stream_load: entries never arrived: {sorted(missing)[:8]}{' ...' if len(missing) > 8 else ''}")
    return stats


def init_from_tensor_stream(tensors: Iterable[tuple[str, torch.Tensor]], stats_out: dict | None = None):
    """`init=` callable for thunder.transforms.MaterializationTransform: non-persistent buffers come from the
    modules' own `reset_parameters`, everything else from the stream (quantized on the way in)."""
    from thunder.transforms.materialization import module_init_from_original_module_init

    def init(transform, model):
        module_init_from_original_module_init(transform, model, non_persistent_only=True)
        stats = stream_load(model, tensors)
        if stats_out is not None:
            stats_out.update(stats)

    return init


def seeded_tensors(model: torch.nn.Module, seed: int, *, device="cuda", std: float = 0.02) -> Iterator[tuple[str, torch.Tensor]]:
    """The random-init checkpoint of the benchmark configurations as a stream: N(0, std) for every matrix
    (one generator per tensor, seeded from `seed` and the tensor's position), ones for the norm weights.
    Tensors are produced on `device` in the parameter's dtype, one at a time, in module order; `model` may
    live on the meta device (only names, shapes and dtypes are read)."""
    chunk_elems = 1 << 25          # fp32 draws are made 32 Mi elements at a time, so a tensor costs ~its own size
    for i, (name, p) in enumerate(model.named_parameters()):
        if p.dim() < 2:
            yield name, torch.ones(p.shape, dtype=p.dtype, device=device)
            continue
        g = torch.Generator(device=device).manual_seed(seed * 1000003 + i)
        out = torch.empty(p.shape, dtype=p.dtype, device=device)
        rows = max(1, chunk_elems // max(1, p[0].numel()))
        for r0 in range(0, p.shape[0], rows):
            part = out[r0:r0 + rows]
            part.copy_(torch.randn(part.shape, generator=g, device=device, dtype=torch.float32).mul_(std))
        yield name, out
        del out, part            # the consumer's reference is the only one left: freed before the next tensor is drawn
