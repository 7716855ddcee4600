"""Thunder side of the NF4 path: a `thunder.extend` operator executor whose one symbol runs the
sm_100a kernels, a `Transform` that quantizes every nn.Linear weight at jit time and replaces
`ltorch.linear` on those weights by that symbol, and a plugin.

Drop-in for thunder.transforms.quantization (get_bitsandbytes_executor / bnb_matmul_nf4 /
BitsAndBytesLinearQuant4bit, quantization.py:19-293) and thunder.plugins.quantization.QuantizeInt4
(plugins/quantization.py:4-37): same hook methods, same parameter names in the module and in
state dicts ("<w>", "<w>.absmax", "<w>.code"), same `quant_states` entries, same symbol signature
`(x, qweight, bias, absmax, quant_map, blocksize, dtype, shape)`, trace provenance "quant pass".

    import thunder
    from nf4_b200.thunder_executor import NF4LinearQuant4bit, get_nf4_executor
    jm = thunder.jit(model, transforms=[NF4LinearQuant4bit()], executors=(get_nf4_executor(),))

Two more routes to the same kernels:
  * `register_plugin()` re-binds the plugin name "quantize-int4" to `QuantizeNF4`;
  * `install_as_bitsandbytes()` exposes this package under the module name the reference imports,
    so the reference's own, unmodified transform drives these kernels.
"""

from __future__ import annotations

import sys
import types
from collections.abc import Sequence

import torch

from . import functional
from .thunder_support import bootstrap

thunder = bootstrap()

from thunder.core import prims  # noqa: E402
from thunder.core.proxies import ProxyTag  # noqa: E402
from thunder.core.trace import TraceProvenance, tracectx  # noqa: E402
from thunder.core.trace_interpreter import TraceSubstitutionProcessor  # noqa: E402
from thunder.core.transform_common import Transform  # noqa: E402
from thunder.transforms.utils import add_trace_output, get_checks, trace_with_replaced_proxy_metadata  # noqa: E402

EXECUTOR_NAME = "quant_nf4_b200"
_executor = None
nf4_matmul = None       # the Symbol, set by get_nf4_executor()
nf4_matmul_bwd = None   # its input gradient: g . dequant(W)


def get_nf4_executor():
    """Creates (once) the operator executor and its symbol `nf4_b200_matmul`."""
    global _executor, nf4_matmul, nf4_matmul_bwd
    if _executor is not None:
        return _executor
    ex = thunder.extend.OperatorExecutor(EXECUTOR_NAME, version=0.1)

    def nf4_matmul_meta(x, qweight, bias, absmax, quant_map, blocksize, dtype, shape):
        assert isinstance(shape, Sequence) and len(shape) == 2
        assert x.shape[-1] == shape[1], f"{x.shape=}, rhs {shape=}"
        return thunder.TensorProxy(like=x, shape=(*x.shape[:-1], shape[0]))

    def nf4_matmul_impl(x, qweight, bias, absmax, quant_map, blocksize, dtype, shape):
        # functional is looked up at call time so tests can substitute a checker on CPU
        return functional.linear_nf4(x, qweight, bias, absmax, quant_map, blocksize, shape)

    nf4_matmul = ex.register_operator("nf4_b200_matmul", meta=nf4_matmul_meta, fn=nf4_matmul_impl)

    # Input gradient.  The reference's symbol has no grad rule (training through bnb_matmul_nf4 is unsupported
    # there); the quantized weight stays frozen, which is what QLoRA needs: adapters added by
    # thunder.transforms.qlora.LORATransform train, gradients flow through the 4-bit linears.
    def nf4_matmul_bwd_meta(g, qweight, absmax, quant_map, blocksize, dtype, shape):
        assert g.shape[-1] == shape[0], f"{g.shape=}, weight {shape=}"
        return thunder.TensorProxy(like=g, shape=(*g.shape[:-1], shape[1]))

    def nf4_matmul_bwd_impl(g, qweight, absmax, quant_map, blocksize, dtype, shape):
        return functional.linear_nf4_input_grad(g, qweight, absmax, quant_map, blocksize, shape)

    nf4_matmul_bwd = ex.register_operator("nf4_b200_matmul_bwd", meta=nf4_matmul_bwd_meta, fn=nf4_matmul_bwd_impl)

    def nf4_matmul_grad(x, qweight, bias, absmax, quant_map, blocksize, dtype, shape):
        from thunder.core.transforms import get_grad, put_grad

        y = nf4_matmul(x, qweight, bias, absmax, quant_map, blocksize, dtype, shape)
        g = get_grad(y)
        put_grad(x, nf4_matmul_bwd(g, qweight, absmax, quant_map, blocksize, dtype, shape))
        if bias is not None and getattr(bias, "requires_grad", False):
            put_grad(bias, thunder.torch.sum(thunder.torch.reshape(g, (-1, shape[0])), 0))
        return y

    ex.register_implementation(nf4_matmul, nf4_matmul, checker=lambda *a, **k: True, grad_transform=nf4_matmul_grad)

    # The two torch-level ops at the ends of a decode step are claimed too when they have the form this
    # library's kernels take (thunder/extend/__init__.py:264-281: an implementation + a checker; everything the
    # checkers refuse stays with the executors behind this one): the token embedding lookup and the greedy
    # argmax over the vocabulary.
    def _on_cuda(p):
        return getattr(getattr(p, "device", None), "devicetype", None) == thunder.devices.DeviceType.CUDA

    def embedding_checker(a, weight, padding_idx=None, max_norm=None, norm_type=2.0, scale_grad_by_freq=False, sparse=False):
        return (_on_cuda(weight) and _on_cuda(a) and weight.dtype == thunder.dtypes.bfloat16 and a.dtype == thunder.dtypes.int64
                and weight.ndim == 2 and weight.shape[1] % 8 == 0 and padding_idx is None and max_norm is None
                and not getattr(weight, "requires_grad", False))

    def embedding_impl(a, weight, padding_idx=None, max_norm=None, norm_type=2.0, scale_grad_by_freq=False, sparse=False):
        return functional.embedding(a, weight)

    nf4_embedding = ex.register_operator("nf4_b200_embedding", like=thunder.torch.embedding, fn=embedding_impl)
    ex.register_implementation(thunder.torch.embedding, nf4_embedding, checker=embedding_checker)

    def argmax_checker(a, dim=None, keepdim=False):
        return (_on_cuda(a) and a.dtype == thunder.dtypes.bfloat16 and a.ndim >= 1 and dim is not None
                and (dim == -1 or dim == a.ndim - 1))

    def argmax_impl(a, dim=None, keepdim=False):
        return functional.argmax_last(a, bool(keepdim))

    nf4_argmax = ex.register_operator("nf4_b200_argmax", like=thunder.torch.argmax, fn=argmax_impl)
    ex.register_implementation(thunder.torch.argmax, nf4_argmax, checker=argmax_checker)
    _executor = ex
    return ex


class NF4LinearQuant4bit(Transform):
    """Quantizes the weights of all torch.nn.Linear submodules to NF4 (blocksize 64, fp32 absmax)
    and routes their `linear` calls to the `nf4_b200_matmul` symbol."""

    def __init__(self):
        self.quant_states: dict[str, dict] = {}
        self.quantized_submodule_names: set[str] = set()
        get_nf4_executor()

    # ---- weights ------------------------------------------------------------------------------
    def quantize_weight(self, w: torch.Tensor):
        """The kernels run on CUDA only: host weights are moved there, meta weights become zeros
        (as the reference does, quantization.py:53-63)."""
        if w.device.type == "meta":
            w_dev = torch.zeros_like(w, device="cuda")
        elif w.device.type != "cuda":
            with torch.no_grad():
                w_dev = w.to("cuda")
        else:
            w_dev = w
        return functional.quantize_4bit(w_dev, quant_type="nf4")

    def _store(self, tm, weight_name: str, w: torch.Tensor) -> None:
        packed, state = self.quantize_weight(w)
        tm._overrides_parameters[weight_name] = packed.to(w.device)
        tm._overrides_parameters[f"{weight_name}.absmax"] = state.absmax.to(w.device)
        tm._overrides_parameters[f"{weight_name}.code"] = state.code.to(w.device)
        self.quant_states[weight_name] = {
            "dtype": state.dtype,
            "shape": tuple(state.shape),
            "blocksize": state.blocksize,
            "qweight.dtype": packed.dtype,
            "qweight.shape": tuple(packed.shape),
            "absmax.dtype": state.absmax.dtype,
            "absmax.shape": tuple(state.absmax.shape),
            "code.dtype": state.code.dtype,
            "code.shape": tuple(state.code.shape),
            "device": getattr(w, "_thunder_device", w.device),
        }

    def transform_module(self, model) -> None:
        self.thunder_module = model
        aliases = model._get_shared_names()      # weight name -> all names bound to the same tensor
        done: set[str] = set()
        for name, sub in model._model.named_modules():
            if not isinstance(sub, torch.nn.Linear):
                continue
            self.quantized_submodule_names.add(name)
            wname = f"{name}.weight"
            twin = next(iter(aliases[wname] & done), None)
            if twin is not None:
                # a tied weight quantized earlier: share its tensors and its state
                self.quant_states[wname] = self.quant_states[twin]
                for suffix in ("", ".absmax", ".code"):
                    model._overrides_parameters[wname + suffix] = model._overrides_parameters[twin + suffix]
            else:
                self._store(model, wname, model.get_parameter(wname))
            done.add(wname)

    def transform_state_dict_for_submodule(self, model, submodule_name: str, state_dict: dict) -> dict:
        if submodule_name not in self.quantized_submodule_names:
            return state_dict
        expect = self.quant_states[f"{submodule_name}.weight"]
        w = state_dict["weight"]
        assert w.dtype == expect["dtype"]
        assert w.shape == expect["shape"]
        packed, state = self.quantize_weight(w)
        # the results go where the module keeps the parameter (the loader copies them in place): when that is
        # the device they were computed on, they stay there instead of travelling to the source's device and back
        held = model._overrides_parameters.get(f"{submodule_name}.weight")
        dst = held.device if held is not None and held.device == packed.device else w.device
        out = dict(state_dict)
        out["weight"] = packed.to(dst)
        out["weight.absmax"] = state.absmax.to(dst)
        out["weight.code"] = state.code.to(dst)
        return out

    # ---- traces -------------------------------------------------------------------------------
    def transform_traces_pre_prologue(self, prologue_trace, computation_trace, epilogue_trace, **kwargs):
        tm = self.thunder_module
        qstates = self.quant_states

        # 1. the prologue unpacks each weight: retype those proxies to the packed uint8 tensors
        retype = {}
        for pname, (_, unpack) in get_checks(prologue_trace).items():
            if pname in qstates:
                retype[unpack.output.name] = dict(shape=qstates[pname]["qweight.shape"],
                                                  dtype=thunder.dtypes.to_dtype(qstates[pname]["qweight.dtype"]))
        prologue_trace = trace_with_replaced_proxy_metadata(prologue_trace, retype)
        checks = get_checks(prologue_trace)
        passed_on = {o.name for o in prologue_trace.output[0]}

        # 2. per quantized weight: fix its check, unpack + check absmax/code, hand them to the computation
        weight_of_proxy: dict[str, str] = {}
        extra: dict[str, object] = {}         # "<w>.absmax" / "<w>.code" -> proxy
        new_prologue_bsyms, new_inputs = [], []
        for pname, st in qstates.items():
            for n in (pname, f"{pname}.absmax", f"{pname}.code"):
                tm.get_parameter(n)           # raises if the module lost one of them
            check, unpack = checks[pname]
            weight_of_proxy[unpack.output.name] = pname
            proxy, _, device, _, _ = check.args
            check.args = (proxy, st["qweight.shape"], device, st["qweight.dtype"], False)
            if unpack.output.name not in passed_on:
                continue
            with tracectx(prologue_trace):
                for kind in ("absmax", "code"):
                    p = thunder.TensorProxy(
                        name=f"{unpack.output.name}_{kind}",
                        shape=st[f"{kind}.shape"],
                        dtype=thunder.dtypes.to_dtype(st[f"{kind}.dtype"]),
                        device=thunder.devices.to_device(device),
                        requires_grad=False,
                        tags={ProxyTag.STATIC_MEMORY_LOCATION},
                    )
                    new_prologue_bsyms.append(unpack.sym.bind(unpack.args[0], f"{pname}.{kind}", output=p))
                    new_prologue_bsyms.append(prims.check_tensor_shape_and_metadata.bind(
                        p, st[f"{kind}.shape"], device, st[f"{kind}.dtype"], False, output=None))
                    add_trace_output(prologue_trace, p, subindex=0)
                    new_inputs.append(p)
                    extra[f"{pname}.{kind}"] = p
        prologue_trace.bound_symbols[-1:-1] = new_prologue_bsyms

        # 3. computation trace: new arguments, retyped weight proxies
        retype_c = {c.name: dict(shape=p.shape, dtype=p.dtype)
                    for p, c in zip(prologue_trace.bound_symbols[-1].args[0][0], computation_trace.args)
                    if p.shape != c.shape or p.dtype != c.dtype}
        computation_trace.args = (*computation_trace.args, *new_inputs)
        computation_trace.names.update(i.name for i in new_inputs)
        computation_trace._siginfo.args = [(a.name, None) for a in computation_trace.args]
        with tracectx(computation_trace):
            unpacks = [prims.unpack_trivial.bind(i, output=i, name=i.name) for i in new_inputs]
        at = len(computation_trace.bound_symbols)
        for i, b in enumerate(computation_trace.bound_symbols):
            if b.sym.id == prims.PrimIDs.UNPACK_TRIVIAL:
                at = i + 1
        computation_trace.bound_symbols[at:at] = unpacks
        computation_trace = trace_with_replaced_proxy_metadata(computation_trace, retype_c)

        # 4. linear(x, w, b) on a quantized weight -> nf4_b200_matmul(x, w, b, absmax, code, 64, dtype, (N, K))
        class _Rewrite(TraceSubstitutionProcessor):
            def process_bsym(self, bsym):
                if bsym.sym == thunder.torch.linear and bsym.args[1].name in weight_of_proxy:
                    assert len(bsym.args) == 3
                    pname = weight_of_proxy[bsym.args[1].name]
                    st = qstates[pname]
                    self.add_processed_bsyms([bsym.from_bsym(
                        sym=nf4_matmul, subsymbols=[],
                        args=(*bsym.args[:3], extra[f"{pname}.absmax"], extra[f"{pname}.code"], st["blocksize"],
                              st["dtype"], st["shape"]))])
                elif bsym.sym == prims.python_return:
                    assert len(bsym.args) == 1 and isinstance(bsym.args[0], dict)
                    ret = dict(bsym.args[0])
                    ret["flat_args"] = list(self.new_trace.args)
                    self.add_processed_bsyms([bsym.from_bsym(args=(ret,))])
                else:
                    self.add_processed_bsyms([bsym.from_bsym()])
                self.set_result(bsym.output)

        new_computation, _ = _Rewrite(computation_trace)()
        new_computation.set_provenance(TraceProvenance("quant pass"))
        return prologue_trace, new_computation, epilogue_trace


class QuantizeNF4(thunder.Plugin):
    """Plugin form: `thunder.compile(model, plugins=QuantizeNF4())`."""

    def setup_transforms(self):
        return [NF4LinearQuant4bit()]

    def setup_executors(self):
        return [get_nf4_executor()]


def register_plugin(name: str = "quantize-int4") -> None:
    """Makes `plugins="<name>"` resolve to QuantizeNF4 (default: the reference's own name)."""
    import thunder.plugins

    thunder.plugins.register_plugin(name, QuantizeNF4)


def install_as_bitsandbytes() -> types.ModuleType:
    """Registers a module named `bitsandbytes` exposing `functional.quantize_4bit`,
    `functional.QuantState` and `matmul_4bit`, the three entry points the reference's transform
    uses (quantization.py:35-39, 63).  Refuses to shadow a real installation."""
    existing = sys.modules.get("bitsandbytes")
    if existing is not None and not getattr(existing, "_nf4_b200_alias", False):
        raise RuntimeError("a real `bitsandbytes` module is already imported")
    mod = types.ModuleType("bitsandbytes")
    mod._nf4_b200_alias = True
    mod.functional = functional
    mod.matmul_4bit = lambda *a, **k: functional.matmul_4bit(*a, **k)
    mod.__version__ = "0.48.0+nf4_b200"
    sys.modules["bitsandbytes"] = mod
    sys.modules["bitsandbytes.functional"] = functional
    return mod
