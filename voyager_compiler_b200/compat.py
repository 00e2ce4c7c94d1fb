"""Optional shim for the callers in voyager-compiler that bypass the dispatcher.

``quantization/fake_quantize.py:10`` and ``quantization/gptq.py:26`` import the *Python functions*
``vmap``, ``quantize_mx``, ``expand`` and ``calculate_mx_qparam`` directly, and inside
``ops/quantized.py`` the ops call each other as Python functions, so kernels registered on
``torch.ops.quantized_ops`` are not reached from the prepare-time fake-quant path.  ``patch_reference()``
rebinds those names to wrappers that send CUDA tensors through the dispatcher (and therefore to this
package's kernels) and everything else to the original function.  The forwards of upstream's
``FakeQuantizeFunction``, ``MXFakeQuantizeFunction`` and ``GroupWiseAffineFakeQuantFunction``
(quantization/fake_quantize.py:101-214) are
rebound the same way to the fused one-pass kernels of :mod:`voyager_compiler_b200.fake_quantize`, and
``compensate_weight`` of ``quantization/gptq.py`` to :mod:`voyager_compiler_b200.gptq`, ``_accumulate`` of
``quantization/lcq.py`` to :mod:`voyager_compiler_b200.lcq`.
Off by default; undo with ``unpatch_reference()``.
"""
from __future__ import annotations

import functools
import importlib
import sys
from typing import Dict, List, Tuple

import torch

_PATCHED: List[Tuple[object, str, object]] = []

_TARGETS: Dict[str, Tuple[str, ...]] = {
    "voyager_compiler.ops.quantized": ("vmap", "quantize", "dequantize", "calculate_mx_qparam", "quantize_mx"),
    "voyager_compiler.ops": ("vmap", "quantize", "dequantize", "calculate_mx_qparam", "quantize_mx"),
    "voyager_compiler.quantization.fake_quantize": ("vmap", "quantize_mx"),
    "voyager_compiler.quantization.gptq": ("vmap", "calculate_mx_qparam"),
}


def _wrap(name: str, original):
    op = getattr(torch.ops.quantized_ops, name)

    @functools.wraps(original)
    def dispatching(input, *args, **kwargs):
        if isinstance(input, torch.Tensor) and input.is_cuda:
            return op(input, *args, **kwargs)
        return original(input, *args, **kwargs)

    dispatching.__wrapped_original__ = original
    return dispatching


def patch_reference() -> List[str]:
    """Rebind the directly imported functions in every already-imported upstream module.  Returns
    the patched ``module.name`` strings."""
    done = []
    for modname, names in _TARGETS.items():
        mod = sys.modules.get(modname)
        if mod is None:
            try:
                mod = importlib.import_module(modname)
            except Exception:  # noqa: BLE001  (module needs packages that are not installed)
                continue
        for n in names:
            fn = getattr(mod, n, None)
            if fn is None or hasattr(fn, "__wrapped_original__"):
                continue
            setattr(mod, n, _wrap(n, fn))
            _PATCHED.append((mod, n, fn))
            done.append(f"{modname}.{n}")
    _patch_fake_quant_functions(done)
    _patch_gptq(done)
    _patch_lcq(done)
    return done


def _patch_lcq(done: List[str]) -> None:
    """``_accumulate`` of upstream's codebook fit (quantization/lcq.py:601-626: unit scale, weights, three
    ``index_add_``) -> one launch of :func:`voyager_compiler_b200.lcq.accumulate_moments` for CUDA tensors whose
    blocks run along the last axis."""
    mod = sys.modules.get("voyager_compiler.quantization.lcq")
    if mod is None or not hasattr(mod, "_accumulate"):
        return
    original = mod._accumulate
    if hasattr(original, "__wrapped_original__"):
        return
    from . import lcq as ours

    @functools.wraps(original)
    def _accumulate(tensor, module, energy, histogram):
        axis = module.ch_axis[0] if isinstance(module.ch_axis, (tuple, list)) else module.ch_axis
        fused = (isinstance(tensor, torch.Tensor) and tensor.is_cuda and axis in (-1, tensor.dim() - 1)
                 and tensor.shape[-1] % module.block_size == 0 and tensor.numel() >= module.block_size)
        if not fused:
            return original(tensor, module, energy, histogram)
        if histogram.weight is None:
            histogram.weight, histogram.total, histogram.square = (
                torch.zeros(histogram.bins, dtype=torch.float64, device=tensor.device) for _ in range(3))
        ours.accumulate_moments(histogram.weight, histogram.total, histogram.square, histogram.quant_min, histogram.quant_max,
                                tensor.detach(), module.block_size, module.quant_max, energy)

    _accumulate.__wrapped_original__ = original
    mod._accumulate = _accumulate
    _PATCHED.append((mod, "_accumulate", original))
    done.append("voyager_compiler.quantization.lcq._accumulate")


def _patch_gptq(done: List[str]) -> None:
    """``compensate_weight`` of upstream's GPTQ driver (quantization/gptq.py:184-270) -> the block-per-launch
    walk of :mod:`voyager_compiler_b200.gptq` for CUDA weights with blocks of up to 64 input channels."""
    mod = sys.modules.get("voyager_compiler.quantization.gptq")
    if mod is None or not hasattr(mod, "compensate_weight"):
        return
    original = mod.compensate_weight
    if hasattr(original, "__wrapped_original__"):
        return
    from . import gptq as ours

    @functools.wraps(original)
    def compensate_weight(weight, hessian, tokens, fake_quant, *args, **kwargs):
        if isinstance(weight, torch.Tensor) and weight.is_cuda and weight.dim() == 2 and fake_quant.block_size <= 64:
            return ours.compensate_weight(weight, hessian, tokens, fake_quant, *args, **kwargs)
        return original(weight, hessian, tokens, fake_quant, *args, **kwargs)

    compensate_weight.__wrapped_original__ = original
    mod.compensate_weight = compensate_weight
    _PATCHED.append((mod, "compensate_weight", original))
    done.append("voyager_compiler.quantization.gptq.compensate_weight")


def _patch_fake_quant_functions(done: List[str]) -> None:
    mod = sys.modules.get("voyager_compiler.quantization.fake_quantize")
    if mod is None:
        return
    from . import fake_quantize as ours

    def wrap_forward(cls, fused):
        original = cls.__dict__["forward"]
        original_fn = original.__func__ if isinstance(original, staticmethod) else original
        if hasattr(original_fn, "__wrapped_original__"):
            return

        @functools.wraps(original_fn)
        def forward(ctx, input, *args, **kwargs):
            if isinstance(input, torch.Tensor) and input.is_cuda and input.dtype in (torch.float32, torch.bfloat16):
                return fused(ctx, input, *args, **kwargs)
            return original_fn(ctx, input, *args, **kwargs)

        forward.__wrapped_original__ = original_fn
        setattr(cls, "forward", staticmethod(forward))
        _PATCHED.append((cls, "forward", original))
        done.append(f"voyager_compiler.quantization.fake_quantize.{cls.__name__}.forward")

    if hasattr(mod, "FakeQuantizeFunction"):
        wrap_forward(mod.FakeQuantizeFunction, ours.FakeQuantizeFunction.forward)
    if hasattr(mod, "MXFakeQuantizeFunction"):
        wrap_forward(mod.MXFakeQuantizeFunction, ours.MXFakeQuantizeFunction.forward)
    if hasattr(mod, "GroupWiseAffineFakeQuantFunction"):
        def group_affine(ctx, input, fake_quant_enabled, scale, zero_point, axes, *rest, **kw):
            one_axis = isinstance(axes, int) or len(axes) == 1
            target = ours.GroupWiseAffineFakeQuantFunction.forward if one_axis else \
                mod.GroupWiseAffineFakeQuantFunction.forward.__wrapped_original__       # several block axes: upstream's own ops
            return target(ctx, input, fake_quant_enabled, scale, zero_point, axes, *rest, **kw)
        wrap_forward(mod.GroupWiseAffineFakeQuantFunction, group_affine)


def unpatch_reference() -> None:
    while _PATCHED:
        mod, n, fn = _PATCHED.pop()
        setattr(mod, n, fn)


# ---------------------------------------------------------------------------------------------
def fuse_dynamic_linear(gm: "torch.fx.GraphModule") -> int:
    """Graph pass over a converted model: the node group the converter emits for a dynamically
    quantized linear (quantization/quantize_pt2e.py:431-712),

        q = quantized_ops.quantize_mx(x, qmap, (-1,), block, quant_max, pow2, scale_qmap, None)
        s, c = q[0], q[1]
        y = quantized_ops.linear_mx(c, w, bias, input_scale=s, weight_scale=ws, block_size=block, ...)

    becomes one call of :func:`voyager_compiler_b200.gemm_native.linear_mx_dynamic` when nothing else
    reads the codes or the scale: the activation's ``codes * scale`` are then written straight into the
    GEMM's left operand by one pass instead of travelling through HBM as two tensors and back.  The
    result is bit-identical.  Nodes that do not match (other block axes, a codebook on the activation,
    the sparse outlier side path, a ``"ck"`` weight) are left as they are.  Returns the number of
    fused linears; the module is recompiled when that is not zero."""
    import operator

    from .gemm_native import linear_mx_dynamic

    Q = torch.ops.quantized_ops
    fused = 0
    for lin in list(gm.graph.nodes):
        if lin.op != "call_function" or lin.target is not Q.linear_mx.default:
            continue
        kw = dict(lin.kwargs)
        codes, scale = lin.args[0], kw.get("input_scale")
        if not (isinstance(codes, torch.fx.Node) and isinstance(scale, torch.fx.Node)):
            continue
        if codes.target is not operator.getitem or scale.target is not operator.getitem:
            continue
        q = codes.args[0]
        if q is not scale.args[0] or codes.args[1] != 1 or scale.args[1] != 0:
            continue
        if not (isinstance(q, torch.fx.Node) and q.op == "call_function" and q.target is Q.quantize_mx.default):
            continue
        if set(codes.users) != {lin} or set(scale.users) != {lin} or set(q.users) != {codes, scale}:
            continue
        qa = list(q.args) + [None] * (8 - len(q.args))
        x, qmap, axes, block, qmax, pow2, scale_qmap, out_code = qa[:8]
        pow2 = q.kwargs.get("force_scale_power_of_two", pow2 if pow2 is not None else False)
        scale_qmap = q.kwargs.get("scale_qmap", scale_qmap)
        axes = tuple(axes) if isinstance(axes, (list, tuple)) else (axes,)
        if axes != (-1,) or kw.get("block_size") != block or kw.get("input_code") is not None:
            continue
        if any(kw.get(k) is not None for k in ("A_data", "A_indices", "A_indptr")) or kw.get("weight_layout", "kc") != "kc":
            continue
        bias = lin.args[2] if len(lin.args) > 2 else None
        with gm.graph.inserting_before(lin):
            new = gm.graph.call_function(linear_mx_dynamic, (x, lin.args[1], bias), {
                "qmap": qmap, "weight_scale": kw.get("weight_scale"), "block_size": block, "quant_max": qmax,
                "force_scale_power_of_two": bool(pow2), "scale_qmap": scale_qmap, "weight_code": kw.get("weight_code")})
        new.meta = dict(lin.meta)
        lin.replace_all_uses_with(new)
        for dead in (lin, codes, scale, q):
            gm.graph.erase_node(dead)
        fused += 1
    if fused:
        gm.graph.lint()
        gm.recompile()
    return fused
