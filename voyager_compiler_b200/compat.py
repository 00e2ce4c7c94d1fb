"""Optional shim for the callers in voyager-compiler that bypass the dispatcher.

``quantization/fake_quantize.py:10`` and ``quantization/gptq.py:26`` import the *Python functions*
``vmap``, ``quantize_mx``, ``expand`` and ``calculate_mx_qparam`` directly, and inside
``ops/quantized.py`` the ops call each other as Python functions, so kernels registered on
``torch.ops.quantized_ops`` are not reached from the prepare-time fake-quant path.  ``patch_reference()``
rebinds those names to wrappers that send CUDA tensors through the dispatcher (and therefore to this
package's kernels) and everything else to the original function.  Off by default; undo with
``unpatch_reference()``.
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
    return done


def unpatch_reference() -> None:
    while _PATCHED:
        mod, n, fn = _PATCHED.pop()
        setattr(mod, n, fn)
