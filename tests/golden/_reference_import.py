"""Import the upstream voyager-compiler hot-path modules without its heavy package
``__init__`` files.

Only used by ``make_golden.py`` (fixture generation, run once where the upstream
checkout is available).  Nothing in the test-suite, the benchmark or the package
imports this module.

The upstream package ``__init__`` pulls in torchao / accelerate / transformers export
helpers that are not needed for the quantized ops.  We therefore pre-seed empty
namespace packages whose ``__path__`` points at the upstream directories, and install
a minimal ``torchao.quantization.pt2e`` stand-in that only supplies the base classes
``fake_quantize.py`` subclasses.
"""
import importlib
import os
import sys
import types


def _namespace(name, path):
    mod = types.ModuleType(name)
    mod.__path__ = [path]
    sys.modules[name] = mod
    return mod


def _install_torchao_stub():
    import torch

    if "torchao" in sys.modules:
        return
    tao = types.ModuleType("torchao")
    q = types.ModuleType("torchao.quantization")
    p = types.ModuleType("torchao.quantization.pt2e")
    p.FakeQuantizeBase = torch.ao.quantization.FakeQuantizeBase
    p.ObserverOrFakeQuantize = object
    tao.quantization = q
    q.pt2e = p
    sys.modules["torchao"] = tao
    sys.modules["torchao.quantization"] = q
    sys.modules["torchao.quantization.pt2e"] = p


def default_reference_root():
    """``$VOYAGER_REFERENCE``, else a ``reference`` checkout next to this repository."""
    here = os.path.dirname(os.path.abspath(__file__))
    repo = os.path.dirname(os.path.dirname(here))
    return os.environ.get("VOYAGER_REFERENCE", os.path.join(os.path.dirname(repo), "reference"))


def import_reference(root=None):
    """Returns a dict of the upstream modules needed to generate fixtures."""
    root = root or default_reference_root()
    src = os.path.join(root, "src", "voyager_compiler")
    if not os.path.isdir(src):
        raise FileNotFoundError(f"upstream checkout not found at {root}")
    _install_torchao_stub()
    _namespace("voyager_compiler", src)
    _namespace("voyager_compiler.quantization", os.path.join(src, "quantization"))
    _namespace("voyager_compiler.codegen", os.path.join(src, "codegen"))
    ops = importlib.import_module("voyager_compiler.ops")
    fq = importlib.import_module("voyager_compiler.quantization.fake_quantize")
    mx = importlib.import_module("voyager_compiler.quantization.mx_utils")
    dtypes = importlib.import_module("voyager_compiler.quantization.dtypes")
    qspec = importlib.import_module("voyager_compiler.quantization.qspec")
    return {"ops": ops, "fake_quantize": fq, "mx_utils": mx, "dtypes": dtypes, "qspec": qspec}
