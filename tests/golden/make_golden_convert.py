"""Fixtures of upstream's ``convert_pt2e`` on hand-prepared graphs (run once, where an upstream
checkout is available; the output is committed):

    python tests/golden/make_golden_convert.py

Each case is an ``aten.linear`` (or ``aten.matmul``) whose activation and weight pass through two
``FusedAmaxObsFakeQuantize`` modules with the microscaling scheme -- the graph ``prepare_pt2e``
leaves behind.  The script records the fake-quantized output, runs upstream's
``convert_pt2e`` (src/voyager_compiler/quantization/quantize_pt2e.py:930-967, MX branch
:431-712) and stores the converted graph as data: every node with its op, target, args and
kwargs, every buffer the conversion created, the input and the output upstream's own CPU
kernels give for it.  ``tests/test_convert_replay.py`` rebuilds that graph over
``torch.ops.quantized_ops.*`` and runs it on CUDA.

``golden_convert.json``: cases -> node lists.  ``golden_convert.npz``: tensors as raw bit patterns.
"""
import importlib
import json
import operator
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def _import_convert():
    """Upstream's quantize_pt2e next to a stand-in for the torchao pieces it only uses as base
    classes (torchao is not installed here); transformers is imported first because its lazy
    modules probe for torchao and must not meet the stand-in."""
    import transformers  # noqa: F401
    import transformers.modeling_utils  # noqa: F401
    import _reference_import as ri

    ri._install_torchao_stub()
    p = sys.modules["torchao.quantization.pt2e"]

    class QuantizationSpecBase:
        pass

    class Quantizer:
        pass

    class QuantizationAnnotation:
        def __init__(self, input_qspec_map=None, output_qspec=None, allow_implicit_sharing=True, _annotated=False):
            self.input_qspec_map = input_qspec_map or {}
            self.output_qspec = output_qspec
            self._annotated = _annotated

    mods = [types.ModuleType("torchao.quantization.pt2e.quantizer" + s) for s in ("", ".quantizer", ".utils")]
    for m in mods:
        m.QuantizationSpecBase, m.Quantizer, m.QuantizationAnnotation, m.EdgeOrNode = QuantizationSpecBase, Quantizer, QuantizationAnnotation, object
        m.annotate_input_qspec_map = m.annotate_output_qspec = lambda *a, **k: None
        m.SharedQuantizationSpec = type("SharedQuantizationSpec", (QuantizationSpecBase,), {})
        m.FixedQParamsQuantizationSpec = type("FixedQParamsQuantizationSpec", (QuantizationSpecBase,), {})
        sys.modules[m.__name__] = m
    p.quantizer, mods[0].quantizer, mods[0].utils = mods[0], mods[1], mods[2]
    ref = ri.import_reference()
    src = os.path.join(ri.default_reference_root(), "src", "voyager_compiler")
    ri._namespace("voyager_compiler.quantization.quantizer", os.path.join(src, "quantization", "quantizer"))
    ref["quantize_pt2e"] = importlib.import_module("voyager_compiler.quantization.quantize_pt2e")
    return ref


def _bits(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy(), "bf16"
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32).copy(), "f32"
    if t.dtype == torch.int64:
        return t.numpy().copy(), "i64"
    if t.dtype == torch.int32:
        return t.numpy().copy(), "i32"
    if t.dtype == torch.uint8:
        return t.numpy().copy(), "u8"
    raise TypeError(t.dtype)


def _target_name(t):
    if t is operator.getitem:
        return "getitem"
    if t is torch.Tensor.to:
        return "Tensor.to"
    if isinstance(t, torch._ops.OpOverload):
        return t.name() + "." + t._overloadname            # e.g. quantized_ops::linear_mx.default
    if isinstance(t, str):
        return t
    raise TypeError(f"unexpected call target {t!r}")


def _arg(a):
    if isinstance(a, torch.fx.Node):
        return {"node": a.name}
    if isinstance(a, (list, tuple)):
        return {"seq": [_arg(v) for v in a]}
    if isinstance(a, torch.device):
        return {"device": True}
    if a is None or isinstance(a, (bool, int, float, str)):
        return {"value": a}
    raise TypeError(f"unexpected argument {a!r}")


def _graph_data(gm):
    nodes = []
    for n in gm.graph.nodes:
        nodes.append({"name": n.name, "op": n.op, "target": _target_name(n.target) if n.op != "output" else "output",
                      "args": [_arg(a) for a in n.args], "kwargs": {k: _arg(v) for k, v in n.kwargs.items()},
                      "dtype": n.meta.get("dtype")})
    return nodes


def _linear_case(ref, name, dtype_act, dtype_w, block_w, x, weight, bias, act_kw=None, matmul_other=None):
    fqm, QS = ref["fake_quantize"], ref["qspec"].QScheme
    root = torch.nn.Module()
    root.weight = torch.nn.Parameter(weight, requires_grad=False)
    if bias is not None:
        root.bias = torch.nn.Parameter(bias, requires_grad=False)
    qmax = {"int8": 127.0, "nf4": 1.0, "fp8_e4m3": 448.0, "int4": 7.0}
    act_kw = act_kw or {}
    root.activation_post_process_0 = fqm.FusedAmaxObsFakeQuantize(
        dtype_act, qscheme=QS.MICROSCALING, quant_max=qmax[dtype_act], ch_axis=-1, block_size=32,
        force_scale_power_of_two=True, **act_kw)
    w_axis = -1 if matmul_other is None else -2
    root.activation_post_process_1 = fqm.FusedAmaxObsFakeQuantize(
        dtype_w, qscheme=QS.MICROSCALING, quant_max=qmax[dtype_w], ch_axis=w_axis, block_size=block_w,
        force_scale_power_of_two=dtype_w != "nf4")
    g = torch.fx.Graph()
    xin = g.placeholder("x")
    w = g.get_attr("weight")
    xq = g.call_module("activation_post_process_0", (xin,))
    wq = g.call_module("activation_post_process_1", (w,))
    if matmul_other is None:
        b = g.get_attr("bias") if bias is not None else None
        y = g.call_function(torch.ops.aten.linear.default, (xq, wq, b))
    else:
        y = g.call_function(torch.ops.aten.matmul.default, (xq, wq))
    g.output(y)
    gm = torch.fx.GraphModule(root, g)
    fake = gm(x).clone()                                             # the fake-quantized model's output
    conv = ref["quantize_pt2e"].convert_pt2e(gm)
    # upstream's CPU kernels on the converted graph, every node's result kept
    class Keep(torch.fx.Interpreter):
        def __init__(self, m):
            super().__init__(m)
            self.seen = {}

        def run_node(self, n):
            r = super().run_node(n)
            if n.op == "call_function" and isinstance(r, torch.Tensor):
                self.seen[n.name] = r.clone()
            return r

    keep = Keep(conv)
    out = keep.run(x).clone()
    tensors = {"x": x, "fake_quant_out": fake, "converted_out": out}
    for k, t in keep.seen.items():
        tensors["node/" + k] = t
    for n in conv.graph.nodes:
        if n.op == "get_attr":
            tensors["attr/" + n.target] = getattr(conv, n.target)
    targets = [_target_name(n.target) for n in conv.graph.nodes if n.op == "call_function"]
    print(f"{name}: {targets}")
    return {"name": name, "nodes": _graph_data(conv), "note": f"act {dtype_act}, weight {dtype_w} block {block_w}"}, tensors


def main():
    ref = _import_convert()
    torch.manual_seed(20)
    cases, arrays = [], {}

    def add(case, tensors):
        case["tensors"] = {}
        for k, t in tensors.items():
            a, tag = _bits(t)
            arrays[f"{case['name']}/{k}"] = a
            case["tensors"][k] = {"tag": tag, "shape": list(t.shape)}
        cases.append(case)

    x = torch.randn(48, 128).bfloat16()
    x[3, :32] = 0
    w = (torch.randn(96, 128) * 0.05).bfloat16()
    b = torch.randn(96).bfloat16()
    add(*_linear_case(ref, "linear_int8_int8_bf16", "int8", "int8", 32, x, w, b))
    add(*_linear_case(ref, "linear_int8_nf4_codebook_bf16", "int8", "nf4", 32, x, w, None))
    xf = torch.randn(2, 40, 64)
    wf = torch.randn(72, 64) * 0.1
    add(*_linear_case(ref, "linear_fp8_int8_f32_3d", "fp8_e4m3", "int8", 32, xf, wf, torch.randn(72)))
    xo = torch.randn(64, 128).bfloat16()
    xo[torch.rand(64, 128) < 0.01] *= 40
    add(*_linear_case(ref, "linear_int8_outliers_bf16", "int8", "int8", 32, xo, w, b, act_kw={"outlier_threshold": 6.0}))
    other = (torch.randn(128, 80) * 0.05).bfloat16()
    add(*_linear_case(ref, "matmul_int8_int8_bf16", "int8", "int8", 32, x, other, None, matmul_other=True))

    np.savez_compressed(os.path.join(HERE, "golden_convert.npz"), **arrays)
    with open(os.path.join(HERE, "golden_convert.json"), "w") as f:
        json.dump({"cases": cases, "torch": torch.__version__}, f, indent=1)
    print(f"wrote {len(cases)} cases, {len(arrays)} arrays")


if __name__ == "__main__":
    main()
