"""Converted graphs of upstream's ``convert_pt2e`` replayed on the CUDA kernels.

``tests/golden/make_golden_convert.py`` ran upstream's converter
(src/voyager_compiler/quantization/quantize_pt2e.py:930-967) on hand-prepared graphs -- a linear /
matmul between two MX fake-quantize modules -- and stored the resulting graph as data together
with what upstream's CPU kernels compute for it.  Here the graph is rebuilt node for node over
``torch.ops.quantized_ops.*`` (this package's registration, positional ``None``s and explicit
``input_code=None`` keywords included) and executed on the GPU: the drop-in consumer's view of the
ops.  Codes and scales must match bit for bit, the contraction within the linear's tolerance.
"""
import json
import operator
import os

import numpy as np
import pytest
import torch

from golden_util import GOLDEN, from_bits

with open(os.path.join(GOLDEN, "golden_convert.json")) as _f:
    CASES = json.load(_f)["cases"]
_Z = None


def _tensor(case, key):
    global _Z
    if _Z is None:
        _Z = np.load(os.path.join(GOLDEN, "golden_convert.npz"))
    meta = case["tensors"][key]
    a = _Z[f"{case['name']}/{key}"]
    if meta["tag"] in ("i32", "u8"):
        return torch.from_numpy(a.copy()).reshape(meta["shape"])
    return from_bits(a, meta["tag"], meta["shape"])


def _target(name):
    if name == "getitem":
        return operator.getitem
    if name == "Tensor.to":
        return torch.Tensor.to
    ns_op, overload = name.rsplit(".", 1)
    ns, op = ns_op.split("::")
    return getattr(getattr(getattr(torch.ops, ns), op), overload)


def _rebuild(case, device):
    """torch.fx.GraphModule equal to the stored converted graph, its buffers on ``device``."""
    root = torch.nn.Module()
    for key in case["tensors"]:
        if key.startswith("attr/"):
            root.register_buffer(key[5:], _tensor(case, key).to(device))
    g = torch.fx.Graph()
    env = {}

    def arg(a):
        if "node" in a:
            return env[a["node"]]
        if "seq" in a:
            return tuple(arg(v) for v in a["seq"])
        if "device" in a:
            return torch.device(device)
        return a["value"]

    for n in case["nodes"]:
        args = tuple(arg(a) for a in n["args"])
        kwargs = {k: arg(v) for k, v in n["kwargs"].items()}
        if n["op"] == "placeholder":
            env[n["name"]] = g.placeholder(n["target"])
        elif n["op"] == "get_attr":
            env[n["name"]] = g.get_attr(n["target"])
        elif n["op"] == "call_function":
            env[n["name"]] = g.call_function(_target(n["target"]), args, kwargs)
        elif n["op"] == "output":
            g.output(args[0])
        else:
            raise AssertionError(f"unexpected node kind {n['op']}")
        if n["op"] != "output":
            env[n["name"]].name = n["name"]
    return torch.fx.GraphModule(root, g)


def test_fixture_graphs_use_the_op_set_this_package_registers():
    import voyager_compiler_b200 as vb
    from voyager_compiler_b200 import ops
    seen = set()
    for case in CASES:
        for n in case["nodes"]:
            if n["op"] == "call_function" and n["target"].startswith("quantized_ops::"):
                op = n["target"].split("::")[1].split(".")[0]
                seen.add(op)
                assert op in ops.SCHEMAS, op
                _target(n["target"])                     # resolves on the dispatcher
    assert {"quantize_mx", "linear_mx", "matmul_mx", "quantize_mx_outlier"} <= seen
    # the converter's calling convention: scale_qmap / output_code passed as positional None,
    # block_size and the codes as keywords on the contraction
    lin = next(n for n in CASES[0]["nodes"] if n["target"].startswith("quantized_ops::linear_mx"))
    assert set(lin["kwargs"]) >= {"input_scale", "weight_scale", "block_size", "input_code", "weight_code"}
    assert vb.REGISTERED_AS in ("def", "impl")


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_converted_graph_runs_on_cuda_like_upstream_on_cpu(case):
    import voyager_compiler_b200  # noqa: F401  (registers the CUDA kernels)

    gm = _rebuild(case, "cuda")

    class Keep(torch.fx.Interpreter):
        def __init__(self, m):
            super().__init__(m)
            self.seen = {}

        def run_node(self, n):
            r = super().run_node(n)
            if n.op == "call_function" and isinstance(r, torch.Tensor):
                self.seen[n.name] = r
            return r

    keep = Keep(gm)
    x = _tensor(case, "x").cuda()
    out = keep.run(x)
    torch.cuda.synchronize()
    want = _tensor(case, "converted_out")
    assert out.shape == want.shape and out.dtype == want.dtype and out.is_cuda
    contraction = {n["name"] for n in case["nodes"]
                   if n["op"] == "call_function" and n["target"].split("::")[-1].split(".")[0] in ("linear_mx", "matmul_mx")}
    compared = 0
    for name, got in keep.seen.items():
        ref = _tensor(case, "node/" + name)
        if name in contraction:
            rel = ((got.double().cpu() - ref.double()).norm() / ref.double().norm()).item()
            assert rel <= 1e-2, (name, rel)                 # bf16 / fp32-accumulate contraction
        else:
            g, r = got.cpu(), ref
            assert g.shape == r.shape and g.dtype == r.dtype, name
            if g.is_floating_point():
                same = (g == r) | (torch.isnan(g) & torch.isnan(r))
                assert bool(same.all()), f"{name}: codes / scales / CSR values differ"
            else:
                assert torch.equal(g, r), name
        compared += 1
    assert compared >= 3
    # the converted model still computes what the fake-quantized model computed
    fake = _tensor(case, "fake_quant_out").double()
    rel = ((out.double().cpu() - fake).norm() / fake.norm()).item()
    assert rel <= 2e-2, rel


def test_fuse_dynamic_linear_rewrites_only_the_matching_node_groups():
    """Graph surgery is host work: the pass is checked on the stored graphs without running them."""
    from voyager_compiler_b200 import compat, gemm_native
    want = {"linear_int8_int8_bf16": 1, "linear_int8_nf4_codebook_bf16": 1, "linear_fp8_int8_f32_3d": 1,
            "linear_int8_outliers_bf16": 0, "matmul_int8_int8_bf16": 0}
    for case in CASES:
        gm = _rebuild(case, "cpu")
        assert compat.fuse_dynamic_linear(gm) == want[case["name"]], case["name"]
        targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
        if want[case["name"]]:
            assert targets == [gemm_native.linear_mx_dynamic]
            (n,) = [n for n in gm.graph.nodes if n.op == "call_function"]
            assert n.kwargs["block_size"] == 32 and n.kwargs["force_scale_power_of_two"] is True
        assert compat.fuse_dynamic_linear(gm) == 0                  # idempotent


@pytest.mark.gpu
@pytest.mark.parametrize("case", [c for c in CASES if c["name"] in ("linear_int8_int8_bf16", "linear_int8_nf4_codebook_bf16")],
                         ids=lambda c: c["name"])
def test_fused_dynamic_linear_equals_the_two_node_form_bitwise(case):
    import voyager_compiler_b200  # noqa: F401
    from voyager_compiler_b200 import compat
    x = _tensor(case, "x").cuda()
    plain = _rebuild(case, "cuda")
    want = plain(x)
    fused = _rebuild(case, "cuda")
    assert compat.fuse_dynamic_linear(fused) == 1
    got = fused(x)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
