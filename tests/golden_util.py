"""Loading and replaying the golden fixtures (upstream inputs/outputs) in tests/golden/."""
import json
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

_cache = {}


def _load():
    if not _cache:
        _cache["tables"] = np.load(os.path.join(GOLDEN, "golden_tables.npz"))
        _cache["ops"] = np.load(os.path.join(GOLDEN, "golden_ops.npz"))
        with open(os.path.join(GOLDEN, "golden_ops.json")) as f:
            _cache["manifest"] = json.load(f)
    return _cache


def from_bits(arr, tag, shape=None):
    if tag == "f32":
        t = torch.from_numpy(arr.view(np.int32).copy()).view(torch.float32)
    elif tag == "bf16":
        t = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    elif tag == "i64":
        t = torch.from_numpy(arr.copy())
    else:
        raise ValueError(tag)
    return t.reshape(shape) if shape is not None else t


def golden_table(name) -> torch.Tensor:
    """A 65 536-entry bf16 value table produced by the upstream builders."""
    return from_bits(_load()["tables"][name], "bf16")


def golden_table_names():
    return [k for k in _load()["tables"].files if "/" not in k]


def golden_aux(name):
    return _load()["tables"][name]


def index_table_of(name):
    """(int64 index table, levels) as quantize_pt2e.py:456-466 derives them."""
    tab = golden_table(name)
    levels = torch.unique(tab)
    return torch.searchsorted(levels, tab).to(torch.int64), levels


def cases(op=None):
    return [c for c in _load()["manifest"]["cases"] if op is None or c["op"] == op]


def case_ids(op=None):
    return [c["name"] for c in cases(op)]


def materialize(case, device="cpu"):
    """Returns (tensors dict, params dict, expected outputs list) of one case."""
    ops = _load()["ops"]
    tensors = {}
    for arg, spec in case["tensors"].items():
        if "table" in spec:
            t = golden_table(spec["table"])
        else:
            t = from_bits(ops[spec["key"]], spec["dtype"], spec["shape"])
        tensors[arg] = t.to(device)
    params = dict(case["params"])
    if params.get("index_table_of"):
        tensors["qmap"] = index_table_of(params.pop("index_table_of"))[0].to(device)
    params.pop("index_table_of", None)
    if params.pop("transpose_input", False):
        # stored as the contiguous logical tensor; rebuild the non-contiguous view
        tensors["input"] = tensors["input"].t().contiguous().t()
    expected = [from_bits(ops[o["key"]], o["dtype"], o["shape"]) for o in case["outputs"]]
    return tensors, params, expected


def same_bits(a: torch.Tensor, b: torch.Tensor):
    """Bitwise equality except that any NaN equals any NaN.  Returns (ok, message)."""
    a, b = a.detach().cpu(), b.detach().cpu()
    if a.dtype != b.dtype or a.shape != b.shape:
        return False, f"dtype/shape {a.dtype}{tuple(a.shape)} vs {b.dtype}{tuple(b.shape)}"
    if a.is_floating_point():
        na, nb = torch.isnan(a), torch.isnan(b)
        if not torch.equal(na, nb):
            return False, f"NaN positions differ ({int((na != nb).sum())})"
        it = torch.int32 if a.dtype == torch.float32 else torch.int16
        ai = torch.where(na, torch.zeros_like(a), a).contiguous().view(it)
        bi = torch.where(nb, torch.zeros_like(b), b).contiguous().view(it)
    else:
        ai, bi = a, b
    bad = ai != bi
    n = int(bad.sum())
    if n:
        i = bad.flatten().nonzero()[0].item()
        return False, f"{n} of {a.numel()} differ; first at flat {i}: {a.flatten()[i].item()!r} vs {b.flatten()[i].item()!r}"
    return True, ""


def run_case(case, backend, device="cpu"):
    """Replay a case through ``backend`` — an object exposing vmap/quantize/dequantize/
    calculate_mx_qparam/quantize_mx/linear_mx/matmul_mx with the upstream signatures."""
    t, p, expected = materialize(case, device)
    op = case["op"]
    if op == "vmap":
        out = backend.vmap(t["input"], t["qmap"])
    elif op == "quantize":
        out = backend.quantize(t["input"], t["scale"], t.get("zero_point"), p.get("axes"), p.get("block_size"),
                               t["qmap"])
    elif op == "dequantize":
        out = backend.dequantize(t["input"], t["scale"], t.get("zero_point"), p.get("axes"), p.get("block_size"),
                                 t.get("input_qmap"), t.get("output_qmap"))
    elif op == "calculate_mx_qparam":
        out = backend.calculate_mx_qparam(t["input"], p["axes"], p["block_size"], p["quant_max"],
                                          p["force_scale_power_of_two"], t.get("scale_qmap"))
    elif op == "quantize_mx":
        out = backend.quantize_mx(t["input"], t["qmap"], p["axes"], p["block_size"], p["quant_max"],
                                  p["force_scale_power_of_two"], t.get("scale_qmap"))
    elif op == "linear_mx":
        out = backend.linear_mx(t["input"], t["weight"], t.get("bias"), input_scale=t.get("input_scale"),
                                weight_scale=t.get("weight_scale"), block_size=p["block_size"],
                                input_code=t.get("input_code"), weight_code=t.get("weight_code"),
                                weight_layout=p["weight_layout"])
    elif op == "matmul_mx":
        out = backend.matmul_mx(t["input"], t["other"], input_scale=t.get("input_scale"),
                                weight_scale=t.get("weight_scale"), block_size=p["block_size"],
                                input_code=t.get("input_code"), weight_code=t.get("weight_code"),
                                weight_layout=p["weight_layout"])
    elif op == "conv2d_mx":
        out = backend.conv2d_mx(t["input"], t["weight"], t.get("bias"), p["stride"], p["padding"], p["dilation"],
                                p["groups"], input_scale=t.get("input_scale"), weight_scale=t.get("weight_scale"),
                                block_size=p["block_size"], layout=p["layout"])
    else:
        raise ValueError(op)
    outs = list(out) if isinstance(out, (tuple, list)) else [out]
    return outs, expected
