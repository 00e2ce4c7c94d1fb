"""Generate the golden fixtures in this directory by running the UPSTREAM voyager-compiler code.

Run once, where an upstream checkout is available (``$VOYAGER_REFERENCE``, or a ``reference``
directory next to this repository):

    python tests/golden/make_golden.py

Outputs (committed):
  golden_tables.npz   65 536-entry tables produced by upstream ``get_quantization_map`` /
                      ``codebook_qmap`` semantics, stored as uint16 bf16 bit patterns (or int64
                      index tables as uint8).
  golden_ops.npz      inputs and upstream outputs for small seeded op cases and edge cases.
  golden_ops.json     the manifest: op name, arguments, which arrays are inputs/outputs.

Float tensors are stored as raw bit patterns (uint32 for fp32, uint16 for bf16) so NaN payloads
and signed zeros survive.  The tests replay each case through the CPU oracle (CPU suite) and
through the CUDA ops (GPU suite) and compare with the stored upstream outputs.
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _reference_import import default_reference_root, import_reference  # noqa: E402

TABLE_DTYPES = [
    "int8", "int4", "int6", "int2", "uint8", "uint4", "e4m3", "e5m2", "posit8_1", "posit8_0",
    "posit8_2", "posit6_1", "nf4", "nf4_6", "nf3", "fp8_e5m3", "fp8_e4m3", "fp6_e3m2", "fp6_e2m3",
    "fp4_e2m1", "float16", "bfloat16", "posit16_1", "int16",
]


def bits_of(t: torch.Tensor):
    t = t.detach().contiguous()
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32), "f32"
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16), "bf16"
    if t.dtype == torch.int64:
        return t.numpy(), "i64"
    raise TypeError(t.dtype)


class Recorder:
    def __init__(self):
        self.arrays = {}
        self.cases = []

    def put(self, key, t):
        arr, tag = bits_of(t)
        self.arrays[key] = arr
        return {"key": key, "dtype": tag, "shape": list(t.shape)}

    def case(self, name, op, tensors, params, outputs):
        entry = {"name": name, "op": op, "tensors": {}, "params": params, "outputs": []}
        for arg, t in tensors.items():
            if t is None:
                continue
            if isinstance(t, str):          # a named table from golden_tables.npz
                entry["tensors"][arg] = {"table": t}
            else:
                entry["tensors"][arg] = self.put(f"{name}/{arg}", t)
        if isinstance(outputs, torch.Tensor):
            outputs = [outputs]
        for i, o in enumerate(outputs):
            entry["outputs"].append(self.put(f"{name}/out{i}", o))
        self.cases.append(entry)


def main():
    ref = import_reference()
    fq = ref["fake_quantize"]
    qops = torch.ops.quantized_ops
    torch.manual_seed(1234)
    torch.set_num_threads(1)  # scalar-tail vs vector-body position effects stay reproducible

    # ------------------------------------------------------------------ tables
    tables = {}
    tt = {}  # name -> torch table used by ops below
    for dt in TABLE_DTYPES:
        t = fq.get_quantization_map(dt)
        if isinstance(t, tuple):
            idx, lv = t
            tables[dt + "/indices"] = idx.numpy().astype(np.uint8)
            tables[dt + "/levels"] = bits_of(lv)[0]
            t = lv[idx]
        tables[dt] = bits_of(t)[0]
        tt[dt] = t
    # arbitrary codebooks through upstream lcq.codebook_qmap semantics.  lcq.py imports the
    # exporter stack, so its six-line function body is evaluated here from its source text.
    import ast
    src = open(os.path.join(default_reference_root(), "src/voyager_compiler/quantization/lcq.py")).read()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "codebook_qmap")
    ns = {"torch": torch}
    exec(compile(ast.Module([fn], []), "lcq_codebook_qmap", "exec"), ns)
    codebooks = {
        "cb4": [-3.0, -1.0, 1.0, 3.0],
        "cb16": sorted(torch.randn(16).mul(4).round().unique().tolist()),
        "cb7": [-7.0, -2.5, -1.0, 0.0, 0.75, 3.0, 6.0],
    }
    for name, entries in codebooks.items():
        t = ns["codebook_qmap"](entries)
        tables[name] = bits_of(t)[0]
        tables[name + "/entries"] = np.asarray(entries, dtype=np.float32)
        tt[name] = t
    np.savez_compressed(os.path.join(HERE, "golden_tables.npz"), **tables)

    # index-table conversion of quantize_pt2e.py:456-466 for codebook formats
    def idx_table(name):
        values = torch.unique(tt[name])
        return torch.searchsorted(values, tt[name]).to(torch.int64), values

    # ------------------------------------------------------------------ op cases
    R = Recorder()

    def outliers(shape, dtype=torch.float32, mul=1.0):
        x = torch.randn(shape) * mul
        m = torch.rand(shape) < 0.01
        x[m] *= 50
        return x.to(dtype)

    # vmap: every pattern, and random fp32 (double rounding through bf16)
    every = torch.arange(1 << 16, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    for dt in ["int8", "posit8_1", "nf4", "e4m3", "fp6_e3m2", "cb7"]:
        R.case(f"vmap_every_{dt}", "vmap", {"input": every, "qmap": dt}, {}, qops.vmap(every, tt[dt]))
    xf = outliers((37, 53), mul=20.0)
    R.case("vmap_f32_int8", "vmap", {"input": xf, "qmap": "int8"}, {}, qops.vmap(xf, tt["int8"]))
    R.case("vmap_f32_posit", "vmap", {"input": xf * 0.01, "qmap": "posit8_1"}, {}, qops.vmap(xf * 0.01, tt["posit8_1"]))
    xt = outliers((24, 40), mul=3.0).t()
    R.case("vmap_noncontig", "vmap", {"input": xt.contiguous(), "qmap": "int4"}, {"transpose_input": True},
           qops.vmap(xt, tt["int4"]))

    # quantize_mx / calculate_mx_qparam
    def mx_cases(tag, x, dt, axes, bs, qmax, pow2, scale_dt=None):
        sq = tt[scale_dt] if scale_dt else None
        s, q = qops.quantize_mx(x, tt[dt], axes, bs, qmax, pow2, sq)
        params = {"axes": list(axes), "block_size": bs, "quant_max": qmax, "force_scale_power_of_two": pow2}
        R.case(f"qmx_{tag}", "quantize_mx", {"input": x, "qmap": dt, "scale_qmap": scale_dt}, params, [s, q])
        s2 = qops.calculate_mx_qparam(x, axes, bs, qmax, pow2, sq)
        assert torch.equal(s2.view(torch.int32 if s2.dtype == torch.float32 else torch.int16),
                           s.view(torch.int32 if s.dtype == torch.float32 else torch.int16))
        R.case(f"mxs_{tag}", "calculate_mx_qparam", {"input": x, "scale_qmap": scale_dt}, params, s2)
        return s, q

    x1 = outliers((16, 96))
    mx_cases("f32_int8_pow2", x1, "int8", (-1,), 32, 127.0, True)
    mx_cases("f32_int8_amax", x1, "int8", (-1,), 32, 127.0, False)
    mx_cases("f32_int8_e5m3scale", x1, "int8", (-1,), 32, 127.0, False, "fp8_e5m3")
    mx_cases("f32_int4_bs16", x1 * 1e-3, "int4", (-1,), 16, 7.0, True)
    mx_cases("f32_e4m3_bs32", x1 * 1e4, "e4m3", (-1,), 32, 448.0, True)
    mx_cases("f32_fp4_bs32", x1, "fp4_e2m1", (-1,), 32, 6.0, True)
    xb = outliers((16, 128), torch.bfloat16)
    mx_cases("bf16_int8_pow2", xb, "int8", (-1,), 32, 127.0, True)
    mx_cases("bf16_int8_amax", xb, "int8", (-1,), 32, 127.0, False)
    wb = (torch.randn(24, 192) * 0.02).to(torch.bfloat16)
    mx_cases("bf16_nf4_bs64", wb, "nf4", (-1,), 64, 1.0, False)
    mx_cases("bf16_nf4_6_bs64_e5m3", wb, "nf4_6", (-1,), 64, 31.0, False, "fp8_e5m3")
    mx_cases("f32_ragged40", outliers((3, 40)), "int8", (-1,), 32, 127.0, True)
    mx_cases("f32_short8", outliers((5, 8)), "int8", (-1,), 32, 127.0, True)
    mx_cases("bf16_ragged72", outliers((4, 72), torch.bfloat16), "int8", (-1,), 32, 127.0, False)
    mx_cases("f32_axis0", outliers((80, 24)), "int8", (0,), 32, 127.0, True)
    mx_cases("f32_axis_m2_3d", outliers((2, 70, 12)), "int8", (-2,), 32, 127.0, True)
    mx_cases("bf16_axis1_4d", outliers((2, 40, 3, 5), torch.bfloat16), "int8", (1,), 16, 127.0, True)
    mx_cases("f32_two_axes", outliers((48, 64)), "int8", (-2, -1), 8, 127.0, True)
    mx_cases("f32_posit_bs32", x1, "posit8_1", (-1,), 32, 4096.0, True)
    # edge blocks (one block per row)
    e = torch.zeros(10, 32)
    e[0, 3] = float("nan"); e[0, 5] = 2.0
    e[1, 7] = float("inf"); e[1, 8] = -3.0
    e[2] = 0.0
    e[3] = 1e-42
    e[4] = 3.0e38
    e[5, 0] = -0.0; e[5, 1] = 127.5 / 128; e[5, 2] = -127.5 / 128; e[5, 3] = 1.0
    e[6, :] = torch.linspace(-2, 2, 32); e[6, 4] = float("-inf")
    e[7, 0] = 1.4e-45
    e[8, :] = torch.tensor(7.9999995)
    e[9, 0] = 1.1754942e-38; e[9, 1] = -5e-39
    mx_cases("f32_edges_pow2", e, "int8", (-1,), 32, 127.0, True)
    mx_cases("f32_edges_amax", e, "int8", (-1,), 32, 127.0, False)
    mx_cases("bf16_edges_pow2", e.to(torch.bfloat16), "int8", (-1,), 32, 127.0, True)
    mx_cases("bf16_edges_amax", e.to(torch.bfloat16), "nf4", (-1,), 32, 1.0, False)

    # shared exponent sweep: every positive bf16 amax, and fp32 values hugging each power of two
    pos = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    sweep_b = torch.stack([pos, torch.zeros_like(pos)], dim=1)
    R.case("mxs_sweep_bf16", "calculate_mx_qparam", {"input": sweep_b},
           {"axes": [-1], "block_size": 2, "quant_max": 127.0, "force_scale_power_of_two": True},
           qops.calculate_mx_qparam(sweep_b, (-1,), 2, 127.0, True))
    R.case("mxs_sweep_bf16_q1", "calculate_mx_qparam", {"input": sweep_b},
           {"axes": [-1], "block_size": 2, "quant_max": 1.0, "force_scale_power_of_two": True},
           qops.calculate_mx_qparam(sweep_b, (-1,), 2, 1.0, True))
    pats = []
    for ex in range(0, 255):
        base = (ex + 1) << 23
        pats += list(range(base - 50, base)) + [ex << 23 if ex else 1, (ex << 23) + 12345]
    sweep_f = torch.tensor(pats, dtype=torch.int64).clamp(min=1).to(torch.int32).view(torch.float32)
    sweep_f = torch.stack([sweep_f, -sweep_f * 0.5], dim=1)
    R.case("mxs_sweep_f32", "calculate_mx_qparam", {"input": sweep_f},
           {"axes": [-1], "block_size": 2, "quant_max": 127.0, "force_scale_power_of_two": True},
           qops.calculate_mx_qparam(sweep_f, (-1,), 2, 127.0, True))
    R.case("mxs_sweep_f32_q448", "calculate_mx_qparam", {"input": sweep_f},
           {"axes": [-1], "block_size": 2, "quant_max": 448.0, "force_scale_power_of_two": True},
           qops.calculate_mx_qparam(sweep_f, (-1,), 2, 448.0, True))

    # quantize / dequantize
    def q_case(tag, x, scale, dt, zp=None, axes=None, bs=None, index=False):
        if index:
            tab, _ = idx_table(dt)
            key = {"key_table": dt}
            out = qops.quantize(x, scale, zp, axes, bs, tab)
            R.case(f"q_{tag}", "quantize", {"input": x, "scale": scale, "zero_point": zp},
                   {"axes": axes, "block_size": bs, "index_table_of": dt}, out)
        else:
            out = qops.quantize(x, scale, zp, axes, bs, tt[dt])
            R.case(f"q_{tag}", "quantize", {"input": x, "scale": scale, "zero_point": zp, "qmap": dt},
                   {"axes": axes, "block_size": bs}, out)
        return out

    def dq_case(tag, x, scale, zp=None, axes=None, bs=None, in_dt=None, out_dt=None):
        out = qops.dequantize(x, scale, zp, axes, bs, tt[in_dt] if in_dt else None, tt[out_dt] if out_dt else None)
        R.case(f"dq_{tag}", "dequantize",
               {"input": x, "scale": scale, "zero_point": zp, "input_qmap": in_dt, "output_qmap": out_dt},
               {"axes": axes, "block_size": bs}, out)
        return out

    w4 = torch.empty(8, 4, 3, 3); torch.nn.init.kaiming_normal_(w4, mode="fan_in")
    s4 = w4.abs().amax(dim=(1, 2, 3), keepdim=True) / 4096.0
    q4 = q_case("perchannel_posit_f32", w4, s4, "posit8_1")
    dq_case("perchannel_posit_f32", q4, s4)
    w2 = torch.randn(12, 20)
    s2 = w2.abs().amax(dim=1, keepdim=True) / 127.0
    q_case("perrow_int8_f32", w2, s2, "int8")
    s2c = w2.abs().amax(dim=0, keepdim=True) / 127.0
    q_case("percol_int8_f32", w2, s2c, "int8")
    st = torch.tensor([0.037])
    qa = q_case("pertensor_e4m3_f32", x1, st, "e4m3")
    dq_case("pertensor_e4m3_f32", qa, st)
    q_case("pertensor0d_int8_f32", x1, torch.tensor(0.05), "int8")
    xb2 = outliers((9, 33), torch.bfloat16)
    sb = torch.tensor([0.0213], dtype=torch.bfloat16)
    qb = q_case("pertensor_int8_bf16", xb2, sb, "int8")
    dq_case("pertensor_int8_bf16", qb, sb)
    q_case("bf16_in_f32_scale", xb2, torch.tensor([0.0213]), "int8")
    q_case("f32_in_bf16_scale", x1, sb, "int8")
    # block scale + index table (nf4) as convert_pt2e does for weights
    sw = qops.calculate_mx_qparam(wb, (-1,), 64, 1.0, False)
    qi = q_case("block_nf4_index_bf16", wb, sw, "nf4", axes=(-1,), bs=64, index=True)
    q_case("block_nf4_value_bf16", wb, sw, "nf4", axes=(-1,), bs=64)
    # group-wise affine: uint4 with zero point, block along last axis, ragged
    xg = torch.randn(6, 50) * 2 + 1
    lo = torch.stack([xg[:, i:i + 16].amin(1) for i in range(0, 50, 16)], 1)
    hi = torch.stack([xg[:, i:i + 16].amax(1) for i in range(0, 50, 16)], 1)
    sg = (hi - lo) / 15.0
    zg = torch.round(-lo / sg)
    qg = q_case("groupwise_uint4_zp", xg, sg, "uint4", zp=zg, axes=(-1,), bs=16)
    dq_case("groupwise_uint4_zp", qg, sg, zp=zg, axes=(-1,), bs=16)
    # block scale along axis 0 and on two axes
    s_ax0 = qops.calculate_mx_qparam(w2, (0,), 4, 127.0, True)
    q_case("block_axis0", w2, s_ax0, "int8", axes=(0,), bs=4)
    s_2ax = qops.calculate_mx_qparam(w2, (0, 1), 4, 127.0, True)
    q_case("block_two_axes", w2, s_2ax, "int8", axes=(0, 1), bs=4)
    # dequantize with tables (accumulator re-quantisation and fused dq->q, quant_folding.py:1121-1178)
    acc = torch.round(torch.randn(10, 30) * 3000)
    dq_case("acc_int24_in", acc, torch.tensor([1.7e-4]), in_dt="int16")
    dq_case("requant_out_int8", acc, torch.tensor([0.013]), out_dt="int8")
    dq_case("requant_out_posit_zp", acc, torch.tensor([0.0011]), zp=torch.tensor([3.0]), out_dt="posit8_1")
    dq_case("block_bf16", qb[:, :32], torch.rand(9, 2).add(0.5).to(torch.bfloat16), axes=(-1,), bs=16)
    qe = qops.quantize_mx(e, tt["int8"], (-1,), 32, 127.0, True)
    dq_case("edges_block", qe[1], qe[0], axes=(-1,), bs=32)

    # linear_mx / matmul_mx (small)
    X = outliers((32, 64), torch.bfloat16)
    W = (torch.randn(48, 64) * 0.02).to(torch.bfloat16)
    xs, xq = qops.quantize_mx(X, tt["int8"], (-1,), 32, 127.0, True)
    ws = qops.calculate_mx_qparam(W, (-1,), 32, 127.0, True)
    wq = qops.quantize(W, ws, None, (-1,), 32, tt["int8"])
    bias = torch.randn(48).to(torch.bfloat16)
    lin_p = {"block_size": 32, "weight_layout": "kc"}
    R.case("lin_int8_bf16", "linear_mx", {"input": xq, "weight": wq, "input_scale": xs, "weight_scale": ws}, lin_p,
           qops.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32))
    R.case("lin_int8_bf16_bias", "linear_mx",
           {"input": xq, "weight": wq, "bias": bias, "input_scale": xs, "weight_scale": ws}, lin_p,
           qops.linear_mx(xq, wq, bias, input_scale=xs, weight_scale=ws, block_size=32))
    wq_ck, ws_ck = wq.t().contiguous(), ws.t().contiguous()
    R.case("lin_int8_bf16_ck", "linear_mx", {"input": xq, "weight": wq_ck, "input_scale": xs, "weight_scale": ws_ck},
           {"block_size": 32, "weight_layout": "ck"},
           qops.linear_mx(xq, wq_ck, None, input_scale=xs, weight_scale=ws_ck, block_size=32, weight_layout="ck"))
    # nf4 index weights with code table, fp32 activations un-quantised
    tab_i, levels = idx_table("nf4")
    ws4 = qops.calculate_mx_qparam(W, (-1,), 32, 1.0, False)
    wq4 = qops.quantize(W, ws4, None, (-1,), 32, tab_i)
    R.case("lin_nf4_code", "linear_mx",
           {"input": xq, "weight": wq4, "input_scale": xs, "weight_scale": ws4, "weight_code": levels}, lin_p,
           qops.linear_mx(xq, wq4, None, input_scale=xs, weight_scale=ws4, block_size=32, weight_code=levels))
    Xf = X.float()
    xsf, xqf = qops.quantize_mx(Xf, tt["int8"], (-1,), 32, 127.0, True)
    wsf = qops.calculate_mx_qparam(W.float(), (-1,), 32, 127.0, True)
    wqf = qops.quantize(W.float(), wsf, None, (-1,), 32, tt["int8"])
    R.case("lin_int8_f32", "linear_mx", {"input": xqf, "weight": wqf, "input_scale": xsf, "weight_scale": wsf}, lin_p,
           qops.linear_mx(xqf, wqf, None, input_scale=xsf, weight_scale=wsf, block_size=32))
    # matmul_mx: batched attention-like, right operand [K, N] with blocks along -2
    A = outliers((2, 3, 16, 64), torch.bfloat16)
    B = outliers((2, 3, 64, 24), torch.bfloat16)
    as_, aq = qops.quantize_mx(A, tt["int8"], (-1,), 32, 127.0, True)
    bs_, bq = qops.quantize_mx(B, tt["int8"], (-2,), 32, 127.0, True)
    R.case("mm_int8_bf16", "matmul_mx", {"input": aq, "other": bq, "input_scale": as_, "weight_scale": bs_},
           {"block_size": 32, "weight_layout": "ck"},
           qops.matmul_mx(aq, bq, input_scale=as_, weight_scale=bs_, block_size=32))

    # conv2d_mx: blocks along the channel axis (ax=1 for NCHW, last axis for NHWC / HWIO)
    xc = outliers((2, 32, 9, 9), torch.bfloat16)
    wc = (torch.randn(24, 32, 3, 3) * 0.1).to(torch.bfloat16)
    bc = torch.randn(24).to(torch.bfloat16)
    xcs, xcq = qops.quantize_mx(xc, tt["int8"], (1,), 16, 127.0, True)
    wcs, wcq = qops.quantize_mx(wc, tt["int8"], (1,), 16, 127.0, True)
    for tag, bias_t, stride, pad in (("basic", None, [1, 1], [1, 1]), ("bias_s2", bc, [2, 2], [0, 0])):
        R.case(f"conv_nchw_{tag}", "conv2d_mx",
               {"input": xcq, "weight": wcq, "bias": bias_t, "input_scale": xcs, "weight_scale": wcs},
               {"stride": stride, "padding": pad, "dilation": [1, 1], "groups": 1, "block_size": 16, "layout": "nchw"},
               qops.conv2d_mx(xcq, wcq, bias_t, stride, pad, [1, 1], 1, input_scale=xcs, weight_scale=wcs, block_size=16))
    xh = xc.permute(0, 2, 3, 1).contiguous()
    wh = wc.permute(2, 3, 1, 0).contiguous()                       # HWIO
    xhs, xhq = qops.quantize_mx(xh, tt["int8"], (-1,), 16, 127.0, True)
    whs, whq = qops.quantize_mx(wh, tt["int8"], (2,), 16, 127.0, True)
    R.case("conv_nhwc", "conv2d_mx", {"input": xhq, "weight": whq, "bias": bc, "input_scale": xhs, "weight_scale": whs},
           {"stride": [1, 1], "padding": [1, 1], "dilation": [1, 1], "groups": 1, "block_size": 16, "layout": "nhwc"},
           qops.conv2d_mx(xhq, whq, bc, [1, 1], [1, 1], [1, 1], 1, input_scale=xhs, weight_scale=whs, block_size=16,
                          layout="nhwc"))

    np.savez_compressed(os.path.join(HERE, "golden_ops.npz"), **R.arrays)
    with open(os.path.join(HERE, "golden_ops.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": R.cases}, f, indent=1)
    print(f"{len(tables)} table arrays, {len(R.cases)} op cases")


if __name__ == "__main__":
    main()
