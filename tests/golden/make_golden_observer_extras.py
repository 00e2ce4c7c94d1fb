"""Golden vectors for the observer's optional steps -- the exponent histogram and outlier filtering --
produced by UPSTREAM's ``FusedAmaxObsFakeQuantize`` (quantization/fake_quantize.py:368-432) stepping on the CPU.

    python tests/golden/make_golden_observer_extras.py        # needs an upstream checkout

Output (committed): golden_observer_extras.npz + golden_observer_extras.json.  Per case: the constructor
arguments, and per step the input, the output, ``scale``, and where present ``histogram``,
``outlier_threshold`` and ``max_outlier_pct`` after the step (tensors as raw bit patterns).
"""
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _reference_import import import_reference  # noqa: E402
from make_golden import bits_of  # noqa: E402


def special_values(n, dtype, g):
    """Inputs that exercise the bin edges: powers of two, the patterns just below them (where the fp32
    logarithm rounds up), subnormals, zeros and infinities, mixed into normal data."""
    x = torch.randn(n, generator=g) * torch.exp2(torch.randint(-20, 20, (n,), generator=g).float())
    e = torch.randint(-126, 128, (n // 4,), generator=g)
    pow2 = torch.exp2(e.float())
    below = (pow2.view(torch.int32) - torch.randint(1, 60, (n // 4,), generator=g).int()).view(torch.float32)
    x[: n // 4] = pow2
    x[n // 4: n // 2] = below * (torch.randint(0, 2, (n // 4,), generator=g).float() * 2 - 1)
    x[n // 2: n // 2 + 8] = torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 1e-40, -3e-39, 1.17549421e-38, 3.4e38])
    return x.to(dtype)


def main():
    ref = import_reference()
    fq, qspec = ref["fake_quantize"], ref["qspec"]
    Q = qspec.QScheme
    g = torch.Generator().manual_seed(123)
    torch.set_num_threads(1)
    arrays, cases = {}, []

    def run(name, make_x, xdtype, steps, **kw):
        kw_json = {k: (v.value if isinstance(v, Q) else v) for k, v in kw.items()}
        m = fq.FusedAmaxObsFakeQuantize(**kw)
        entry = {"name": name, "kwargs": kw_json, "xdtype": str(xdtype).split(".")[-1], "steps": steps, "max_outlier_pct": []}
        for t in range(steps):
            x = make_x(t).to(xdtype)
            y = m(x)
            rec = [("x", x), ("y", y), ("scale", m.scale.detach().clone())]
            if kw.get("record_histogram"):
                rec.append(("histogram", m.histogram.detach().clone()))
            if kw.get("qscheme") == Q.GROUP_WISE_AFFINE:
                rec.append(("zero_point", m.zero_point.detach().clone()))
            if isinstance(m.outlier_threshold, torch.Tensor):
                rec.append(("outlier_threshold", m.outlier_threshold.detach().clone()))
            for key, val in rec:
                arr, tag = bits_of(val)
                arrays[f"{name}/{t}/{key}"] = arr
                entry.setdefault("tags", {})[key] = tag
                entry.setdefault("shapes", {}).setdefault(key, []).append(list(val.shape))
            entry["max_outlier_pct"].append(float(m.max_outlier_pct))
        cases.append(entry)

    run("hist_tensor_int8_f32", lambda t: special_values(4096, torch.float32, g).reshape(64, 64) * (1.0 + t), torch.float32, 3,
        dtype="int8", qscheme=Q.PER_TENSOR_SYMMETRIC, quant_max=127.0, amax_history_len=2, record_histogram=True)
    run("hist_mx_nf4_bf16", lambda t: special_values(4104, torch.float32, g)[:4096].reshape(32, 128), torch.bfloat16, 2,
        dtype="nf4", qscheme=Q.MICROSCALING, quant_max=1.0, ch_axis=-1, block_size=64, record_histogram=True)
    run("outlier_fixed_tensor_int8_f32", lambda t: torch.randn(37, 50, generator=g) * (1.0 + 0.5 * t), torch.float32, 3,
        dtype="int8", qscheme=Q.PER_TENSOR_SYMMETRIC, quant_max=127.0, amax_history_len=2, outlier_threshold=2.5)
    run("outlier_pct_channel_e4m3_bf16", lambda t: torch.randn(24, 33, generator=g) * (2.0 - 0.3 * t), torch.bfloat16, 4,
        dtype="fp8_e4m3", qscheme=Q.PER_CHANNEL_SYMMETRIC, quant_max=448.0, amax_history_len=2, ch_axis=0, outlier_pct=0.02)
    run("outlier_pct_mx_int8_f32", lambda t: torch.randn(16, 96, generator=g) * (1.0 + t), torch.float32, 3,
        dtype="int8", qscheme=Q.MICROSCALING, quant_max=127.0, ch_axis=-1, block_size=32, force_scale_power_of_two=True,
        outlier_pct=0.01, outlier_ema_decay=0.75)
    run("outlier_fixed_hist_bf16", lambda t: torch.randn(9, 130, generator=g) * 3.0, torch.bfloat16, 2,
        dtype="posit8_1", qscheme=Q.PER_TENSOR_SYMMETRIC, quant_max=4096.0, amax_history_len=3, outlier_threshold=4.3,
        record_histogram=True)
    def affine_input(shape, t):
        x = torch.randn(shape, generator=g) * (1.0 + t) + 0.3 * t
        x.view(-1)[:shape[-1] if len(shape) > 1 else 4] = 0.0          # a block without range
        if t == 1:
            x.view(-1)[-1] = float("nan")
        return x

    run("gwa_uint4_f32", lambda t: affine_input((6, 96), t), torch.float32, 2,
        dtype="int4", qscheme=Q.GROUP_WISE_AFFINE, quant_min=0.0, quant_max=15.0, ch_axis=-1, block_size=32)
    run("gwa_int8_ragged_bf16", lambda t: affine_input((5, 72), t), torch.bfloat16, 2,
        dtype="int8", qscheme=Q.GROUP_WISE_AFFINE, quant_min=-128.0, quant_max=127.0, ch_axis=-1, block_size=32)
    run("gwa_uint8_axis0_scale_e5m3_f32", lambda t: affine_input((64, 7), t), torch.float32, 2,
        dtype="int8", qscheme=Q.GROUP_WISE_AFFINE, quant_min=0.0, quant_max=255.0, ch_axis=0, block_size=16,
        scale_dtype="fp8_e5m3")
    run("gwa_int4_block8_bf16", lambda t: affine_input((3, 4, 40), t), torch.bfloat16, 2,
        dtype="int4", qscheme=Q.GROUP_WISE_AFFINE, quant_min=-8.0, quant_max=7.0, ch_axis=2, block_size=8)
    np.savez_compressed(os.path.join(HERE, "golden_observer_extras.npz"), **arrays)
    with open(os.path.join(HERE, "golden_observer_extras.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": cases}, f, indent=1)
    print(len(cases), "cases,", len(arrays), "arrays")


if __name__ == "__main__":
    main()
