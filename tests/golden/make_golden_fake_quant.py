"""Golden vectors for the observer + fake-quantize forward, produced by UPSTREAM's
``FusedAmaxObsFakeQuantize`` (quantization/fake_quantize.py) stepping on the CPU.

    python tests/golden/make_golden_fake_quant.py        # needs an upstream checkout

Output (committed): golden_fake_quant.npz + golden_fake_quant.json.  Per case: the constructor
arguments, and per step the input, the output and the module's ``scale`` (and ``amax_history``)
after the step, as raw bit patterns.
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


def main():
    ref = import_reference()
    fq, qspec = ref["fake_quantize"], ref["qspec"]
    Q = qspec.QScheme
    torch.manual_seed(77)
    torch.set_num_threads(1)
    arrays, cases = {}, []

    def run(name, shape, xdtype, steps, **kw):
        kw_json = {k: (v.value if isinstance(v, Q) else v) for k, v in kw.items()}
        m = fq.FusedAmaxObsFakeQuantize(**kw)
        entry = {"name": name, "kwargs": kw_json, "xdtype": str(xdtype).split(".")[-1], "shape": list(shape), "steps": steps}
        for t in range(steps):
            x = (torch.randn(shape) * (0.5 + t)).to(xdtype)
            if t == 1:
                x.view(-1)[3] = 0.0
            y = m(x)
            for key, val in (("x", x), ("y", y), ("scale", m.scale.detach().clone())):
                arr, tag = bits_of(val.float() if val.dtype not in (torch.float32, torch.bfloat16) else val)
                arrays[f"{name}/{t}/{key}"] = arr
                entry.setdefault("tags", {})[key] = tag
                entry.setdefault("shapes", {}).setdefault(key, []).append(list(val.shape))
            if m.amax_history.numel():
                arrays[f"{name}/{t}/history"] = bits_of(m.amax_history.detach().clone())[0]
                entry["history_shape"] = list(m.amax_history.shape)
        cases.append(entry)

    run("tensor_int8_f32", (6, 40), torch.float32, 4, dtype="int8", qscheme=Q.PER_TENSOR_SYMMETRIC, quant_max=127.0,
        amax_history_len=3)
    run("tensor_e4m3_bf16", (5, 33), torch.bfloat16, 3, dtype="fp8_e4m3", qscheme=Q.PER_TENSOR_SYMMETRIC, quant_max=448.0,
        amax_history_len=2)
    run("channel0_posit8_f32", (8, 3, 5, 5), torch.float32, 4, dtype="posit8_1", qscheme=Q.PER_CHANNEL_SYMMETRIC,
        quant_max=4096.0, amax_history_len=2, ch_axis=0)
    run("channel_last_int4_bf16", (7, 24), torch.bfloat16, 3, dtype="int4", qscheme=Q.PER_CHANNEL_SYMMETRIC,
        quant_max=7.0, amax_history_len=2, ch_axis=-1)
    run("channel1_nf4_f32", (2, 6, 4, 4), torch.float32, 3, dtype="nf4", qscheme=Q.PER_CHANNEL_SYMMETRIC,
        quant_max=1.0, amax_history_len=2, ch_axis=1)
    run("mx_int8_pow2_f32", (4, 96), torch.float32, 2, dtype="int8", qscheme=Q.MICROSCALING, quant_max=127.0,
        ch_axis=-1, block_size=32, force_scale_power_of_two=True)
    run("mx_nf4_bf16", (3, 128), torch.bfloat16, 2, dtype="nf4", qscheme=Q.MICROSCALING, quant_max=1.0,
        ch_axis=-1, block_size=64)
    run("mx_fp4_axis0_f32", (64, 5), torch.float32, 2, dtype="fp4_e2m1", qscheme=Q.MICROSCALING, quant_max=6.0,
        ch_axis=0, block_size=32, scale_dtype="fp8_e5m3")
    np.savez_compressed(os.path.join(HERE, "golden_fake_quant.npz"), **arrays)
    with open(os.path.join(HERE, "golden_fake_quant.json"), "w") as f:
        json.dump({"torch": torch.__version__, "cases": cases}, f, indent=1)
    print(len(cases), "cases,", len(arrays), "arrays")


if __name__ == "__main__":
    main()
