"""Golden vectors for the GPTQ weight compensation, produced by UPSTREAM's ``compensate_weight``,
``hessian_inverse_chol`` and ``block_scale`` (quantization/gptq.py) on the CPU.

    python tests/golden/make_golden_gptq.py        # needs an upstream checkout

Output (committed): golden_gptq.npz.  Per case: weight, Hessian, token count, the tables (as 65 536 raw
bf16 patterns), the options, upstream's inverse factor and its compensated weight (raw fp32 patterns).
"""
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def main():
    import transformers  # noqa: F401  (must come before the torchao stand-in)
    from transformers import PreTrainedModel  # noqa: F401
    from _reference_import import import_reference
    import importlib
    ref = import_reference()
    gptq = importlib.import_module("voyager_compiler.quantization.gptq")
    fq = ref["fake_quantize"]
    torch.manual_seed(91)
    torch.set_num_threads(1)
    arrays, cases = {}, []

    def table(name):
        if name is None:
            return None
        t = fq.get_quantization_map(name)
        if isinstance(t, tuple):                                 # codebook types: index table + values, as the module's
            idx, vals = t                                        # constructor folds them (fake_quantize.py:273-278)
            t = vals[idx]
        return t

    def run(name, O, K, tokens, dtype, scale_dtype, quant_max, block, damping, act_order, within_block, shrink, outlier=False):
        w = torch.randn(O, K) * 0.05
        if outlier:
            w[torch.rand(O, K) < 0.02] *= 6
        x = torch.randn(tokens, K) * (0.2 + 2 * torch.rand(K))
        h = x.t() @ x
        fake = types.SimpleNamespace(qmap=table(dtype), scale_qmap=table(scale_dtype), quant_max=quant_max, block_size=block,
                                     ch_axis=-1)
        out = gptq.compensate_weight(w, h.clone(), tokens, fake, damping, act_order=act_order, within_block=within_block,
                                     shrink=shrink)
        perm = gptq.salience_order(h, K, within_block, block) if act_order else None
        hp = h if perm is None else h[perm][:, perm]
        hinv = gptq.hessian_inverse_chol(hp.clone(), tokens, damping)
        for key, val in (("weight", w), ("hessian", h), ("hinv", hinv), ("out", out)):
            arrays[f"{name}/{key}"] = val.contiguous().view(torch.int32).numpy()
        arrays[f"{name}/qmap"] = fake.qmap.view(torch.int16).numpy()
        if fake.scale_qmap is not None:
            arrays[f"{name}/scale_qmap"] = fake.scale_qmap.view(torch.int16).numpy()
        cases.append(dict(name=name, O=O, K=K, tokens=tokens, dtype=dtype, scale_dtype=scale_dtype, quant_max=quant_max,
                          block=block, damping=damping, act_order=act_order, within_block=within_block, shrink=shrink))

    run("nf4_b32_plain", 24, 96, 256, "nf4", None, 1.0, 32, 0.01, False, False, False)
    run("int4_b64_e4m3_ordered", 40, 128, 300, "int4", "fp8_e4m3", 7.0, 64, 0.01, True, True, False)
    run("nf4_b32_shrink", 32, 64, 200, "nf4", "fp8_e4m3", 1.0, 32, 0.05, True, False, True, outlier=True)
    run("int8_b32_ragged", 16, 80, 128, "int8", None, 127.0, 32, 0.01, True, True, False)
    run("posit8_b64_rank_deficient", 12, 128, 40, "posit8_1", None, 4096.0, 64, 0.01, False, False, False)
    arrays["cases"] = np.frombuffer(json.dumps(cases).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "golden_gptq.npz"), **arrays)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
