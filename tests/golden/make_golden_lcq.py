"""Golden vectors for the LCQ statistics pass, produced by UPSTREAM's ``Histogram.add``, ``unit_scale`` and
``_accumulate`` (quantization/lcq.py) on the CPU.

    python tests/golden/make_golden_lcq.py        # needs an upstream checkout

Output (committed): golden_lcq.npz.  Per case: the tensor (raw patterns), the energy, the options and the
three fp64 moment arrays after one or two accumulations, stored sparsely (index + value of the non-zero bins).
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
    import_reference()
    lcq = importlib.import_module("voyager_compiler.quantization.lcq")
    torch.manual_seed(17)
    torch.set_num_threads(1)
    arrays, cases = {}, []

    def run(name, shapes, dtype, block, quant_max, quant_min, with_energy, heavy=False):
        hist = lcq.Histogram(quant_min, quant_max)
        module = types.SimpleNamespace(ch_axis=-1, block_size=block, quant_max=quant_max)
        energy = (torch.rand(shapes[0][-1]) * 2 + 0.01) if with_energy else None
        for i, shape in enumerate(shapes):
            x = torch.randn(shape)
            if heavy:
                x = x * torch.exp(torch.randn(shape))
            x = x.to(dtype)
            if i == 0:
                x.view(-1)[:block] = 0                          # an all-zero block: scale EPS / quant_max
            lcq._accumulate(x, module, energy, hist)
            arrays[f"{name}/x{i}"] = (x.view(torch.int16) if dtype == torch.bfloat16 else x.view(torch.int32)).numpy()
        if energy is not None:
            arrays[f"{name}/energy"] = energy.view(torch.int32).numpy()
        for key, m in (("weight", hist.weight), ("total", hist.total), ("square", hist.square)):
            nz = torch.nonzero(m).reshape(-1)
            arrays[f"{name}/{key}_idx"] = nz.numpy().astype(np.int32)
            arrays[f"{name}/{key}_val"] = m[nz].numpy()
        arrays[f"{name}/edges"] = torch.linspace(quant_min - 0.5, quant_max + 0.5, hist.bins + 1, dtype=torch.float32).view(torch.int32).numpy()
        cases.append(dict(name=name, shapes=[list(s) for s in shapes], dtype=str(dtype).split(".")[-1], block=block,
                          quant_max=quant_max, quant_min=quant_min, energy=with_energy, bins=hist.bins))

    run("nf4_like_f32_flat", [(16, 128)], torch.float32, 64, 7.0, -7.0, False)
    run("int8_bf16_energy_two_adds", [(4, 6, 96), (10, 96)], torch.bfloat16, 32, 127.0, -127.0, True)
    run("unsigned_f32_energy_heavy", [(32, 64)], torch.float32, 16, 15.0, 0.0, True, heavy=True)
    arrays["cases"] = np.frombuffer(json.dumps(cases).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "golden_lcq.npz"), **arrays)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
