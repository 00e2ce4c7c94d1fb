"""Golden vectors for the per-row codebook rule, produced by UPSTREAM code: for every row the
upstream ``codebook_qmap`` (quantization/lcq.py) builds the 65 536-entry table of that row's
levels and the upstream ``vmap`` op applies it to the row.

    python tests/golden/make_golden_row_codebook.py      # needs an upstream checkout

Output (committed): golden_row_codebook.npz with, per case, ``x`` (fp32 or bf16 bit patterns),
``levels`` (fp32) and ``values`` (upstream result, bit patterns in the dtype of x).
"""
import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _reference_import import default_reference_root, import_reference  # noqa: E402
from make_golden import bits_of  # noqa: E402


def main():
    import_reference()
    vmap = torch.ops.quantized_ops.vmap
    src = open(os.path.join(default_reference_root(), "src/voyager_compiler/quantization/lcq.py")).read()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "codebook_qmap")
    ns = {"torch": torch}
    exec(compile(ast.Module([fn], []), "lcq_codebook_qmap", "exec"), ns)
    codebook_qmap = ns["codebook_qmap"]

    torch.manual_seed(3)
    out = {}

    def case(name, x, levels):
        rows = [vmap(x[r], codebook_qmap(levels[r].tolist())) for r in range(x.shape[0])]
        out[name + "/x"] = bits_of(x)[0]
        out[name + "/levels"] = levels.numpy()
        out[name + "/values"] = bits_of(torch.stack(rows))[0]

    q = (2 * torch.arange(16, dtype=torch.float32) + 1) / 32
    # Student-t rows with their own 16 quantiles (the per-channel codebook configuration)
    w = torch.distributions.StudentT(5.0).sample((12, 256)) * 0.02
    lv = torch.quantile(w, q, dim=-1).t().contiguous()
    case("student_f32", w, lv)
    case("student_bf16", w.to(torch.bfloat16), lv)
    # rows with few distinct values: duplicate levels, exact ties between neighbours
    t = torch.randint(-3, 4, (6, 128)).float() * 0.5
    case("ties_f32", t, torch.quantile(t, q, dim=-1).t().contiguous())
    # specials: NaN, +-Inf, zeros, values far outside the codebook, 4- and 7-level codebooks
    s = torch.randn(4, 64)
    s[0, :6] = torch.tensor([float("nan"), float("inf"), float("-inf"), 0.0, -0.0, 1e30])
    s[1, :3] = torch.tensor([1e-40, -1e-40, 3.0])
    case("special_f32", s, torch.sort(torch.randn(4, 7), dim=-1).values)
    case("four_levels_bf16", s.to(torch.bfloat16), torch.tensor([[-3.0, -1.0, 1.0, 3.0]] * 4))
    np.savez_compressed(os.path.join(HERE, "golden_row_codebook.npz"), **out)
    print(sorted(out))


if __name__ == "__main__":
    main()
