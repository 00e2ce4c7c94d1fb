"""Golden vectors for the outlier side path, produced by UPSTREAM ops on the CPU
(``filter_outlier``, ``quantize_mx_outlier``, ``spmm_csr`` and ``linear_mx`` with the sparse
correction; ops/quantized.py:532-895).

    python tests/golden/make_golden_outlier.py        # needs an upstream checkout

Output (committed): golden_outlier.npz; float tensors as raw bit patterns, index arrays as int32.
"""
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _reference_import import import_reference  # noqa: E402
from make_golden import bits_of  # noqa: E402


def main():
    warnings.filterwarnings("ignore")
    ref = import_reference()
    Q = torch.ops.quantized_ops
    int8 = ref["fake_quantize"].get_quantization_map("int8")
    torch.manual_seed(21)
    out = {}

    def put(key, t):
        out[key] = t.numpy() if t.dtype in (torch.int32, torch.int64) else bits_of(t)[0]

    def filt(name, x, thr, pct):
        d, i, p, inl = Q.filter_outlier(x, thr, pct)
        for k, v in (("x", x), ("data", d), ("indices", i), ("indptr", p), ("inlier", inl)):
            put(f"{name}/{k}", v)
        out[f"{name}/args"] = np.asarray([thr, pct], dtype=np.float64)

    x = torch.randn(48, 64)
    x[torch.rand(48, 64) < 0.02] *= 20
    x[3, 5] = float("nan")
    x[0, 0] = -0.0
    filt("f32_2d", x, 6.0, 0.05)
    filt("f32_overflow", x, 1.5, 0.01)                       # more outliers than the CSR holds
    filt("bf16_batched", (torch.randn(2, 3, 16, 32) * 3).to(torch.bfloat16), 1.703, 0.2)   # threshold rounds in bf16
    filt("f32_none", torch.randn(8, 16) * 0.1, 5.0, 0.1)

    # quantize_mx_outlier + the linear with the sparse correction
    X = torch.randn(32, 128)
    X[torch.rand(32, 128) < 0.01] *= 30
    X = X.to(torch.bfloat16)
    W = (torch.randn(24, 128) * 0.1).to(torch.bfloat16)
    d, i, p, s, c = Q.quantize_mx_outlier(X, int8, (-1,), 32, 127.0, True, None, None, 8.0, 0.05, 0)
    ws, wq = Q.quantize_mx(W, int8, (-1,), 32, 127.0, True)
    for k, v in (("X", X), ("W", W), ("data", d), ("indices", i), ("indptr", p), ("scale", s), ("codes", c), ("ws", ws), ("wq", wq)):
        put(f"lin/{k}", v)
    put("lin/spmm", Q.spmm_csr(d, i, p, wq, ws, None, 32, "kc"))
    put("lin/y", Q.linear_mx(c, wq, None, input_scale=s, weight_scale=ws, block_size=32, A_data=d, A_indices=i, A_indptr=p))
    d2, i2, p2, s2, c2 = Q.quantize_mx_outlier(X, int8, (-1,), 32, 127.0, True, None, None, 8.0, 0.05, 7)
    put("lin/indptr_off7", p2)
    # slices of the CSR
    for dim, a, b in ((0, 4, 20), (1, 32, 96)):
        sd, si, sp = Q.slice_csr_tensor(d, i, p, dim, a, b, 1.0)
        put(f"slice{dim}/data", sd); put(f"slice{dim}/indices", si); put(f"slice{dim}/indptr", sp)
    np.savez_compressed(os.path.join(HERE, "golden_outlier.npz"), **out)
    print(len(out), "arrays")


if __name__ == "__main__":
    main()
