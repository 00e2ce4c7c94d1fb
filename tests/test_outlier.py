"""Outlier side path (filter_outlier, quantize_mx_outlier, slice_csr_tensor, spmm_csr, linear_mx with
the sparse correction): oracle against vectors produced by upstream ops (CPU), CUDA kernels against
both (GPU)."""
import os
import sys

import numpy as np
import pytest
import torch

from golden_util import GOLDEN, from_bits, golden_table

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

_Z = None
SHAPES = {"f32_2d": ((48, 64), "f32"), "f32_overflow": ((48, 64), "f32"), "bf16_batched": ((2, 3, 16, 32), "bf16"),
          "f32_none": ((8, 16), "f32")}


def z(key):
    global _Z
    if _Z is None:
        _Z = np.load(os.path.join(GOLDEN, "golden_outlier.npz"))
    return _Z[key]


def ft(key, tag, shape=None):
    return from_bits(z(key), tag, shape)


def it(key):
    return torch.from_numpy(z(key).copy())


def same(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return a.shape == b.shape and bool(((a == b) | (torch.isnan(a) & torch.isnan(b))).all()) and \
        torch.equal(torch.signbit(a)[a == 0], torch.signbit(b)[b == 0])


def _filter_case(name):
    shape, tag = SHAPES[name]
    thr, pct = z(f"{name}/args")
    rows, cols = shape[-2:]
    nnz = int(rows * cols * pct)
    batch = tuple(shape[:-2])
    return (ft(f"{name}/x", tag, shape), float(thr), float(pct), ft(f"{name}/data", tag, batch + (nnz,)),
            it(f"{name}/indices").reshape(batch + (nnz,)), it(f"{name}/indptr").reshape(batch + (rows + 1,)),
            ft(f"{name}/inlier", tag, shape))


def _check_filter(got, want):
    d, i, p, inl = got
    wd, wi, wp, winl = want
    assert torch.equal(p.cpu().to(torch.int32), wp.to(torch.int32))
    assert torch.equal(i.cpu().to(torch.int32), wi.to(torch.int32))
    assert same(d, wd) and same(inl, winl)


@pytest.mark.parametrize("name", list(SHAPES))
def test_oracle_filter_matches_upstream(name):
    x, thr, pct, *want = _filter_case(name)
    _check_filter(vo.filter_outlier(x, thr, pct), want)


def _lin():
    X, W = ft("lin/X", "bf16", (32, 128)), ft("lin/W", "bf16", (24, 128))
    nnz = int(32 * 128 * 0.05)
    return dict(X=X, W=W, data=ft("lin/data", "bf16", (nnz,)), indices=it("lin/indices"), indptr=it("lin/indptr"),
                scale=ft("lin/scale", "bf16", (32, 4)), codes=ft("lin/codes", "bf16", (32, 128)), ws=ft("lin/ws", "bf16", (24, 4)),
                wq=ft("lin/wq", "bf16", (24, 128)), spmm=ft("lin/spmm", "bf16", (32, 24)), y=ft("lin/y", "bf16", (32, 24)),
                indptr7=it("lin/indptr_off7"))


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_oracle_quantize_mx_outlier_spmm_and_linear_match_upstream():
    L = _lin()
    q = golden_table("int8")
    d, i, p, s, c = vo.quantize_mx_outlier(L["X"], q, (-1,), 32, 127.0, True, None, 8.0, 0.05, 0)
    assert same(d, L["data"]) and torch.equal(i, L["indices"]) and torch.equal(p, L["indptr"])
    assert same(s, L["scale"]) and same(c, L["codes"])
    assert torch.equal(vo.quantize_mx_outlier(L["X"], q, (-1,), 32, 127.0, True, None, 8.0, 0.05, 7)[2], L["indptr7"])
    sp = vo.spmm_csr(d, i, p, L["wq"], L["ws"], None, 32, "kc")
    assert _rel(sp, L["spmm"]) < 1e-2           # fp32 accumulation order differs from torch.sparse.mm
    y = vo.linear_mx(c, L["wq"], None, input_scale=s, weight_scale=L["ws"], block_size=32) + sp
    assert _rel(y, L["y"]) < 1e-2


@pytest.mark.parametrize("dim,a,b", [(0, 4, 20), (1, 32, 96)])
def test_oracle_slice_csr_matches_upstream(dim, a, b):
    L = _lin()
    sd, si, sp = vo.slice_csr_tensor(L["data"], L["indices"], L["indptr"].clone(), dim, a, b, 1.0)
    assert same(sd, ft(f"slice{dim}/data", "bf16")) and torch.equal(si.to(torch.int32), it(f"slice{dim}/indices").to(torch.int32))
    assert torch.equal(sp.to(torch.int32), it(f"slice{dim}/indptr").to(torch.int32))


# ------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("name", list(SHAPES))
def test_kernel_filter_matches_upstream(name):
    from voyager_compiler_b200 import ops
    x, thr, pct, *want = _filter_case(name)
    _check_filter(ops.filter_outlier(x.cuda(), thr, pct), want)
    _check_filter(torch.ops.quantized_ops.filter_outlier(x.cuda(), thr, pct), want)     # through the dispatcher


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,thr,pct", [((4096, 1024), 3.0, 0.01), ((3, 257, 100), 2.5, 0.02), ((2, 2, 64, 33), 0.5, 0.9),
                                           ((1500, 7), 1.0, 0.5), ((5, 1, 8), 1.0, 0.3)])
def test_kernel_filter_matches_oracle(dtype, shape, thr, pct):
    from voyager_compiler_b200 import ops
    torch.manual_seed(sum(shape))
    x = torch.randn(shape).to(dtype)
    _check_filter(ops.filter_outlier(x.cuda(), thr, pct), vo.filter_outlier(x, thr, pct))


@pytest.mark.gpu
def test_kernel_quantize_mx_outlier_spmm_and_linear():
    from voyager_compiler_b200 import ops
    L = _lin()
    q = golden_table("int8").cuda()
    d, i, p, s, c = ops.quantize_mx_outlier(L["X"].cuda(), q, (-1,), 32, 127.0, True, None, None, 8.0, 0.05, 0)
    assert same(d, L["data"]) and torch.equal(i.cpu(), L["indices"]) and torch.equal(p.cpu(), L["indptr"])
    assert same(s, L["scale"]) and same(c, L["codes"])
    p7 = ops.quantize_mx_outlier(L["X"].cuda(), q, (-1,), 32, 127.0, True, None, None, 8.0, 0.05, 7)[2]
    assert torch.equal(p7.cpu(), L["indptr7"])
    sp = ops.spmm_csr(d, i, p, L["wq"].cuda(), L["ws"].cuda(), None, 32, "kc")
    assert _rel(sp, L["spmm"]) < 1e-2
    sp7 = ops.spmm_csr(d, i, p7, L["wq"].cuda(), L["ws"].cuda(), None, 32, "kc")       # row pointers that do not start at 0
    assert torch.equal(sp7, sp)
    y = ops.linear_mx(c, L["wq"].cuda(), None, input_scale=s, weight_scale=L["ws"].cuda(), block_size=32,
                      A_data=d, A_indices=i, A_indptr=p)
    assert _rel(y, L["y"]) < 1e-2


@pytest.mark.gpu
def test_matmul_mx_with_sparse_correction_batched():
    """Attention-like batched operands: right operand [K, N] with blocks along -2 ("ck")."""
    from voyager_compiler_b200 import ops
    torch.manual_seed(8)
    q = golden_table("int8")
    A = torch.randn(2, 3, 16, 64)
    A[torch.rand(2, 3, 16, 64) < 0.02] *= 30
    A = A.to(torch.bfloat16)
    B = torch.randn(2, 3, 64, 24).to(torch.bfloat16)
    d, i, p, s, c = vo.quantize_mx_outlier(A, q, (-1,), 32, 127.0, True, None, 8.0, 0.1, 0)
    bs, bq = vo.quantize_mx(B, q, (-2,), 32, 127.0, True)
    want = vo.matmul_mx(c, bq, input_scale=s, weight_scale=bs, block_size=32) + vo.spmm_csr(d, i, p, bq, bs, None, 32, "ck")
    got = ops.matmul_mx(c.cuda(), bq.cuda(), input_scale=s.cuda(), weight_scale=bs.cuda(), block_size=32,
                        A_data=d.cuda(), A_indices=i.cuda(), A_indptr=p.cuda())
    assert _rel(got, want) < 1e-2


@pytest.mark.gpu
def test_spmm_batched_and_ck_layout_against_oracle():
    from voyager_compiler_b200 import ops
    torch.manual_seed(3)
    x = torch.randn(2, 40, 96)
    x[torch.rand(2, 40, 96) < 0.03] *= 25
    d, i, p, _ = vo.filter_outlier(x, 10.0, 0.1)
    B = torch.randn(2, 96, 50)                                  # "ck": [K, N] per batch
    got = ops.spmm_csr(d.cuda(), i.cuda(), p.cuda(), B.cuda(), None, None, None, "ck")
    assert _rel(got, vo.spmm_csr(d, i, p, B, None, None, None, "ck")) < 1e-5
    Bs = torch.randn(70, 96)                                    # "kc": [N, K] shared by the batches
    got = ops.spmm_csr(d.cuda(), i.cuda(), p.cuda(), Bs.cuda(), None, None, None, "kc")
    assert _rel(got, vo.spmm_csr(d, i, p, Bs, None, None, None, "kc")) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dim,a,b", [(0, 4, 20), (1, 32, 96)])
def test_kernel_slice_csr_matches_upstream(dim, a, b):
    """The device-side slice (no host read-back) against upstream's vectors, op function and dispatcher."""
    from voyager_compiler_b200 import ops
    L = _lin()
    args = (L["data"].cuda(), L["indices"].cuda(), L["indptr"].cuda())
    for fn in (ops.slice_csr_tensor, torch.ops.quantized_ops.slice_csr_tensor):
        sd, si, sp = fn(*args, dim, a, b, 1.0)
        assert same(sd, ft(f"slice{dim}/data", "bf16")) and torch.equal(si.cpu(), it(f"slice{dim}/indices").to(torch.int32))
        assert torch.equal(sp.cpu(), it(f"slice{dim}/indptr").to(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols,pct,factor", [(64, 128, 0.05, 1.0), (300, 77, 0.2, 0.5), (1, 40, 0.5, 1.0), (2000, 64, 0.02, 0.25),
                                                  (17, 5000, 0.01, 2.0)])
def test_kernel_slice_csr_matches_oracle(dtype, rows, cols, pct, factor):
    """Random padded CSRs: empty rows, slices that keep nothing, and capacities smaller than what survives
    (surplus dropped, row pointers clamped)."""
    from voyager_compiler_b200 import ops
    g = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    x[rows // 2] = 0
    d, i, p, _ = vo.filter_outlier(x, 1.0, pct)
    for dim, a, b in ((0, 0, rows), (0, rows // 3, rows // 3), (0, rows // 4, rows - rows // 5), (1, 0, cols), (1, cols // 3, cols // 2),
                      (1, cols - 1, cols), (-1, 3, 4)):
        want = vo.slice_csr_tensor(d, i, p.clone(), dim, a, b, factor)
        got = ops.slice_csr_tensor(d.cuda(), i.cuda(), p.cuda(), dim, a, b, factor)
        assert same(got[0], want[0]), (dim, a, b)
        assert torch.equal(got[1].cpu(), want[1].to(torch.int32)) and torch.equal(got[2].cpu(), want[2].to(torch.int32)), (dim, a, b)
