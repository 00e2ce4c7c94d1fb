"""Per-row codebook quantization: oracle against vectors produced by upstream code (CPU), the
CUDA kernel against both (GPU)."""
import os
import sys

import numpy as np
import pytest
import torch

from golden_util import GOLDEN, from_bits

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

CASES = ["student_f32", "student_bf16", "ties_f32", "special_f32", "four_levels_bf16"]


def _case(name):
    z = np.load(os.path.join(GOLDEN, "golden_row_codebook.npz"))
    tag = "bf16" if name.endswith("bf16") else "f32"
    levels = torch.from_numpy(z[name + "/levels"].copy())
    x = from_bits(z[name + "/x"], tag)
    return x, levels, from_bits(z[name + "/values"], tag)


def _same_or_nan(a, b):
    a, b = a.float(), b.float()
    return bool(((a == b) | (torch.isnan(a) & torch.isnan(b))).all()) and \
        torch.equal(torch.signbit(a)[a == 0], torch.signbit(b)[b == 0])


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_upstream_vectors(name):
    x, levels, want = _case(name)
    idx, val = vo.row_codebook(x, levels, reference_rule=True)
    assert _same_or_nan(val, want)
    # the index names the FIRST level with that value's distance: never a later duplicate
    picked = torch.gather(levels, 1, idx.long())
    assert _same_or_nan(picked.to(torch.bfloat16).to(x.dtype), want)
    first = (levels.unsqueeze(1) == picked.unsqueeze(-1)).float().argmax(-1)
    assert torch.equal(first, idx.long())


def test_oracle_literal_rule_differs_only_by_the_bf16_roundings():
    x, levels, _ = _case("student_f32")
    i_ref, _ = vo.row_codebook(x, levels, True)
    i_lit, v_lit = vo.row_codebook(x, levels, False)
    assert torch.equal(v_lit, torch.gather(levels, 1, i_lit.long()))
    i_pre, _ = vo.row_codebook(x.to(torch.bfloat16).float(), levels, False)
    assert torch.equal(i_pre, i_ref)                     # same search once the input is pre-rounded
    assert (i_lit != i_ref).float().mean() < 0.05        # the two rules disagree on few elements


# ------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_kernel_matches_upstream_vectors(name):
    from voyager_compiler_b200 import codebook
    x, levels, want = _case(name)
    idx, val = codebook.row_codebook_quantize(x.cuda(), levels.cuda(), reference_rule=True, check_sorted=True)
    o_idx, o_val = vo.row_codebook(x, levels, True)
    assert _same_or_nan(val.cpu(), want)
    assert torch.equal(idx.cpu(), o_idx)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rule", [True, False], ids=["reference_rule", "fp32_rule"])
@pytest.mark.parametrize("shape,n", [((64, 4096), 16), ((33, 1000), 16), ((5, 37), 7), ((128, 512), 256), ((3, 8), 1)])
def test_kernel_matches_oracle(dtype, rule, shape, n):
    from voyager_compiler_b200 import codebook
    g = torch.Generator().manual_seed(hash((shape, n)) % 1000)
    x = (torch.distributions.StudentT(5.0).sample(shape) * 0.02).to(dtype)
    q = (2 * torch.arange(n, dtype=torch.float32) + 1) / (2 * n)
    levels = torch.quantile(x.float(), q, dim=-1).t().contiguous()
    if n >= 7:
        levels[0, 3] = levels[0, 2]                      # a duplicate level
    x.view(-1)[torch.randint(0, x.numel(), (4,), generator=g)] = float("nan")
    x.view(-1)[torch.randint(0, x.numel(), (4,), generator=g)] = float("inf")
    idx, val = codebook.row_codebook_quantize(x.cuda(), levels.cuda(), reference_rule=rule)
    o_idx, o_val = vo.row_codebook(x, levels, rule)
    assert torch.equal(idx.cpu(), o_idx)
    assert _same_or_nan(val.cpu(), o_val)
    only_idx, none = codebook.row_codebook_quantize(x.cuda(), levels.cuda(), reference_rule=rule, want_values=False)
    assert none is None and torch.equal(only_idx.cpu(), o_idx)


@pytest.mark.gpu
def test_full_size_properties_student_t_11008x4096():
    """The configuration's full size through size-independent properties: quantizing the returned
    levels again is the identity; indices are monotone in x within a row; every index names the
    nearest level (checked against torch on the device for the fp32 rule)."""
    from voyager_compiler_b200 import codebook
    torch.manual_seed(3)
    w = (torch.distributions.StudentT(5.0).sample((11008, 4096)) * 0.02).cuda()
    levels = codebook.row_quantile_levels(w, 16)
    idx, val = codebook.row_codebook_quantize(w, levels, reference_rule=False)
    idx2, val2 = codebook.row_codebook_quantize(val, levels, reference_rule=False)
    assert torch.equal(val2, val)
    assert torch.equal(torch.gather(levels, 1, idx.long()), val)
    order = torch.argsort(w, dim=-1)
    assert bool((torch.gather(idx, 1, order).diff(dim=-1).to(torch.int16) >= 0).all())
    rows = slice(0, 512)
    d = (torch.clamp(w[rows], levels[rows, :1], levels[rows, -1:]).unsqueeze(-1) - levels[rows].unsqueeze(1)).abs()
    assert torch.equal(d.argmin(-1).to(torch.uint8), idx[rows])
    counts = torch.bincount(idx.view(-1).long(), minlength=16).float() / idx.numel()
    assert float((counts - 1 / 16).abs().max()) < 0.01         # quantile codebook: equal occupancy


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,K,n", [(64, 4096, 16), (300, 1000, 16), (17, 37, 7), (5, 8192, 256), (9, 1, 4), (33, 2, 3), (12, 129, 16),
                                      (40, 8192, 16), (50, 2048, 8), (30, 1024, 16), (20, 5000, 3), (600, 4096, 16)])
def test_quantile_fit_matches_torch_cpu(dtype, rows, K, n):
    from voyager_compiler_b200 import codebook
    g = torch.Generator().manual_seed(rows * 7 + K)
    x = (torch.randn(rows, K, generator=g) * torch.exp(torch.randn(rows, 1, generator=g) * 3)).to(dtype)
    if K > 4:
        x[1, :3] = x[1, 3]                                   # repeated values
    if rows > 12 and K > 16:                                 # rows the binned selection cannot split, and ones it barely can
        x[3] = 0.375
        x[4, 0] = 1e30
        x[5, 7] = float("inf")
        x[6, 9] = float("-inf")
        x[7] = (x[7].float() * 4).round().to(dtype)
        x[8, :2] = torch.tensor([-3e38, 3e38]).to(dtype)
        x[9] = x[9].abs()
        x[10, 5] = 1e-3 * float(x[10].float().abs().max()) + 100 * float(x[10].float().abs().max())
        x[11, ::2] = 0.0
        x[11, 1::4] = -0.0
    q = (2 * torch.arange(n, dtype=torch.float32) + 1) / (2 * n)
    want = torch.quantile(x.float(), q, dim=-1).t().contiguous()
    got = codebook.row_quantile_levels(x.cuda(), n).cpu()
    assert torch.equal(got, want)
    if rows > 2 and K > 2:
        x[2, K // 2] = float("nan")
        got = codebook.row_quantile_levels(x.cuda(), n).cpu()
        assert bool(torch.isnan(got[2]).all()) and torch.equal(got[:2], want[:2])


def test_cpu_tensors_rejected():
    from voyager_compiler_b200 import codebook
    with pytest.raises(RuntimeError):
        codebook.row_codebook_quantize(torch.zeros(2, 8), torch.zeros(2, 4))
