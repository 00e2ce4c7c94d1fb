"""LCQ statistics pass (quantization/lcq.py: unit_scale, Histogram.add, _accumulate): the oracle against
vectors upstream produced (CPU), the fused CUDA pass against the oracle (GPU)."""
import json
import os
import sys

import numpy as np
import pytest
import torch

from golden_util import GOLDEN

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

_Z = None


def _z():
    global _Z
    if _Z is None:
        _Z = np.load(os.path.join(GOLDEN, "golden_lcq.npz"))
    return _Z


CASES = json.loads(bytes(_z()["cases"]).decode())


def _inputs(case):
    n = case["name"]
    dt = torch.bfloat16 if case["dtype"] == "bfloat16" else torch.float32
    xs = [torch.from_numpy(_z()[f"{n}/x{i}"].copy()).view(dt).reshape(s) for i, s in enumerate(case["shapes"])]
    energy = torch.from_numpy(_z()[f"{n}/energy"].copy()).view(torch.float32) if case["energy"] else None
    return xs, energy


def _dense(case, key):
    n = case["name"]
    m = torch.zeros(case["bins"], dtype=torch.float64)
    m[torch.from_numpy(_z()[f"{n}/{key}_idx"].astype(np.int64))] = torch.from_numpy(_z()[f"{n}/{key}_val"].copy())
    return m


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_upstream(case):
    torch.set_num_threads(1)
    xs, energy = _inputs(case)
    assert torch.equal(vo.lcq_edges(case["quant_min"], case["quant_max"], case["bins"]).view(torch.int32),
                       torch.from_numpy(_z()[f"{case['name']}/edges"].copy()))
    m = None
    for x in xs:
        m = vo.lcq_accumulate(m, x, case["block"], case["quant_max"], case["quant_min"], energy, case["bins"])
    for got, key in zip(m, ("weight", "total", "square")):
        assert torch.equal(got, _dense(case, key)), key


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_cuda_pass_matches_upstream(case):
    """Bins are exact (the same fp32 quotient against the same boundaries): with unit weights the weight
    moment is a count and must be equal; the fp64 sums depend on the order of addition only in their last bits."""
    from voyager_compiler_b200 import lcq
    xs, energy = _inputs(case)
    h = lcq.Histogram(case["quant_min"], case["quant_max"], case["bins"])
    for x in xs:
        h.accumulate(x.cuda(), case["block"], case["quant_max"], energy.cuda() if energy is not None else None)
    want = [_dense(case, k) for k in ("weight", "total", "square")]
    got = [h.weight.cpu(), h.total.cpu(), h.square.cpu()]
    assert torch.equal(got[0] != 0, want[0] != 0)                  # the same bins are hit
    if not case["energy"]:
        assert torch.equal(got[0], want[0])
    for g, w in zip(got, want):
        assert torch.allclose(g, w, rtol=1e-12, atol=1e-9 * float(w.abs().max()))
    cw, ct, cs = h.cumulative()
    assert cw.shape == (case["bins"] + 1,) and cw[0] == 0 and abs(cw[-1] - float(want[0].sum())) <= 1e-9 * float(want[0].sum())


@pytest.mark.gpu
def test_add_of_normalised_values_and_large_input():
    from voyager_compiler_b200 import lcq
    g = torch.Generator().manual_seed(3)
    v = (torch.randn(1 << 20, generator=g) * 3).clamp_(-9, 9)
    v[:7] = torch.tensor([-7.5, 7.5, -7.4999995, 7.4999995, 0.0, float("inf"), -float("inf")])
    w = torch.rand(1 << 20, generator=g)
    want = vo.lcq_histogram_add(None, v, w, -7.0, 7.0)
    h = lcq.Histogram(-7.0, 7.0)
    h.add(v.cuda(), w.cuda())
    assert torch.equal(h.weight.cpu() != 0, want[0] != 0)
    for gq, wq in zip((h.weight, h.total, h.square), want):
        fin = torch.isfinite(wq)
        assert torch.equal(torch.isfinite(gq.cpu()), fin)
        assert torch.allclose(gq.cpu()[fin], wq[fin], rtol=1e-11, atol=1e-9)
    ones = lcq.Histogram(-7.0, 7.0)
    ones.add(v.cuda(), torch.ones((), device="cuda"))
    cnt = vo.lcq_histogram_add(None, v, torch.ones(()), -7.0, 7.0)[0]
    assert torch.equal(ones.weight.cpu(), cnt)                     # counts are exact in any order


def test_cpu_tensors_rejected():
    from voyager_compiler_b200 import lcq
    with pytest.raises(RuntimeError):
        lcq.Histogram(-7.0, 7.0).add(torch.zeros(8), torch.ones(8))


@pytest.mark.gpu
@pytest.mark.parametrize("entries", [
    [-7.0, -5.0, -3.0, -2.0, -1.0, 0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 7.0],
    [0.0],
    [3.0, -1.0, 2.0, 2.0, -6.0, 0.5, 0.5],                     # unsorted, repeated entries: the first of equal distances
    [-0.0, 0.0, 1e-40, 1.0, 3.3895e38],                        # signed zeros, a subnormal, the largest bf16
    [float("-inf"), -1.0, 1.0, float("inf")],
    [-1.0, float("nan"), 1.0],                                 # a NaN entry poisons min / max: every pattern takes it
    "random16", "random256",
])
def test_codebook_qmap_on_the_device_is_upstreams_table(entries):
    """``lcq.codebook_qmap`` (one kernel) against upstream's tensor expression (lcq.py:270-291) evaluated by torch on
    the CPU, for all 65 536 patterns, bit for bit (NaN == NaN); entries given as a list and as a device tensor."""
    from voyager_compiler_b200 import lcq
    if isinstance(entries, str):
        g = torch.Generator().manual_seed(len(entries))
        entries = (torch.randn(int(entries[6:]), generator=g) * 4).tolist()
    cb = torch.tensor(entries, dtype=torch.float32)
    every = torch.arange(2 ** 16, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).float()
    index = (every.clamp(cb.min(), cb.max()).unsqueeze(-1) - cb).abs().argmin(-1)
    want = cb[index].to(torch.bfloat16).view(torch.int16)
    for given in (entries, cb.cuda()):
        got = lcq.codebook_qmap(given, "cuda")
        assert got.dtype == torch.bfloat16 and got.shape == (65536,) and got.is_cuda
        g16 = got.cpu().view(torch.int16)
        same = (g16 == want) | (torch.isnan(got.cpu().float()) & torch.isnan(want.view(torch.bfloat16).float()))
        assert bool(same.all()), int((~same).sum())


def test_codebook_qmap_rejects_cpu_devices():
    from voyager_compiler_b200 import lcq
    with pytest.raises(RuntimeError):
        lcq.codebook_qmap([0.0, 1.0], "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block,channels,energy_len", [(4, 64, 64), (8, 96, 0), (64, 1024, 1024), (128, 384, 384), (64, 192, 192),
                                                      (24, 96, 96), (256, 512, 0), (64, 192, 1)])
def test_statistics_pass_for_block_sizes_and_weight_layouts(dtype, block, channels, energy_len):
    """Blocks of 4 ... 128 elements go to the kernel in which a group of lanes takes a block (weights read four at a time
    when the channel count allows), other sizes and unaligned tensors to the one in which a thread takes a block; both
    against the oracle: the same bins hit, equal counts without weights, fp64 sums equal up to the order of addition.
    Includes an all-zero block, a NaN and huge values."""
    from voyager_compiler_b200 import lcq
    g = torch.Generator().manual_seed(block * 1000 + channels)
    x = torch.randn(768, channels, generator=g) * torch.logspace(-2, 2, 768).unsqueeze(1)    # 768 and 640 rows: whole blocks
    x[3] = 0.0
    x[5, 7] = 3e38
    x = x.to(dtype)
    energy = None if energy_len == 0 else torch.rand(energy_len, generator=g) + 0.1
    for xs in (x, x.reshape(-1)[block:block + 640 * channels].reshape(640, channels)):   # the second starts `block` elements in
        want = vo.lcq_accumulate(None, xs, block, 7.0, -7.0, energy, 4001)
        h = lcq.Histogram(-7.0, 7.0)
        e_dev = None if energy is None else energy.cuda()
        if energy_len == 192:                                # weights that do not start on a 16-byte boundary: read one by one
            e_dev = torch.cat([torch.zeros(1), energy]).cuda()[1:]
        h.accumulate(xs.cuda(), block, 7.0, e_dev)
        got = [h.weight.cpu(), h.total.cpu(), h.square.cpu()]
        assert torch.equal(got[0] != 0, want[0] != 0)
        if energy is None:
            assert torch.equal(got[0], want[0])
        for a, b in zip(got, want):
            assert torch.allclose(a, b, rtol=1e-11, atol=1e-9 * float(b.abs().max()))
