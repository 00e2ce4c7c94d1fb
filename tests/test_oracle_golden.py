"""The CPU oracle must reproduce the upstream outputs stored in tests/golden bit for bit."""
import os
import sys
import types

import pytest
import torch

from golden_util import case_ids, cases, golden_aux, golden_table, golden_table_names, run_case, same_bits

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

ORACLE = types.SimpleNamespace(
    vmap=vo.lut_map, quantize=vo.quantize, dequantize=vo.dequantize, calculate_mx_qparam=vo.mx_scale,
    quantize_mx=vo.quantize_mx, linear_mx=vo.linear_mx, matmul_mx=vo.matmul_mx, conv2d_mx=vo.conv2d_mx)

BUILTIN = [n for n in golden_table_names() if not n.startswith("cb")]


@pytest.mark.parametrize("name", BUILTIN)
def test_oracle_table_matches_upstream(name):
    ok, msg = same_bits(vo.value_table(name), golden_table(name))
    assert ok, msg


@pytest.mark.parametrize("name", ["nf4", "nf4_6", "nf3"])
def test_oracle_nf_indices(name):
    idx, lv = vo.table_for(name)
    assert (idx.numpy() == golden_aux(name + "/indices")).all()
    ok, msg = same_bits(lv, torch.from_numpy(golden_aux(name + "/levels").view("int16").copy()).view(torch.bfloat16))
    assert ok, msg


@pytest.mark.parametrize("name", ["cb4", "cb16", "cb7"])
def test_oracle_codebook_table(name):
    entries = golden_aux(name + "/entries").tolist()
    ok, msg = same_bits(vo.codebook_table(entries), golden_table(name))
    assert ok, msg


def test_codebook_tie_goes_to_lower_index():
    t = vo.codebook_table([-3.0, -1.0, 1.0, 3.0])
    pat = lambda v: int(torch.tensor([v], dtype=torch.bfloat16).view(torch.int16).item()) & 0xFFFF
    assert t[pat(-2.0)].item() == -3.0 and t[pat(0.0)].item() == -1.0 and t[pat(2.0)].item() == 1.0


@pytest.mark.parametrize("case", cases(), ids=case_ids())
def test_oracle_replays_upstream_case(case):
    outs, expected = run_case(case, ORACLE)
    assert len(outs) == len(expected)
    for o, e in zip(outs, expected):
        if case["op"] in ("linear_mx", "matmul_mx", "conv2d_mx"):
            # same torch CPU GEMM on the same operands: expected to be identical as well
            assert o.dtype == e.dtype and o.shape == e.shape
            rel = (o.double() - e.double()).norm() / e.double().norm()
            assert rel <= 1e-6, rel
        else:
            ok, msg = same_bits(o, e)
            assert ok, f"{case['name']}: {msg}"


def test_int8_table_has_minus_128():
    t = golden_table("int8").float()
    assert t[torch.isfinite(t)].min().item() == -128.0 and t[torch.isfinite(t)].max().item() == 127.0


def test_dtype_range():
    assert vo.dtype_range("int8") == (-128, 127)
    assert vo.dtype_range("posit8_1") == (-4096, 4096)
    assert vo.dtype_range("nf4") == (-1, 1)
    assert vo.dtype_range("nf4_6") == (-31, 31)
    assert vo.dtype_range("fp8_e4m3")[1] == 448.0
