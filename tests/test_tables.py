"""Product table builders and table analysis (host logic, no GPU)."""
import numpy as np
import pytest
import torch

from golden_util import golden_aux, golden_table, golden_table_names
from voyager_compiler_b200 import tables as T

BUILTIN = [n for n in golden_table_names() if not n.startswith("cb")]


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).numpy().view(np.uint16)


def _same(a: np.ndarray, b: np.ndarray):
    ca, cb = T._canon(a), T._canon(b)
    bad = np.flatnonzero(ca != cb)
    return bad


@pytest.mark.parametrize("name", BUILTIN)
def test_builder_matches_upstream_table(name):
    mine = T.build_table(name)
    bad = _same(mine, _bits(golden_table(name)))
    assert bad.size == 0, (f"{bad.size} entries differ, first pattern {bad[0]:#06x}: "
                           f"{T.bf16_bits_to_f32(mine[bad[:1]])} vs {golden_table(name)[int(bad[0])].item()}")


@pytest.mark.parametrize("name", ["cb4", "cb16", "cb7"])
def test_codebook_builder(name):
    mine = T.codebook_table(golden_aux(name + "/entries").tolist())
    assert _same(mine, _bits(golden_table(name))).size == 0


@pytest.mark.parametrize("name", ["nf4", "nf4_6", "nf3"])
def test_nf_levels_and_indices(name):
    import re
    m = re.fullmatch(r"nf(\d+)(?:_(\d+))?", name)
    tab, idx, lv = T._nf_table(int(m.group(1)), int(m.group(2)) if m.group(2) else None)
    assert (idx == golden_aux(name + "/indices")).all()
    assert (T.f32_to_bf16_bits(lv) == golden_aux(name + "/levels")).all()


@pytest.mark.parametrize("name", golden_table_names())
def test_analysis_reproduces_table(name):
    """INT and RUNS descriptions must regenerate the table exactly on every pattern."""
    lut = _bits(golden_table(name))
    an = T.analyse_table(lut)
    canon = T._canon(lut)
    keys = T.sort_key(np.arange(1 << 16, dtype=np.uint32))
    nanp = (np.arange(1 << 16) & 0x7FFF) > 0x7F80
    if an.is_int:
        v = T.bf16_patterns_f32()
        with np.errstate(all="ignore"):
            ref = T.f32_to_bf16_bits(np.clip(np.rint(v), an.lo, an.hi))
        assert (T._canon(ref) == canon).all()
    if an.n_runs:
        idx = np.searchsorted(an.run_keys.astype(np.uint32), keys, side="right")
        out = an.run_vals[np.minimum(idx, an.n_runs - 1)]
        out = np.where(nanp, an.nan_val, out)
        out[0x7F80], out[0xFF80] = an.pinf_val, an.ninf_val
        got = T._canon(out.astype(np.uint16))
        if an.nan_consistent:
            assert (got == canon).all()
        else:
            assert (got[~nanp] == canon[~nanp]).all()
    assert an.is_int == (name.startswith("int") and name != "int16" or name.startswith("uint"))


def test_expected_run_counts():
    runs = {n: T.analyse_table(_bits(golden_table(n))).n_runs for n in ["int8", "int4", "posit8_1", "e4m3", "nf4"]}
    assert runs["nf4"] == 16 and runs["int4"] <= 17 and runs["posit8_1"] == 255 and runs["e4m3"] == 253
    assert runs["int8"] == 257
    assert T.analyse_table(_bits(golden_table("posit16_1"))).n_runs == 0


@pytest.mark.parametrize("name", ["int8", "uint8", "nf4", "posit8_1", "e4m3", "int4", "cb7"])
def test_code_table_roundtrip(name):
    lut = _bits(golden_table(name))
    codes, levels = T.code_table(lut)
    vals = T.bf16_bits_to_f32(lut)
    ok = ~np.isnan(vals)
    assert (levels[codes[ok]] == vals[ok]).all()


def test_code_table_of_index_table():
    from golden_util import index_table_of
    idx, levels = index_table_of("nf4")
    lut = T.f32_to_bf16_bits(idx.numpy().astype(np.float32))
    codes, lv = T.code_table(lut)
    assert (codes == idx.numpy()).all() and lv.size == 16


def test_quant_range():
    assert T.quant_range("int8") == (-128.0, 127.0)
    assert T.quant_range("posit8_1")[1] == 4096.0
    assert T.quant_range("nf4")[1] == 1.0 and T.quant_range("nf4_6")[1] == 31.0
    assert T.quant_range("e4m3")[1] == 448.0
