"""GPTQ weight compensation on the microscaling grid (quantization/gptq.py): the oracle against vectors
upstream's ``compensate_weight`` produced (CPU), the CUDA walk against the oracle (GPU)."""
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
        _Z = np.load(os.path.join(GOLDEN, "golden_gptq.npz"))
    return _Z


def _cases():
    return json.loads(bytes(_z()["cases"]).decode())


def _f32(name, key):
    return torch.from_numpy(_z()[f"{name}/{key}"].copy()).view(torch.float32)


def _table(name, key):
    k = f"{name}/{key}"
    return torch.from_numpy(_z()[k].copy()).view(torch.bfloat16) if k in _z().files else None


CASES = _cases()


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_upstream(case):
    n = case["name"]
    torch.set_num_threads(1)
    w, h = _f32(n, "weight"), _f32(n, "hessian")
    qmap, sq = _table(n, "qmap"), _table(n, "scale_qmap")
    perm = vo.gptq_salience_order(h, case["K"], case["within_block"], case["block"]) if case["act_order"] else None
    hp = h if perm is None else h[perm][:, perm]
    hinv = vo.gptq_hessian_inverse_chol(hp.clone(), case["tokens"], case["damping"])
    assert torch.equal(hinv, _f32(n, "hinv"))
    out = vo.gptq_compensate_weight(w, h.clone(), case["tokens"], qmap, sq, case["quant_max"], case["block"], case["damping"],
                                    case["act_order"], case["within_block"], case["shrink"])
    assert torch.equal(out, _f32(n, "out"))


def test_salience_order_keeps_blocks_whole():
    h = torch.diag(torch.arange(1.0, 129.0))
    perm = vo.gptq_salience_order(h, 128, True, 32)
    assert sorted(perm.tolist()) == list(range(128))
    for b in range(4):
        blk = perm[b * 32:(b + 1) * 32]
        assert len({int(i) // 32 for i in blk}) == 1
    assert perm[0] == 127                                         # most salient column of the most salient block first
    assert vo.gptq_salience_order(h[:80, :80], 80, True, 32) is None
