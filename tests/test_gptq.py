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


# ---------------------------------------------------------------------------------------------
# CUDA walk
# ---------------------------------------------------------------------------------------------
def _random_factor(K, g):
    a = torch.randn(K, K, generator=g) * 0.1
    h = a @ a.t() + torch.eye(K) * 0.5
    return torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(h)), upper=True).contiguous()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,scale_dtype,qmax", [("nf4", None, 1.0), ("int4", "fp8_e4m3", 7.0), ("int8", None, 127.0),
                                                    ("posit8_1", "fp8_e4m3", 4096.0)])
@pytest.mark.parametrize("bw", [16, 32, 64, 24, 7])
def test_single_block_bit_exact(dtype, scale_dtype, qmax, bw):
    """One block is reproduced bit for bit: nothing in it depends on a library's summation order."""
    from golden_util import golden_table
    from voyager_compiler_b200 import gptq
    g = torch.Generator().manual_seed(bw * 13 + len(dtype))
    O = 150
    w = torch.randn(O, bw, generator=g) * 0.05
    w[3] = 0.0
    w[4, 1] = 3.0
    hinv = _random_factor(bw, g)
    qmap = golden_table(dtype)
    sq = golden_table(scale_dtype) if scale_dtype else None
    want = vo.gptq_walk(w, hinv, torch.ones(bw), qmap, sq, qmax, 64, False)
    got, scales = gptq.walk(w.cuda(), hinv.cuda(), None, qmap.cuda(), sq.cuda() if sq is not None else None, qmax, 64, False,
                            return_scales=True)
    assert torch.equal(got.cpu(), want)
    want_s = vo.gptq_block_scale(w, torch.ones(bw), qmap, sq, qmax, False)
    assert torch.equal(scales.cpu()[:, 0], want_s)


@pytest.mark.gpu
@pytest.mark.parametrize("bw", [32, 64, 20])
def test_single_block_shrink(bw):
    from golden_util import golden_table
    from voyager_compiler_b200 import gptq
    g = torch.Generator().manual_seed(bw)
    O = 200
    w = torch.randn(O, bw, generator=g) * 0.05
    w[torch.rand(O, bw, generator=g) < 0.03] *= 6
    hinv = _random_factor(bw, g)
    sal = torch.rand(bw, generator=g) * 3 + 0.1
    qmap, sq = golden_table("nf4"), golden_table("fp8_e4m3")
    want_s = vo.gptq_block_scale(w, sal, qmap, sq, 1.0, True)
    got, scales = gptq.walk(w.cuda(), hinv.cuda(), sal.cuda(), qmap.cuda(), sq.cuda(), 1.0, 64, True, return_scales=True)
    same = scales.cpu()[:, 0] == want_s
    # the row sums of the search run in column order here and in torch's reduction order on the CPU: a row
    # whose two best factors are within rounding of each other may pick the other one
    assert same.float().mean() >= 0.98
    assert bool((want_s < vo.gptq_block_scale(w, sal, qmap, sq, 1.0, False)).any())     # the search does shrink some rows
    want = vo.gptq_walk(w[same], hinv, sal, qmap, sq, 1.0, 64, True)
    assert torch.equal(got.cpu()[same], want)


def _proxy_loss(w, q, h):
    d = (w - q).double()
    return float((d @ h.double() * d).sum())


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_walk_with_upstream_factor(case):
    """Several blocks, fed upstream's own inverse factor: only the fp32 product that carries the error to
    the right of a block is summed in another order, so nearly every value lands on the same grid point."""
    from voyager_compiler_b200 import gptq
    n = case["name"]
    w, h, hinv = _f32(n, "weight"), _f32(n, "hessian"), _f32(n, "hinv")
    qmap, sq = _table(n, "qmap"), _table(n, "scale_qmap")
    perm = vo.gptq_salience_order(h, case["K"], case["within_block"], case["block"]) if case["act_order"] else None
    wp, hp = (w, h) if perm is None else (w[:, perm], h[perm][:, perm])
    sal = hp.diagonal().clone()
    want = vo.gptq_walk(wp, hinv, sal, qmap, sq, case["quant_max"], case["block"], case["shrink"])
    got = gptq.walk(wp.cuda(), hinv.cuda(), sal.cuda(), qmap.cuda(), sq.cuda() if sq is not None else None,
                    case["quant_max"], case["block"], case["shrink"]).cpu()
    assert (got == want).float().mean() >= 0.97
    assert _proxy_loss(wp, got, hp) <= 1.02 * _proxy_loss(wp, want, hp)
    first = slice(0, case["block"])                                # the first block has no product before it
    if not case["shrink"]:
        assert torch.equal(got[:, first], want[:, first])


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_compensate_weight_against_upstream(case):
    """The whole entry point on the GPU (ordering, damping, Cholesky by the device library, walk) against
    upstream's result: same proxy loss tr((W - Q) H (W - Q)^T) within 2 %, far below plain rounding."""
    import types
    from voyager_compiler_b200 import gptq
    n = case["name"]
    w, h = _f32(n, "weight"), _f32(n, "hessian")
    qmap, sq = _table(n, "qmap"), _table(n, "scale_qmap")
    fake = types.SimpleNamespace(qmap=qmap.cuda(), scale_qmap=sq.cuda() if sq is not None else None, quant_max=case["quant_max"],
                                 block_size=case["block"], ch_axis=-1)
    got = gptq.compensate_weight(w.cuda(), h.cuda().clone(), case["tokens"], fake, case["damping"], act_order=case["act_order"],
                                 within_block=case["within_block"], shrink=case["shrink"]).cpu()
    want = _f32(n, "out")
    assert got.shape == want.shape and got.dtype == torch.float32
    s = vo.mx_scale(w, -1, case["block"], case["quant_max"], False, sq)
    plain = vo.quantize(w, s, None, (-1,), case["block"], qmap) * vo.spread_scale(s, w.shape, case["block"])
    hn = h / case["tokens"]
    loss_got, loss_want, loss_plain = _proxy_loss(w, got, hn), _proxy_loss(w, want, hn), _proxy_loss(w, plain, hn)
    assert loss_got <= 1.02 * loss_want
    assert loss_want < loss_plain and loss_got < loss_plain
    with pytest.raises(ValueError):
        fake.ch_axis = 0
        gptq.compensate_weight(w.cuda(), h.cuda(), case["tokens"], fake, case["damping"])


def test_cpu_tensors_rejected():
    from voyager_compiler_b200 import gptq
    with pytest.raises(RuntimeError):
        gptq.walk(torch.zeros(4, 32), torch.eye(32), None, torch.zeros(65536, dtype=torch.bfloat16), None, 1.0, 32)
