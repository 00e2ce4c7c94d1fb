"""The observer's optional steps (quantization/fake_quantize.py:368-432): exponent histogram and outlier
filtering.  The oracle against vectors produced by upstream's module (CPU); the CUDA module and kernels
against the vectors and the oracle (GPU)."""
import json
import os
import sys

import numpy as np
import pytest
import torch

from golden_util import GOLDEN, from_bits, golden_table

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

with open(os.path.join(GOLDEN, "golden_observer_extras.json")) as _f:
    CASES = json.load(_f)["cases"]
_Z = None


def _arr(case, t, key):
    global _Z
    if _Z is None:
        _Z = np.load(os.path.join(GOLDEN, "golden_observer_extras.npz"))
    return from_bits(_Z[f"{case['name']}/{t}/{key}"], case["tags"][key], case["shapes"][key][t])


def _same(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return a.shape == b.shape and bool(((a == b) | (torch.isnan(a) & torch.isnan(b))).all()) and \
        torch.equal(torch.signbit(a)[a == 0], torch.signbit(b)[b == 0])


def _table(name):
    try:
        return golden_table(name)
    except KeyError:
        return vo.value_table(name)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_steps_like_upstream(case):
    kw = case["kwargs"]
    qmap = _table(kw["dtype"])
    mx = kw["qscheme"] == "microscaling"
    history, scale, hist, thr_state, max_pct = None, torch.tensor([1.0]), torch.zeros(254), None, 0.0
    for t in range(case["steps"]):
        x = _arr(case, t, "x")
        if kw.get("record_histogram"):
            hist = hist + vo.exponent_histogram(x)
            assert torch.equal(hist, _arr(case, t, "histogram"))
        thr = kw.get("outlier_threshold")
        if kw.get("outlier_pct") is not None:
            thr_state = vo.outlier_threshold_ema(thr_state, vo.outlier_threshold_topk(x, kw["outlier_pct"]),
                                                 kw.get("outlier_ema_decay", 0.9))
            assert _same(thr_state, _arr(case, t, "outlier_threshold"))
            thr = thr_state
        skip, xin = None, x
        if thr is not None:
            skip, xin = vo.outlier_split(x, thr)
            max_pct = max(max_pct, skip.sum().item() / x.numel())
            assert max_pct == case["max_outlier_pct"][t]
        if kw["qscheme"] == "group_wise_affine":
            sq = _table(kw["scale_dtype"]) if kw.get("scale_dtype") else None
            scale, zp, y = vo.group_affine_fake_quantize(xin, kw["ch_axis"], kw["block_size"], kw["quant_min"], kw["quant_max"], sq)
            assert _same(zp, _arr(case, t, "zero_point"))
        elif mx:
            scale, y = vo.mx_fake_quantize(xin, qmap, kw["ch_axis"], kw["block_size"], kw["quant_max"],
                                           kw.get("force_scale_power_of_two", False), None)
        else:
            cur = vo.observe_amax(xin, kw.get("ch_axis") if kw["qscheme"] == "per_channel_symmetric" else None)
            if history is None:
                history = torch.zeros((kw["amax_history_len"],) + tuple(cur.shape))
                scale = torch.ones(cur.shape)
            history, scale = vo.update_amax_scale(history, scale, cur, kw["quant_max"], False)
            y = vo.fake_quantize(xin, scale, qmap)
        if skip is not None:
            y = vo.outlier_merge(skip, x, y)
        assert _same(y, _arr(case, t, "y")) and _same(scale, _arr(case, t, "scale"))


# ------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_module_steps_like_upstream(case):
    from voyager_compiler_b200 import fake_quantize as fq
    m = fq.FusedAmaxObsFakeQuantize(device="cuda", **dict(case["kwargs"]))
    for t in range(case["steps"]):
        x = _arr(case, t, "x").cuda().requires_grad_(True)
        y = m(x)
        assert _same(y, _arr(case, t, "y")), (case["name"], t)
        assert _same(m.scale, _arr(case, t, "scale")), (case["name"], t)
        if case["kwargs"]["qscheme"] == "group_wise_affine":
            assert _same(m.zero_point, _arr(case, t, "zero_point")), (case["name"], t)
            assert all(_same(a, b) for a, b in zip(m.calculate_qparams(), (m.scale, m.zero_point)))
        if case["kwargs"].get("record_histogram"):
            assert torch.equal(m.histogram.cpu(), _arr(case, t, "histogram")), (case["name"], t)
        if case["kwargs"].get("outlier_pct") is not None:
            assert _same(m.outlier_threshold, _arr(case, t, "outlier_threshold")), (case["name"], t)
        if case["kwargs"].get("outlier_pct") is not None or case["kwargs"].get("outlier_threshold") is not None:
            assert m.max_outlier_pct == case["max_outlier_pct"][t], (case["name"], t)
        y.sum().backward()
        assert torch.equal(x.grad, torch.ones_like(x))          # straight-through estimator


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,form", [(1, None), (31, None), (4099, None), (1 << 20, None), ((1 << 22) + 5, None),
                                    ((1 << 22) + 5, "match"), ((1 << 23) + 3, "flush")])
def test_exponent_histogram_matches_oracle(dtype, n, form, monkeypatch):
    """From 2^18 aligned elements on every lane counts into its own column of shared-memory counters; "match" keeps the
    warp-vote kernel for the large case too, "flush" makes the lanes empty their 16-bit counters every 8 vectors (three rounds at this size)."""
    from voyager_compiler_b200 import fake_quantize as fq
    if form == "match":
        monkeypatch.setenv("VOYAGER_B200_HISTOGRAM", "match")
    if form == "flush":
        monkeypatch.setenv("VOYAGER_B200_HISTOGRAM_FLUSH_EVERY", "8")
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g) * torch.exp2(torch.randint(-140, 130, (n,), generator=g).float())
    k = min(n, 2000)
    e = torch.randint(-126, 128, (k,), generator=g)
    edge = (torch.exp2(e.float()).view(torch.int32) - torch.randint(0, 50, (k,), generator=g).int()).view(torch.float32)
    x[:k] = edge
    if n > 8:
        x[-8:] = torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 1e-40, float("nan"), 1.17549421e-38, -3.4e38])
    x = x.to(dtype)
    xs = x[~torch.isnan(x)]                                     # NaNs are not counted on the device; torch's histc on them is not pinned
    hist = torch.full((254,), 3.0, device="cuda")
    fq.exponent_histogram(x.cuda(), hist)
    assert torch.equal(hist.cpu(), 3.0 + vo.exponent_histogram(xs))
    off = x[1:]                                                 # a pointer that is not 16-byte aligned
    hist2 = torch.zeros(254, device="cuda")
    fq.exponent_histogram(x.cuda()[1:], hist2)
    assert torch.equal(hist2.cpu(), vo.exponent_histogram(off[~torch.isnan(off)]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,thr", [(5, 0.7), (4099, 1.003), (1 << 20, 2.5), ((1 << 21) + 3, 0.0)])
def test_outlier_split_and_merge_match_oracle(dtype, n, thr):
    from voyager_compiler_b200 import fake_quantize as fq
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g).to(dtype)
    x[n // 2] = float("nan")
    x[0] = thr                                                  # |x| == threshold (after rounding to the dtype) is an outlier
    t_dev = torch.tensor([thr], dtype=torch.float32, device="cuda")
    skip, want = vo.outlier_split(x, thr)
    got, count = fq.outlier_split(x.cuda(), t_dev)
    assert _same(got, want) and int(count.item()) == int(skip.sum().item())
    q = (x.float() * 0.5).to(dtype)
    assert _same(fq.outlier_merge(x.cuda(), q.cuda(), t_dev), vo.outlier_merge(skip, x, q))
    got1, count1 = fq.outlier_split(x.cuda()[1:], t_dev)        # unaligned start
    skip1, want1 = vo.outlier_split(x[1:], thr)
    assert _same(got1, want1) and int(count1.item()) == int(skip1.sum().item())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,axis,block,qmin,qmax", [((512, 4096), -1, 32, 0.0, 15.0), ((300, 1000), 1, 128, -128.0, 127.0),
                                                       ((64, 96, 5), 1, 32, 0.0, 255.0), ((7, 50), -1, 16, -8.0, 7.0),
                                                       ((33, 257), -1, 64, 0.0, 3.0), ((4, 8), 0, 32, -128.0, 127.0)])
def test_group_affine_fake_quantize_matches_oracle(dtype, shape, axis, block, qmin, qmax):
    from voyager_compiler_b200 import fake_quantize as fq
    g = torch.Generator().manual_seed(sum(shape) + block)
    x = (torch.randn(shape, generator=g) * 2 + 0.5).to(dtype)
    x.view(-1)[5] = float("nan")
    x.view(-1)[-3:] = 0.0
    for sq in (None, _table("fp8_e5m3")):
        sf, zp, y = fq.group_affine_fake_quantize(x.cuda(), axis, block, qmin, qmax, None if sq is None else sq.cuda())
        sf_ref, zp_ref, y_ref = vo.group_affine_fake_quantize(x, axis, block, qmin, qmax, sq)
        assert _same(sf, sf_ref) and _same(zp, zp_ref) and _same(y, y_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block", [32, 64, 128, 256, 512])
@pytest.mark.parametrize("form", ["default", "held", "sweeps"])
def test_group_affine_blocks_held_in_registers_and_extreme_values(dtype, block, form, monkeypatch):
    """Block sizes that take the kernel which keeps a block in registers and multiplies by a reciprocal where that
    gives the same quotient, against the two-sweep form and the oracle: blocks of tiny (the checked division), huge,
    zero, constant, infinite and NaN values, negative-only and positive-only blocks, a range that overflows."""
    from voyager_compiler_b200 import fake_quantize as fq
    # default: bf16 blocks in packed bf16x2 arithmetic; "held": the fp32-register form for bf16 too; "sweeps": two sweeps
    if form != "default":
        monkeypatch.setenv("VOYAGER_B200_GROUP_AFFINE", form)
    g = torch.Generator().manual_seed(block)
    rows, K = 96, 2048
    x = torch.randn(rows, K, generator=g) * torch.logspace(-3, 3, rows).unsqueeze(1)
    x[3] *= 1e-30
    x[4] *= 1e-38
    x[5] *= 1e25
    x[6] *= 1e35                                                # max - min overflows in places
    x[7] = 0.0
    x[8] = 0.37
    x[9, 5] = float("inf")
    x[10, 7] = float("-inf")
    x[11, 9] = float("nan")
    x[12] = x[12].abs() + 1.0
    x[13] = -x[13].abs() - 1.0
    x[14, ::3] = 0.0
    x[15, :40] = torch.tensor([1e-19, -1e-19, 8.7e-19, 1e-18] * 10)    # around 2^-60
    x[16] *= 1e-17
    x = x.to(dtype)
    for qmin, qmax in ((0.0, 15.0), (-128.0, 127.0), (-8.0, 7.0), (0.0, 255.0), (-7.0, 119.0), (1.0, 3.0), (-64.0, -2.0)):
        sf, zp, y = fq.group_affine_fake_quantize(x.cuda(), -1, block, qmin, qmax, None)
        sf_ref, zp_ref, y_ref = vo.group_affine_fake_quantize(x, -1, block, qmin, qmax, None)
        assert _same(sf, sf_ref) and _same(zp, zp_ref) and _same(y, y_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [(1 << 20) + 7, 3 << 20])
def test_exponent_histogram_on_ordinary_data(dtype, n):
    """Values as tensors hold them (a few binades around one, many exact zeros), which the large-tensor kernel counts
    without looking at the thresholds, with a sprinkling of what sends a batch to the exact rule: patterns just below a
    power of two, subnormals, values outside 2^-62 .. 2^65, infinities."""
    from voyager_compiler_b200 import fake_quantize as fq
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g) * 3
    x[torch.rand(n, generator=g) < 0.3] = 0.0
    k = 300
    at = torch.randint(0, n, (k,), generator=g)
    e = torch.randint(-3, 4, (k,), generator=g)
    x[at] = (torch.exp2(e.float()).view(torch.int32) - torch.randint(0, 50, (k,), generator=g).int()).view(torch.float32)
    x[torch.randint(0, n, (40,), generator=g)] = torch.tensor([1e-39, -3e-42, 1e-25, 1e30, float("inf"), -1e-20, 7e19, 2.0 ** -62] * 5)
    x = x.to(dtype)
    hist = torch.zeros(254, device="cuda")
    fq.exponent_histogram(x.cuda(), hist)
    assert torch.equal(hist.cpu(), vo.exponent_histogram(x))
    fq.exponent_histogram(x.cuda(), hist)                       # accumulates
    assert torch.equal(hist.cpu(), 2 * vo.exponent_histogram(x))


@pytest.mark.gpu
def test_exponent_histogram_with_the_smallest_workspace_takes_a_launch_for_the_addition():
    """2032 bytes of workspace leave no room for the ticket by which the counting kernel's last CTA finishes the call:
    the counts are then added to the histogram by a launch of its own, with the same result."""
    from voyager_compiler_b200 import _lib
    from voyager_compiler_b200.qtables import exp_tables
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(1 << 20, generator=g) * 5).cuda()
    et = exp_tables(torch.float32, 1.0, x.device)
    want = vo.exponent_histogram(x.cpu())
    for words in (254, 255, 256):
        hist = torch.zeros(254, device="cuda")
        ws = torch.empty(words, dtype=torch.int64, device="cuda")
        rc = _lib.lib.vq_exp_histogram(x.data_ptr(), _lib.VQ_F32, x.numel(), et.ptr(), hist.data_ptr(), ws.data_ptr(), words * 8,
                                       torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        assert torch.equal(hist.cpu(), want), words


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lower_by", [0, 0x40, 0x2000, 0x200000])
@pytest.mark.parametrize("form", ["lanes", "match"])
def test_exponent_histogram_follows_the_thresholds_it_is_given(dtype, lower_by, form, monkeypatch):
    """The kernels take the patterns at which floor(log2) rounds up from a table; with thresholds moved down by 64 patterns
    the large-tensor kernel still counts most elements without looking at them, with 2^13 or 2^21 patterns it must look
    for every element (and a bf16 value can now reach a threshold).  Checked against the rule itself in numpy."""
    import numpy as np
    from voyager_compiler_b200 import _lib, qtables
    if form == "match":
        monkeypatch.setenv("VOYAGER_B200_HISTOGRAM", "match")
    bump, scale_of = qtables.derive_exp_tables_host(torch.float32, 0)
    bump = bump.astype(np.int64)
    first = np.array([((i - 149 + 127) << 23) if i - 149 >= -126 else (1 << i) for i in range(277)], dtype=np.int64)
    bump = np.maximum(bump - lower_by, first)                 # never below the binade's first pattern
    g = torch.Generator().manual_seed(lower_by + 1)
    n = (1 << 20) + 3
    x = torch.randn(n, generator=g) * 2
    x[torch.rand(n, generator=g) < 0.1] = 0.0
    k = 5000
    e = torch.randint(-130, 20, (k,), generator=g)
    near = (torch.exp2(e.float().clamp(min=-126)).view(torch.int32) - torch.randint(0, 2 * max(lower_by, 64), (k,), generator=g).int())
    x[torch.randint(0, n, (k,), generator=g)] = near.view(torch.float32)
    x[:4] = torch.tensor([float("inf"), float("nan"), 1e-40, -3e38])
    x = x.to(dtype)
    bits = x.float().view(torch.int32).numpy().astype(np.int64) & 0x7FFFFFFF
    valid = (bits != 0) & (bits < 0x7F800000)
    b = bits[valid]
    ex = np.where(b >= 0x00800000, (b >> 23) - 127, np.floor(np.log2(np.maximum(b, 1))).astype(np.int64) - 149)
    ex = ex + (b >= bump[ex + 149])
    ok = (ex >= -126) & (ex <= 127)
    want = np.bincount(ex[ok] + 126, minlength=254).astype(np.float32)
    et = qtables.ExpTables(torch.from_numpy(bump.astype(np.uint32).view(np.int32).copy()).cuda(), torch.from_numpy(scale_of).cuda())
    hist = torch.zeros(254, device="cuda")
    ws = torch.empty(256, dtype=torch.int64, device="cuda")
    xd = x.cuda()
    rc = _lib.lib.vq_exp_histogram(xd.data_ptr(), _lib.VQ_F32 if dtype == torch.float32 else _lib.VQ_BF16, n, et.ptr(), hist.data_ptr(),
                                   ws.data_ptr(), 2048, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert np.array_equal(hist.cpu().numpy(), want)
