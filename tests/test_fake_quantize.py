"""Observer + fake-quantize forward: the oracle against vectors produced by upstream's module
(CPU), the CUDA module against both (GPU)."""
import json
import os
import sys

import numpy as np
import pytest
import torch

from golden_util import GOLDEN, from_bits, golden_table

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

with open(os.path.join(GOLDEN, "golden_fake_quant.json")) as _f:
    CASES = json.load(_f)["cases"]
_Z = None


def _arr(case, t, key):
    global _Z
    if _Z is None:
        _Z = np.load(os.path.join(GOLDEN, "golden_fake_quant.npz"))
    shape = case["shapes"][key][t]
    return from_bits(_Z[f"{case['name']}/{t}/{key}"], case["tags"][key], shape)


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
    history, scale = None, torch.tensor([1.0])
    for t in range(case["steps"]):
        x, y_ref, s_ref = _arr(case, t, "x"), _arr(case, t, "y"), _arr(case, t, "scale")
        if mx:
            sq = _table(kw["scale_dtype"]) if kw.get("scale_dtype") else None
            scale, y = vo.mx_fake_quantize(x, qmap, kw["ch_axis"], kw["block_size"], kw["quant_max"],
                                           kw.get("force_scale_power_of_two", False), sq)
        else:
            cur = vo.observe_amax(x, kw.get("ch_axis") if kw["qscheme"] == "per_channel_symmetric" else None)
            if history is None:
                history = torch.zeros((kw["amax_history_len"],) + tuple(cur.shape))
                scale = torch.ones(cur.shape)
            history, scale = vo.update_amax_scale(history, scale, cur, kw["quant_max"], kw.get("force_scale_power_of_two", False))
            y = vo.fake_quantize(x, scale, qmap)
        assert _same(y, y_ref) and _same(scale, s_ref)


def test_cpu_tensors_rejected():
    from voyager_compiler_b200 import fake_quantize as fq
    with pytest.raises(RuntimeError):
        fq.amax(torch.zeros(4))
    with pytest.raises(RuntimeError):
        fq.fake_quantize(torch.zeros(4), torch.ones(1), golden_table("int8"))


def test_module_on_another_device_than_its_input_is_refused_on_the_host():
    """A module built without ``device=`` keeps its buffers on the CPU; handing their addresses to a
    kernel together with a device input would read the wrong memory.  The check is a Python
    exception before any launch (a ``meta`` input stands in for a device one here)."""
    from voyager_compiler_b200 import fake_quantize as fq
    x = torch.empty(4, 64, device="meta")
    for kw in (dict(qscheme="per_tensor_symmetric", quant_max=127.0, amax_history_len=4),
               dict(qscheme="per_channel_symmetric", quant_max=127.0, amax_history_len=4, ch_axis=0),
               dict(qscheme="microscaling", quant_max=127.0, ch_axis=-1, block_size=32),
               dict(qscheme="per_tensor_symmetric", quant_max=127.0, amax_history_len=4, outlier_threshold=3.0),
               dict(qscheme="per_tensor_symmetric", quant_max=127.0, amax_history_len=4, outlier_pct=0.01)):
        m = fq.FusedAmaxObsFakeQuantize("int8", **kw)
        with pytest.raises(RuntimeError, match="same device"):
            m(x)
    with pytest.raises(RuntimeError, match="same device"):
        fq.outlier_split(x, torch.tensor([3.0]))
    with pytest.raises(RuntimeError, match="same device"):
        fq.outlier_merge(x, x, torch.tensor([3.0]))
    with pytest.raises(ValueError):
        fq.outlier_split(x, torch.tensor([3.0], dtype=torch.float64))
    with pytest.raises(ValueError):
        fq.outlier_split(x, 3.0)


def test_state_dict_round_trip_resizes_buffers_and_refreshes_the_switches():
    """fake_quantize.py:434-463: a checkpoint saved after calibration loads into a fresh module, and
    the switches it carries (or that are written into the buffers directly) reach the host mirrors
    the forward reads."""
    from voyager_compiler_b200 import fake_quantize as fq
    kw = dict(qscheme="per_channel_symmetric", quant_max=127.0, amax_history_len=4, ch_axis=0)
    a = fq.FusedAmaxObsFakeQuantize("int8", **kw)
    a.amax_history.resize_(4, 6, 1).copy_(torch.arange(24.0).reshape(4, 6, 1))      # as after a forward on [6, k]
    a.scale.resize_(6, 1).copy_(torch.arange(6.0).reshape(6, 1) + 0.5)
    a.observer_enabled[0] = 0                                                          # written in place, not via the method
    a._refresh_switches()
    assert a._obs_on is False and a._fq_on is True
    sd = a.state_dict()
    assert set(sd) >= {"scale", "amax_history", "fake_quant_enabled", "observer_enabled", "zero_point"}
    b = fq.FusedAmaxObsFakeQuantize("int8", **kw)
    assert b._obs_on is True
    b.load_state_dict(sd)
    assert torch.equal(b.amax_history, a.amax_history) and torch.equal(b.scale, a.scale)
    assert b._obs_on is False and b._fq_on is True and int(b._fq_host[0]) == 1
    b.fake_quant_enabled[0] = 0
    b._refresh_switches()
    assert b._fq_on is False and int(b._fq_host[0]) == 0
    b.enable_fake_quant()
    b.enable_observer()
    assert b._fq_on and b._obs_on and int(b.observer_enabled[0]) == 1
    # strict loading still reports what is missing
    c = fq.FusedAmaxObsFakeQuantize("int8", **kw)
    with pytest.raises(RuntimeError, match="amax_history"):
        c.load_state_dict({k: v for k, v in sd.items() if k != "amax_history"})


# ------------------------------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_module_steps_like_upstream(case):
    from voyager_compiler_b200 import fake_quantize as fq
    kw = dict(case["kwargs"])
    m = fq.FusedAmaxObsFakeQuantize(device="cuda", **kw)
    for t in range(case["steps"]):
        x = _arr(case, t, "x").cuda().requires_grad_(True)
        y = m(x)
        assert _same(y, _arr(case, t, "y")), (case["name"], t)
        assert _same(m.scale, _arr(case, t, "scale")), (case["name"], t)
        y.sum().backward()
        assert torch.equal(x.grad, torch.ones_like(x))          # straight-through estimator
    m.disable_fake_quant()
    x = _arr(case, 0, "x").cuda()
    assert m(x) is x


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,ch_axis", [((4096, 1024), None), ((64, 3, 7, 7), 0), ((2, 96, 56, 56), 1), ((33, 5, 2), 1),
                                           ((512, 768), -1), ((1000, 3), -1), ((7,), None), ((3, 70000), 0)])
def test_amax_matches_torch(dtype, shape, ch_axis):
    from voyager_compiler_b200 import fake_quantize as fq
    g = torch.Generator().manual_seed(len(shape) * 7 + (ch_axis or 0))
    x = (torch.randn(shape, generator=g) * 3).to(dtype)
    assert _same(fq.amax(x.cuda(), ch_axis), vo.observe_amax(x, ch_axis))
    x.view(-1)[x.numel() // 2] = float("nan")
    assert _same(fq.amax(x.cuda(), ch_axis), vo.observe_amax(x, ch_axis))
    x = torch.zeros(shape, dtype=dtype)
    assert _same(fq.amax(x.cuda(), ch_axis), vo.observe_amax(x, ch_axis))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("table", ["int8", "posit8_1", "nf4", "fp8_e4m3"])
def test_fake_quantize_matches_oracle(dtype, table):
    from voyager_compiler_b200 import fake_quantize as fq
    torch.manual_seed(9)
    qmap = golden_table(table)
    for shape, sshape in (((257, 130), ()), ((48, 16, 3, 3), (48, 1, 1, 1)), ((4, 10, 6), (1, 10, 1)), ((2048, 1024), ())):
        x = torch.randn(shape).to(dtype)
        x.view(-1)[1] = float("nan")
        s = (torch.rand(sshape) + 0.05).to(torch.float32) * 0.03
        got = fq.fake_quantize(x.cuda(), s.cuda(), qmap.cuda())
        assert _same(got, vo.fake_quantize(x, s, qmap)), (shape, sshape)


@pytest.mark.gpu
def test_mx_fake_quantize_matches_oracle_large():
    from voyager_compiler_b200 import fake_quantize as fq
    torch.manual_seed(10)
    x = torch.randn(512, 4096).to(torch.bfloat16)
    x[3, :64] = 0
    for table, qmax, pow2, block in (("int8", 127.0, True, 32), ("nf4", 1.0, False, 64)):
        qmap = golden_table(table)
        s, y = fq.mx_fake_quantize(x.cuda(), qmap.cuda(), -1, block, qmax, pow2)
        s_ref, y_ref = vo.mx_fake_quantize(x, qmap, -1, block, qmax, pow2)
        assert _same(s, s_ref) and _same(y, y_ref)


@pytest.mark.gpu
def test_per_channel_observer_refuses_a_new_channel_count_and_loads_a_checkpoint():
    from voyager_compiler_b200 import fake_quantize as fq
    kw = dict(qscheme="per_channel_symmetric", quant_max=127.0, amax_history_len=4, ch_axis=0)
    m = fq.FusedAmaxObsFakeQuantize("int8", device="cuda", **kw)
    torch.manual_seed(0)
    x = torch.randn(6, 40, device="cuda")
    y1 = m(x)
    with pytest.raises(RuntimeError, match="observer state"):
        m(torch.randn(9, 40, device="cuda"))                   # larger count: would index past the history
    with pytest.raises(RuntimeError, match="observer state"):
        m(torch.randn(3, 40, device="cuda"))
    y2 = m(x)                                                   # the module is still usable
    # save -> load into a fresh module -> same next step, observer switch included
    n = fq.FusedAmaxObsFakeQuantize("int8", device="cuda", **kw)
    n.load_state_dict(m.state_dict())
    assert torch.equal(n.scale, m.scale) and torch.equal(n.amax_history, m.amax_history)
    assert torch.equal(n(x), m(x))
    m.observer_enabled[0] = 0                                   # in-place write: the mirror follows
    before = m.amax_history.clone()
    m(x * 3)
    assert torch.equal(m.amax_history, before)
    n.load_state_dict(m.state_dict())
    n(x * 3)
    assert torch.equal(n.amax_history, before)
    # a module left on the CPU refuses a device input instead of handing host addresses to a kernel
    cpu_mod = fq.FusedAmaxObsFakeQuantize("int8", **kw)
    with pytest.raises(RuntimeError, match="same device"):
        cpu_mod(x)
    del y1, y2


def test_pow2_stay_table_reproduces_ceil_log2_of_the_cpu():
    """The table the observer kernel uses for ``2 ** ceil(log2(scale))`` against the CPU formula itself, on the
    values where it matters (just above a power of two, every exponent) and on random scales."""
    import numpy as np
    from voyager_compiler_b200 import qtables
    stay = qtables.derive_pow2_stay_host()
    g = torch.Generator().manual_seed(1)
    e = np.arange(1, 255, dtype=np.uint32)
    near = ((e[:, None] << 23) | np.arange(0, 300, dtype=np.uint32)[None, :]).reshape(-1)
    rnd = torch.randint(1 << 23, 255 << 23, (200000,), generator=g).numpy().astype(np.uint32)
    bits = np.concatenate([near, rnd])
    x = torch.from_numpy(bits.view(np.float32).copy())
    want = torch.pow(2, torch.ceil(torch.log2(x)))
    E = (bits >> 23) & 0xFF
    mant = bits & 0x7FFFFF
    r = E.astype(np.int64) - 127 + (mant >= stay[E]).astype(np.int64)
    got = torch.where(torch.from_numpy(r > 127), torch.tensor(float("inf")), torch.pow(2.0, torch.from_numpy(r.astype(np.float32))))
    assert torch.equal(got, want)


@pytest.mark.gpu
def test_observer_power_of_two_scale_equals_the_cpu_formula_near_powers_of_two():
    """``force_scale_power_of_two`` in the per-channel observer: channel maxima chosen so that amax / quant_max lands on
    and just above powers of two, where a device log2 could round differently from the CPU's."""
    import numpy as np
    from voyager_compiler_b200.fake_quantize import FusedAmaxObsFakeQuantize
    qmax = 127.0
    ks = np.arange(-20, 20)
    ms = np.arange(0, 40, dtype=np.uint32)
    sbits = (((ks[:, None] + 127).astype(np.uint32) << 23) | ms[None, :]).reshape(-1)
    target = torch.from_numpy(sbits.view(np.float32).copy())           # the scales we want to hit
    amax = (target.double() * qmax).float()                             # amax / qmax lands on or next to them
    C = amax.numel()
    x = torch.zeros(C, 8)
    x[:, 0] = amax
    x[:, 1] = -amax / 3
    mod = FusedAmaxObsFakeQuantize("int8", qscheme="per_channel_symmetric", quant_max=qmax, ch_axis=0, amax_history_len=1,
                                   force_scale_power_of_two=True, device="cuda")
    mod(x.cuda())
    mod(x.cuda())                                                       # the second call uses the first call's maximum
    sf = x.abs().amax(dim=1, keepdim=True) / qmax
    want = torch.pow(2, torch.ceil(torch.log2(sf)))
    assert torch.equal(mod.scale.cpu().view(torch.int32), want.view(torch.int32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,ch_axis,pow2", [((64, 4096), None, False), ((64, 4096), None, True), ((96, 32, 3, 3), 0, False),
                                                ((8, 40, 100), 1, True), ((300, 129), 1, False), ((5, 7, 11), 1, False),
                                                ((4, 6, 33), 2, True), ((0, 16), None, False)])
def test_observer_step_in_one_launch_equals_the_separate_launches(dtype, shape, ch_axis, pow2, monkeypatch):
    """The state update by the reduction's last CTA (one launch per step, scratch left at zero) against the memset +
    reduction + update launches, over six steps of changing data including an all-zero, a NaN and an Inf step: history,
    scale and outputs bit for bit, for the three shapes of the reduction (rows, columns, flat) and an empty tensor."""
    from voyager_compiler_b200 import fake_quantize as fq
    from voyager_compiler_b200.fake_quantize import QScheme

    def make():
        kw = dict(dtype="int8", quant_max=127.0, amax_history_len=4, force_scale_power_of_two=pow2, device="cuda")
        if ch_axis is not None:
            kw.update(qscheme=QScheme.PER_CHANNEL_SYMMETRIC, ch_axis=ch_axis)
        return fq.FusedAmaxObsFakeQuantize(**kw)

    g = torch.Generator().manual_seed(sum(shape) + 1)
    steps = []
    for t in range(6):
        x = (torch.randn(shape, generator=g) * (0.3 + t)).to(dtype)
        if x.numel():
            if t == 2:
                x.zero_()
            if t == 3:
                x.view(-1)[x.numel() // 2] = float("nan")
            if t == 4:
                x.view(-1)[0] = float("inf")
        steps.append(x.cuda())
    results = {}
    for mode in ("separate", "fused"):
        if mode == "separate":
            monkeypatch.setenv("VOYAGER_B200_OBSERVER", "separate")
        else:
            monkeypatch.delenv("VOYAGER_B200_OBSERVER", raising=False)
        m = make()
        outs = []
        for x in steps:
            outs.append(m(x).cpu())
            outs.append(m.scale.detach().cpu().clone())
            outs.append(m.amax_history.detach().cpu().clone())
        if mode == "fused" and m._amax_cur is not None:
            assert int((m._amax_cur.view(torch.int32) != 0).sum()) == 0        # maxima and ticket back at zero
        results[mode] = outs
    for a, b in zip(results["separate"], results["fused"]):
        assert a.shape == b.shape and a.dtype == b.dtype
        same = (a.view(torch.int32 if a.element_size() == 4 else torch.int16) == b.view(torch.int32 if b.element_size() == 4 else torch.int16))
        assert bool((same | (torch.isnan(a.float()) & torch.isnan(b.float()))).all())
