"""Seeded random shapes / axes / block sizes / dtypes / tables through the CUDA ops, checked bit
for bit against the CPU oracle (generic, strided and specialised kernel paths all get traffic)."""
import os
import random
import sys

import pytest
import torch

import voyager_compiler_b200 as vb
from golden_util import golden_table, index_table_of, same_bits

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

pytestmark = pytest.mark.gpu
Q = torch.ops.quantized_ops

TABLES = {"int8": 127.0, "int4": 7.0, "posit8_1": 4096.0, "e4m3": 448.0, "nf4": 1.0, "fp6_e3m2": 28.0, "cb7": 6.0}


def _rand_tensor(rng, shape, dtype):
    g = torch.Generator().manual_seed(rng.randrange(1 << 30))
    x = torch.randn(shape, generator=g) * (10.0 ** rng.uniform(-3, 3))
    if rng.random() < 0.3:
        x[torch.rand(shape, generator=g) < 0.05] = 0.0
    if rng.random() < 0.15 and x.numel() > 3:
        flat = x.view(-1)
        flat[rng.randrange(x.numel())] = float("inf") if rng.random() < 0.5 else float("nan")
    return x.to(dtype)


@pytest.mark.parametrize("seed", range(40))
def test_random_mx_quantize_dequantize(seed):
    rng = random.Random(1000 + seed)
    nd = rng.randint(1, 4)
    shape = [rng.choice([1, 2, 3, 5, 8, 16, 17, 32, 40, 64, 96]) for _ in range(nd)]
    if rng.random() < 0.4:
        shape[-1] = rng.choice([32, 64, 128, 256, 512])       # specialised-kernel territory
    dtype = rng.choice([torch.float32, torch.bfloat16])
    name = rng.choice(list(TABLES))
    qmax = TABLES[name]
    bs = rng.choice([1, 2, 4, 8, 16, 32, 64])
    axis = rng.randrange(-nd, nd)
    pow2 = rng.random() < 0.5
    tab = golden_table(name)
    x = _rand_tensor(rng, shape, dtype)
    s_ref, c_ref = vo.quantize_mx(x, tab, (axis,), bs, qmax, pow2)
    s, c = Q.quantize_mx(x.cuda(), tab.cuda(), (axis,), bs, qmax, pow2)
    ok, msg = same_bits(s, s_ref)
    assert ok, f"scale {shape} {dtype} {name} bs={bs} ax={axis} pow2={pow2}: {msg}"
    ok, msg = same_bits(c, c_ref)
    assert ok, f"codes {shape} {dtype} {name} bs={bs} ax={axis} pow2={pow2}: {msg}"
    s2 = Q.calculate_mx_qparam(x.cuda(), (axis,), bs, qmax, pow2)
    assert same_bits(s2, s_ref)[0]
    c2 = Q.quantize(x.cuda(), s, None, (axis,), bs, tab.cuda())
    assert same_bits(c2, c_ref)[0]
    d_ref = vo.dequantize(c_ref, s_ref, None, (axis,), bs)
    ok, msg = same_bits(Q.dequantize(c, s, None, (axis,), bs), d_ref)
    assert ok, f"dequant: {msg}"


@pytest.mark.parametrize("seed", range(20))
def test_random_broadcast_scales_and_zero_points(seed):
    rng = random.Random(5000 + seed)
    nd = rng.randint(1, 4)
    shape = [rng.choice([1, 2, 3, 4, 7, 16, 33]) for _ in range(nd)]
    dtype = rng.choice([torch.float32, torch.bfloat16])
    x = _rand_tensor(rng, shape, dtype)
    sshape = [n if rng.random() < 0.5 else 1 for n in shape]
    if rng.random() < 0.3:
        sshape = sshape[rng.randrange(nd):]
    g = torch.Generator().manual_seed(seed)
    scale = (torch.rand(sshape, generator=g) + 0.05).to(dtype)
    zp = torch.round(torch.randn(sshape, generator=g) * 3).to(dtype) if rng.random() < 0.5 else None
    name = rng.choice(["int8", "uint8", "posit8_1"])
    tab = golden_table(name)
    want = vo.quantize(x, scale, zp, None, None, tab)
    got = Q.quantize(x.cuda(), scale.cuda(), zp.cuda() if zp is not None else None, None, None, tab.cuda())
    ok, msg = same_bits(got, want)
    assert ok, f"quantize {shape} scale {sshape} zp={zp is not None} {dtype} {name}: {msg}"
    wd = vo.dequantize(want, scale, zp, None, None, None, tab if rng.random() < 0.5 else None)
    # replay with the same choice of output table
    rng2 = random.Random(5000 + seed)
    out_tab = None
    if not torch.equal(torch.nan_to_num(wd.float()), torch.nan_to_num(vo.dequantize(want, scale, zp).float())):
        out_tab = tab
    gd = Q.dequantize(got, scale.cuda(), zp.cuda() if zp is not None else None, None, None, None,
                      out_tab.cuda() if out_tab is not None else None)
    ok, msg = same_bits(gd, vo.dequantize(want, scale, zp, None, None, None, out_tab))
    assert ok, f"dequantize: {msg}"


@pytest.mark.parametrize("seed", range(8))
def test_random_index_tables_and_multi_tensor(seed):
    from voyager_compiler_b200 import model_quant as mq
    rng = random.Random(9000 + seed)
    tab_i, levels = index_table_of("nf4")
    tab_v = golden_table("nf4")
    shapes = [(rng.choice([1, 3, 16, 100]), rng.choice([64, 128, 448])) for _ in range(rng.randint(1, 5))]
    ws = [_rand_tensor(rng, s, torch.bfloat16) for s in shapes]
    packed = mq.quantize_tensors_mx([w.cuda() for w in ws], tab_v, 64, 1.0, code_bits=4)
    for w, p in zip(ws, packed):
        s_ref = vo.mx_scale(w, (-1,), 64, 1.0, False)
        i_ref = vo.quantize(w, s_ref, None, (-1,), 64, tab_i)
        assert same_bits(p.scale, s_ref.float())[0]
        assert torch.equal(mq.unpack_codes(p).cpu().float(), i_ref.float())


# ---------------------------------------------------------------------------------------------
# the kernels outside the reference op set: per-row codebooks, per-channel multi-tensor pass,
# observer reduction + fused fake-quantize, outlier split
# ---------------------------------------------------------------------------------------------
def _eq(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return a.shape == b.shape and bool(((a == b) | (torch.isnan(a) & torch.isnan(b))).all()) and \
        torch.equal(torch.signbit(a)[a == 0], torch.signbit(b)[b == 0])


@pytest.mark.parametrize("seed", range(16))
def test_random_row_codebooks(seed):
    from voyager_compiler_b200 import codebook
    rng = random.Random(3000 + seed)
    rows, K = rng.choice([1, 3, 17, 64, 300]), rng.choice([1, 5, 32, 100, 256, 1023, 4096])
    n = rng.choice([1, 2, 3, 4, 7, 16, 17, 64, 200, 256])
    dtype = rng.choice([torch.float32, torch.bfloat16])
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, K, generator=g) * (10.0 ** rng.uniform(-2, 2))).to(dtype)
    levels = torch.sort(torch.randn(rows, n, generator=g) * float(x.float().abs().max() + 1e-3), dim=-1).values
    if n > 2 and rng.random() < 0.5:
        levels[:, 1] = levels[:, 0]                      # duplicates: the tie walk
    if rng.random() < 0.3:
        levels = torch.round(levels * 4) / 4             # many exact ties between neighbours
        levels = torch.sort(levels, dim=-1).values
    if x.numel() > 2:
        x.view(-1)[0] = float("nan")
        x.view(-1)[-1] = float("-inf")
    rule = rng.random() < 0.5
    idx, val = codebook.row_codebook_quantize(x.cuda(), levels.cuda(), reference_rule=rule, check_sorted=True)
    o_idx, o_val = vo.row_codebook(x, levels, rule)
    assert torch.equal(idx.cpu(), o_idx), (rows, K, n, dtype, rule)
    assert _eq(val, o_val)


@pytest.mark.parametrize("seed", range(12))
def test_random_per_channel_multi_tensor(seed):
    from voyager_compiler_b200 import model_quant as mq
    rng = random.Random(4000 + seed)
    dtype = rng.choice([torch.float32, torch.bfloat16])
    name = rng.choice(["int8", "posit8_1", "e4m3", "int4", "nf4"])
    qmax = TABLES[name]
    ws = []
    for _ in range(rng.randint(1, 6)):
        shape = [rng.choice([1, 3, 16, 70, 513])] + [rng.choice([1, 3, 4, 7, 64]) for _ in range(rng.randint(1, 3))]
        ws.append(_rand_tensor(rng, shape, dtype))
    tab = golden_table(name)
    want_codes = name != "nf4" or True
    got = mq.quantize_tensors_per_channel([w.cuda() for w in ws], tab, qmax, want_values=True, want_codes=want_codes,
                                          want_dequant=True, want_amax=True)
    for w, r in zip(ws, got):
        s_ref = vo.channel_scale(w, qmax)
        q_ref = vo.quantize(w, s_ref, None, None, None, tab)
        assert _eq(r.scale, s_ref) and _eq(r.values, q_ref) and _eq(r.dequant, vo.dequantize(q_ref, s_ref))
        assert _eq(r.amax, vo.observe_amax(w, 0))


@pytest.mark.parametrize("seed", range(16))
def test_random_amax_and_fake_quantize(seed):
    from voyager_compiler_b200 import fake_quantize as fq
    rng = random.Random(5000 + seed)
    dtype = rng.choice([torch.float32, torch.bfloat16])
    nd = rng.randint(1, 4)
    shape = [rng.choice([1, 2, 5, 16, 33, 64, 130]) for _ in range(nd)]
    x = _rand_tensor(rng, shape, dtype)
    axis = rng.choice([None] + list(range(-nd, nd)))
    assert _eq(fq.amax(x.cuda(), axis), vo.observe_amax(x, axis)), (shape, axis)
    name = rng.choice(list(TABLES))
    tab = golden_table(name)
    sshape = () if axis is None else tuple(shape[i] if i == axis % nd else 1 for i in range(nd))
    s = ((torch.rand(sshape) + 0.01) * float(x.float().abs().nan_to_num(0, 0, 0).max() + 1e-3) / TABLES[name]).float()
    assert _eq(fq.fake_quantize(x.cuda(), s.cuda(), tab.cuda()), vo.fake_quantize(x, s, tab)), (shape, axis, name)


@pytest.mark.parametrize("seed", range(10))
def test_random_filter_outlier(seed):
    rng = random.Random(6000 + seed)
    dtype = rng.choice([torch.float32, torch.bfloat16])
    shape = [rng.choice([1, 2, 3]) for _ in range(rng.randint(0, 2))] + [rng.choice([1, 7, 64, 300]), rng.choice([1, 5, 33, 128, 1000])]
    x = _rand_tensor(rng, shape, dtype)
    thr = rng.choice([0.0, 0.5, 2.0, 1e6]) * float(x.float().abs().nan_to_num(0, 0, 0).mean() + 1e-6)
    pct = rng.choice([0.001, 0.01, 0.2, 1.0])
    d, i, p, inl = Q.filter_outlier(x.cuda(), thr, pct)
    od, oi, op, oinl = vo.filter_outlier(x, thr, pct)
    assert torch.equal(p.cpu(), op) and torch.equal(i.cpu(), oi), (shape, thr, pct)
    assert _eq(d, od) and _eq(inl, oinl)
