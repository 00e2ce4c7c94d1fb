"""GPU parity on seeded tensors with the shapes and distributions of the benchmark configs,
checked against the CPU oracle on the same tensors, plus size-independent properties."""
import os
import sys

import pytest
import torch

import voyager_compiler_b200 as vb
from golden_util import golden_table, index_table_of, same_bits

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

pytestmark = pytest.mark.gpu
Q = torch.ops.quantized_ops


def _cfg1_input(rows=4096, cols=4096):
    torch.manual_seed(0)
    x = torch.randn(rows, cols)
    m = torch.rand_like(x) < 0.001
    x[m] *= 50
    return x


@pytest.mark.parametrize("policy", ["int", "lut"])
def test_cfg1_quantize_mx_int8_pow2_full_size(policy):
    """fp32 [4096,4096], block 32, int8 table, power-of-two scale: codes, scales, dequant."""
    vb.set_table_policy(runs_max=0, allow_int=(policy == "int"))
    try:
        x = _cfg1_input()
        q = golden_table("int8")
        s_ref, c_ref = vo.quantize_mx(x, q, (-1,), 32, 127.0, True)
        d_ref = vo.dequantize(c_ref, s_ref, None, (-1,), 32)
        xs = x.cuda()
        s, c = Q.quantize_mx(xs, q.cuda(), (-1,), 32, 127.0, True)
        d = Q.dequantize(c, s, None, (-1,), 32)
        for got, want in ((s, s_ref), (c, c_ref), (d, d_ref)):
            ok, msg = same_bits(got, want)
            assert ok, msg
        # the table clamps to [-128, 127]: -128 is a legal code
        assert c.min().item() >= -128 and c.max().item() <= 127
        s2 = Q.calculate_mx_qparam(xs, (-1,), 32, 127.0, True)
        assert torch.equal(s2, s)
    finally:
        vb.set_table_policy(runs_max=0, allow_int=True)


def test_cfg2_posit8_per_channel_resnet_shapes():
    torch.manual_seed(1)
    q = golden_table("posit8_1")
    shapes = [(64, 3, 7, 7), (64, 64, 1, 1), (256, 64, 1, 1), (128, 128, 3, 3), (512, 512, 3, 3), (2048, 512, 1, 1),
              (1000, 2048)]
    for shp in shapes:
        w = torch.empty(shp)
        torch.nn.init.kaiming_normal_(w, mode="fan_in")
        scale = vo.channel_scale(w, 4096.0, 0)
        want_q = vo.quantize(w, scale, qmap=q)
        want_d = vo.dequantize(want_q, scale)
        got_q = Q.quantize(w.cuda(), scale.cuda(), None, None, None, q.cuda())
        got_d = Q.dequantize(got_q, scale.cuda())
        ok, msg = same_bits(got_q, want_q)
        assert ok, f"{shp}: {msg}"
        ok, msg = same_bits(got_d, want_d)
        assert ok, f"{shp}: {msg}"


@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 11008)])
def test_cfg3_nf4_block64_bf16(shape):
    torch.manual_seed(2)
    w = (torch.randn(shape) * 0.02).to(torch.bfloat16)
    tab_v = golden_table("nf4")
    tab_i, levels = index_table_of("nf4")
    s_ref = vo.mx_scale(w, (-1,), 64, 1.0, False)
    i_ref = vo.quantize(w, s_ref, None, (-1,), 64, tab_i)
    v_ref = vo.quantize(w, s_ref, None, (-1,), 64, tab_v)
    wc = w.cuda()
    s = Q.calculate_mx_qparam(wc, (-1,), 64, 1.0, False)
    i = Q.quantize(wc, s, None, (-1,), 64, tab_i.cuda())
    s2, v = Q.quantize_mx(wc, tab_v.cuda(), (-1,), 64, 1.0, False)
    for got, want in ((s, s_ref), (i, i_ref), (s2, s_ref), (v, v_ref)):
        ok, msg = same_bits(got, want)
        assert ok, msg
    # decoding the indices gives the values
    assert torch.equal(levels.cuda()[i.long()], v)


def test_cfg5_activation_quantize_bf16():
    torch.manual_seed(4)
    x = torch.randn(2048, 4096).to(torch.bfloat16)
    q = golden_table("int8")
    s_ref, c_ref = vo.quantize_mx(x, q, (-1,), 32, 127.0, True)
    s, c = Q.quantize_mx(x.cuda(), q.cuda(), (-1,), 32, 127.0, True)
    assert same_bits(s, s_ref)[0] and same_bits(c, c_ref)[0]


def test_large_lut_path_posit_fp32_and_bf16():
    """> 2^21 elements: the table is staged in shared memory."""
    torch.manual_seed(7)
    q = golden_table("posit8_1")
    for dt in (torch.float32, torch.bfloat16):
        x = (torch.randn(2048, 2048) * 3).to(dt)
        sc = torch.tensor([0.37], dtype=dt)
        want = vo.quantize(x, sc, qmap=q)
        got = Q.quantize(x.cuda(), sc.cuda(), None, None, None, q.cuda())
        ok, msg = same_bits(got, want)
        assert ok, msg
        want = vo.lut_map(x, q)
        ok, msg = same_bits(Q.vmap(x.cuda(), q.cuda()), want)
        assert ok, msg


def test_idempotence_and_scale_linearity_properties():
    """Size-independent checks at full size: quantizing the dequantized tensor again with the same
    scales returns the same codes; scaling the input by a power of two scales the scale and leaves
    the codes alone."""
    x = _cfg1_input().cuda()
    q = golden_table("int8").cuda()
    s, c = Q.quantize_mx(x, q, (-1,), 32, 127.0, True)
    d = Q.dequantize(c, s, None, (-1,), 32)
    c2 = Q.quantize(d, s, None, (-1,), 32, q)
    assert torch.equal(c2, c)
    s4, c4 = Q.quantize_mx(x * 4.0, q, (-1,), 32, 127.0, True)
    assert torch.equal(c4, c) and torch.equal(s4, s * 4.0)


def test_every_bf16_pattern_through_every_table():
    from golden_util import golden_table_names
    every = torch.arange(1 << 16, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    for pol in (dict(runs_max=0, allow_int=True), dict(runs_max=512, allow_int=False)):
        vb.set_table_policy(**pol)
        try:
            for name in golden_table_names():
                tab = golden_table(name)
                got = Q.vmap(every.cuda(), tab.cuda())
                ok, msg = same_bits(got, vo.lut_map(every, tab))
                assert ok, f"{name} {pol}: {msg}"
        finally:
            vb.set_table_policy(runs_max=0, allow_int=True)
