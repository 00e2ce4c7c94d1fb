"""bf16 kernels divide by multiplying with a reciprocal.  Every bf16 value over every scale
significand must round exactly like the CPU's fp32 division: checked through tables that keep the
full bf16 resolution of the quotient, so that a single wrong rounding shows."""
import os
import sys

import pytest
import torch

import voyager_compiler_b200 as vb  # noqa: F401  (registers the ops)

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

pytestmark = pytest.mark.gpu
Q = torch.ops.quantized_ops


def _resolution_table(flat_below_exponent):
    """Identity on bf16 patterns (NaN -> one NaN); values below 2^flat_below_exponent go to +0 when
    an exponent is given, which makes the table constant over the tiny patterns."""
    t = vo.all_bf16_patterns().clone()
    t[torch.isnan(t)] = float("nan")
    if flat_below_exponent is not None:
        t[t.float().abs() < 2.0 ** flat_below_exponent] = 0.0
    return t


def _same(a, b):
    a, b = a.cpu().view(torch.int16), b.view(torch.int16)
    return torch.equal(a, b)


@pytest.mark.parametrize("flat", [-100, None], ids=["flat_tiny_table", "full_identity_table"])
@pytest.mark.parametrize("exponent", [-3, 40])
def test_every_bf16_value_over_every_scale_significand(flat, exponent):
    tab = _resolution_table(flat)
    x = vo.all_bf16_patterns().repeat(128, 1)                                   # [128, 65536]
    s = ((128 + torch.arange(128, dtype=torch.float32)) / 128.0 * 2.0 ** exponent).to(torch.bfloat16)[:, None]
    want = vo.quantize(x, s, None, None, None, tab)
    got = Q.quantize(x.cuda(), s.cuda(), None, None, None, tab.cuda())
    nan = torch.isnan(want)
    assert torch.equal(torch.isnan(got.cpu()), nan)
    assert _same(torch.where(nan, 0, got.cpu()), torch.where(nan, 0, want))


@pytest.mark.parametrize("flat", [-100, None], ids=["flat_tiny_table", "full_identity_table"])
@pytest.mark.parametrize("exponent", [-6, 20])
def test_block_maximum_scales_over_every_significand(flat, exponent):
    tab = _resolution_table(flat)
    g = torch.Generator().manual_seed(11)
    rows, cols = 256, 64 * 256
    ex_s = 127 + exponent
    bits = (torch.randint(0, 2, (rows, cols), generator=g) << 15) \
        | (torch.randint(ex_s - 24, ex_s, (rows, cols), generator=g) << 7) | torch.randint(0, 128, (rows, cols), generator=g)
    smant = (torch.arange(rows) % 128)[:, None].expand(rows, cols // 64)
    first = (ex_s << 7) | smant                                                   # the block maximum, significand by row
    bits.view(rows, cols // 64, 64)[:, :, 0] = first
    x = bits.to(torch.int16).view(torch.bfloat16)
    s_ref, c_ref = vo.quantize_mx(x, tab, (-1,), 64, 1.0, False)
    s_got, c_got = Q.quantize_mx(x.cuda(), tab.cuda(), (-1,), 64, 1.0, False)
    assert _same(s_got, s_ref)
    assert _same(c_got, c_ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_channel_kernel_divides_like_the_cpu(dtype):
    """The per-channel kernel divides by a corrected reciprocal (fp32-exact by Markstein's theorem).
    Random significands against 64 scales, through a table that keeps the quotient's full bf16
    resolution; scales given explicitly and derived from the channel maximum."""
    from voyager_compiler_b200 import model_quant as mq
    g = torch.Generator().manual_seed(5)
    ch, n = 64, 1 << 18
    bits = (torch.randint(0, 2, (ch, n), generator=g) << 31) | (torch.randint(100, 140, (ch, n), generator=g) << 23) \
        | torch.randint(0, 1 << 23, (ch, n), generator=g)
    x = bits.to(torch.int32).view(torch.float32)
    x[:, :4] = torch.tensor([0.0, -0.0, 1e-30, -3e25])                 # zeros and values outside the corrected range
    x = x.to(dtype)
    sbits = (torch.randint(110, 130, (ch, 1), generator=g) << 23) | torch.randint(0, 1 << 23, (ch, 1), generator=g)
    s = sbits.to(torch.int32).view(torch.float32).to(dtype)
    s[0] = 0.25
    s[1] = 3e-12                                                        # outside the corrected range: IEEE division
    tab = _resolution_table(None)
    (r,) = mq.quantize_tensors_per_channel([x.cuda()], tab, 1.0, scales=[s.cuda()], want_values=True, want_dequant=False)
    assert _same(r.values, vo.quantize(x, s, None, None, None, tab))
    (r2,) = mq.quantize_tensors_per_channel([x.cuda()], tab, 3.0, want_values=True, want_dequant=False)
    s2 = vo.channel_scale(x, 3.0)
    assert _same(r2.scale, s2)
    assert _same(r2.values, vo.quantize(x, s2, None, None, None, tab))
