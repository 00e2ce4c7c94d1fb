"""Whole-model (multi-tensor) MX quantization: sharding plan on CPU, kernel parity on GPU."""
import os
import sys

import pytest
import torch

from voyager_compiler_b200 import model_quant as mq
from golden_util import golden_table, index_table_of, same_bits

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

LLAMA7B = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]


def _llama_shapes():
    return LLAMA7B * 32 + [(32000, 4096)]


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_plan_covers_every_row_once_and_balances(world):
    shapes = _llama_shapes()
    sizes = [r * c for r, c in shapes]
    rows = [r for r, _ in shapes]
    plan = mq.shard_plan(sizes, rows, world)
    seen = {}
    loads = []
    for rank, items in enumerate(plan):
        load = 0
        for i, b, e in items:
            assert 0 <= b < e <= rows[i]
            seen.setdefault(i, []).append((b, e))
            load += (e - b) * shapes[i][1]
        loads.append(load)
    for i, r in enumerate(rows):
        spans = sorted(seen[i])
        assert spans[0][0] == 0 and spans[-1][1] == r
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert sum(loads) == sum(sizes)
    assert max(loads) <= 1.02 * sum(sizes) / world        # >= 7.8x ideal speed-up at 8 ranks


def test_shard_plan_small_and_degenerate():
    assert mq.shard_plan([], [], 4) == [[], [], [], []]
    plan = mq.shard_plan([10], [1], 4)
    assert sum(len(p) for p in plan) == 1
    with pytest.raises(ValueError):
        mq.shard_plan([1], [1], 0)


def test_cpu_tensors_rejected():
    with pytest.raises(RuntimeError):
        mq.quantize_tensors_mx([torch.randn(4, 64)], "nf4", 64, 1.0)


@pytest.mark.gpu
def test_multi_tensor_nf4_matches_oracle_bitwise():
    torch.manual_seed(2)
    shapes = [(256, 4096), (64, 11008), (1, 64), (3, 5, 128), (2049, 192)]
    ws = [(torch.randn(s) * 0.02).to(torch.bfloat16) for s in shapes]
    ws[3][0, 0, :64] = 0                      # an all-zero block
    ws[3][1, 1, 5] = float("nan")
    tab_v = golden_table("nf4")
    tab_i, levels = index_table_of("nf4")
    packed = mq.quantize_tensors_mx([w.cuda() for w in ws], tab_v, 64, 1.0, code_bits=4)
    floats = mq.quantize_tensors_mx([w.cuda() for w in ws], tab_v, 64, 1.0, float_outputs=True)
    torch.cuda.synchronize()
    for w, p, (fs, fc) in zip(ws, packed, floats):
        s_ref = vo.mx_scale(w, (-1,), 64, 1.0, False)
        i_ref = vo.quantize(w, s_ref, None, (-1,), 64, tab_i)
        v_ref = vo.quantize(w, s_ref, None, (-1,), 64, tab_v)
        assert same_bits(fs, s_ref)[0] and same_bits(fc, v_ref)[0]
        assert same_bits(p.scale, s_ref.float())[0]           # fp32 scale is the exact widening
        codes = mq.unpack_codes(p).cpu()
        nan = torch.isnan(i_ref.float())
        assert torch.equal(codes[~nan].long(), i_ref[~nan].long())
        assert p.codes.shape[-1] * 2 == w.shape[-1]
        assert torch.equal(p.levels, levels.float())


@pytest.mark.gpu
def test_multi_tensor_int8_pow2_fp32_with_exponents():
    torch.manual_seed(0)
    xs = [torch.randn(128, 256), torch.randn(7, 32) * 1e-3, torch.zeros(2, 64)]
    q = golden_table("int8")
    packed = mq.quantize_tensors_mx([x.cuda() for x in xs], q, 32, 127.0, True, code_bits=8, want_exp=True)
    for x, p in zip(xs, packed):
        s_ref, c_ref = vo.quantize_mx(x, q, (-1,), 32, 127.0, True)
        assert same_bits(p.scale, s_ref)[0]
        got = mq.unpack_codes(p).cpu().to(torch.int8).float()      # two's-complement bytes
        assert torch.equal(got, c_ref)
        e = torch.log2(s_ref).clamp(-127, 127).to(torch.int8)
        assert torch.equal(p.exp_e8.cpu(), e)
        d = mq.dequantize_packed_reference(p).cpu()
        assert torch.equal(d, vo.dequantize(c_ref, s_ref, None, (-1,), 32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,table,block,qmax,pow2,bits", [
    (torch.bfloat16, "nf4", 64, 1.0, False, 4),
    (torch.bfloat16, "int8", 32, 127.0, True, 8),
    (torch.float32, "int8", 32, 127.0, True, 8),
    (torch.float32, "int4", 128, 7.0, False, 8),
    (torch.bfloat16, "fp8_e4m3", 16, 448.0, False, 8),
])
def test_large_jobs_match_the_oracle(dtype, table, block, qmax, pow2, bits):
    """>= 2^22 elements: 1024-thread CTAs, several inner iterations per tile with the rotating
    prefetch (ragged tails, an all-zero block, NaN and Inf included)."""
    torch.manual_seed(4)
    shapes = [(1024, 4096), (2049, 384), (3, 5, 128), (1, 128), (4099, 128)]
    ws = [(torch.randn(s) * 0.02).to(dtype) for s in shapes]
    ws[2][0, 0, :] = 0
    ws[2][1, 1, 5] = float("nan")
    ws[1][7, 100] = float("inf")
    ws[4][4098, 127] = -3.0
    tab_v = golden_table(table)
    packed = mq.quantize_tensors_mx([w.cuda() for w in ws], tab_v, block, qmax, pow2, code_bits=bits, want_exp=pow2)
    torch.cuda.synchronize()
    for w, p in zip(ws, packed):
        s_ref = vo.mx_scale(w, (-1,), block, qmax, pow2)
        assert same_bits(p.scale, s_ref.float())[0]
        v_ref = vo.quantize(w, s_ref, None, (-1,), block, tab_v).float()
        got = p.levels[mq.unpack_codes(p).cpu().long().clamp(max=p.levels.numel() - 1)]
        ok = ~torch.isnan(v_ref)
        assert torch.equal(got[ok], v_ref[ok])


def _resnet_like_shapes():
    return [(64, 3, 7, 7), (64, 64, 1, 1), (64, 64, 3, 3), (256, 64, 1, 1), (128, 128, 3, 3), (512, 512, 3, 3),
            (2048, 512, 1, 1), (1000, 2048)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,table,qmax", [(torch.float32, "posit8_1", 4096.0), (torch.bfloat16, "posit8_1", 4096.0),
                                               (torch.float32, "int8", 127.0), (torch.float32, "fp8_e4m3", 448.0)])
def test_per_channel_multi_tensor_matches_oracle(dtype, table, qmax):
    torch.manual_seed(1)
    ws = []
    for s in _resnet_like_shapes():
        w = torch.empty(s)
        torch.nn.init.kaiming_normal_(w, mode="fan_in")
        ws.append(w.to(dtype))
    ws[1][3] = 0                                  # an all-zero channel: scale 1
    ws[2][5, 0, 0, 0] = float("nan")              # NaN channel: scale 1, NaN at the element
    ws[3][7, 1, 0, 0] = float("inf")              # Inf channel: scale 1
    tab = golden_table(table)
    got = mq.quantize_tensors_per_channel([w.cuda() for w in ws], tab, qmax, want_values=True, want_codes=True,
                                          want_dequant=True, want_amax=True)
    torch.cuda.synchronize()
    for w, r in zip(ws, got):
        s_ref = vo.channel_scale(w, qmax)
        q_ref = vo.quantize(w, s_ref, None, None, None, tab)
        d_ref = vo.dequantize(q_ref, s_ref)
        amax = torch.amax(torch.abs(w), dim=tuple(range(1, w.ndim)), keepdim=True)
        assert same_bits(r.scale, s_ref)[0]
        assert same_bits(r.amax, amax)[0]
        assert same_bits(r.values, q_ref)[0]
        assert same_bits(r.dequant, d_ref)[0]
        ok = ~torch.isnan(q_ref.float())
        lv = r.levels[r.codes.cpu().long().clamp(max=r.levels.numel() - 1)]
        assert torch.equal(lv[ok], q_ref.float()[ok])


@pytest.mark.gpu
def test_per_channel_with_given_scales_is_quantize_plus_dequantize():
    torch.manual_seed(6)
    w = torch.randn(96, 32, 3, 3)
    s = (torch.rand(96, 1, 1, 1) + 0.1) / 100
    s[4] = 2.0 ** -7                              # an exact-reciprocal scale
    tab = golden_table("int8")
    (r,) = mq.quantize_tensors_per_channel([w.cuda()], tab, 127.0, scales=[s.cuda()], want_values=True)
    q_ref = vo.quantize(w, s, None, None, None, tab)
    assert same_bits(r.values, q_ref)[0]
    assert same_bits(r.dequant, vo.dequantize(q_ref, s))[0]


@pytest.mark.gpu
def test_dequantize_packed_matches_reference_decode():
    torch.manual_seed(3)
    # int8 / pow2 / fp32 and bf16 outputs, through scales and through exponents
    x = torch.randn(96, 256)
    x[5] = 0
    q = golden_table("int8")
    (p,) = mq.quantize_tensors_mx([x.cuda()], q, 32, 127.0, True, code_bits=8, want_exp=True)
    s_ref, c_ref = vo.quantize_mx(x, q, (-1,), 32, 127.0, True)
    want = vo.dequantize(c_ref, s_ref, None, (-1,), 32)
    # value equality: a two's-complement byte has no -0, which the float codes keep for tiny negatives
    assert torch.equal(mq.dequantize_packed(p).cpu(), want)
    assert torch.equal(mq.dequantize_packed(p, use_exponent=True).cpu(), want)    # all-zero block: 0 * 2^-127 = 0
    assert torch.equal(mq.dequantize_packed(p, torch.bfloat16).cpu(), want.to(torch.bfloat16))
    # nf4 / 4-bit / amax scale: equals weight_code[idx] * expand(scale) of linear_mx's operand decode
    w = (torch.randn(40, 192) * 0.02).to(torch.bfloat16)
    tab_i, levels = index_table_of("nf4")
    (p4,) = mq.quantize_tensors_mx([w.cuda()], golden_table("nf4"), 64, 1.0, code_bits=4)
    s4 = vo.mx_scale(w, (-1,), 64, 1.0, False)
    i4 = vo.quantize(w, s4, None, (-1,), 64, tab_i)
    want4 = levels[i4.long()].to(torch.bfloat16) * vo.spread_scale(s4, w.shape, 64)
    assert same_bits(mq.dequantize_packed(p4, torch.bfloat16), want4)[0]


@pytest.mark.gpu
def test_host_pipeline_round_trip():
    torch.manual_seed(5)
    host = [(torch.randn(512, 1024) * 0.02).to(torch.bfloat16).pin_memory() for _ in range(5)]
    pipe = mq.HostPipeline("cuda:0", golden_table("nf4"), 64, 1.0, chunk_bytes=2 << 20)
    outs = pipe.run(host)
    direct = mq.quantize_tensors_mx([h.cuda() for h in host], golden_table("nf4"), 64, 1.0)
    for (hc, hs), p in zip(outs, direct):
        assert torch.equal(hc, p.codes.cpu()) and torch.equal(hs, p.scale.cpu())
    assert pipe.h2d_bytes == sum(h.numel() * 2 for h in host) and pipe.d2h_bytes > 0


def test_chunk_plan_keeps_order_and_covers_everything():
    sizes = [5, 1, 9, 2, 2, 7, 1]
    plan = mq.HostPipeline.chunk_plan(sizes, 8)
    assert [i for ch in plan for i in ch] == list(range(len(sizes)))
    assert all(sum(sizes[i] for i in ch[:-1]) < 8 for ch in plan)     # a chunk closes as soon as it reaches the size
    assert mq.HostPipeline.chunk_plan([], 8) == []
    assert mq.HostPipeline.chunk_plan([100], 8) == [[0]]


_MANY = [(64, 256), (3, 64), (129, 1024), (1, 4096), (17, 128), (256, 512), (33, 192)]


def _many_tensors(count, seed, dtype=torch.bfloat16, scale=0.02):
    """``count`` tensors of mixed sizes (last dims multiples of 128), with an all-zero block, a NaN
    and an Inf planted in three of them."""
    g = torch.Generator().manual_seed(seed)
    ws = [(torch.randn(_MANY[i % len(_MANY)], generator=g) * scale).to(dtype) for i in range(count)]
    ws[1][0, :64] = 0
    ws[4][3, 70] = float("nan")
    ws[count - 1].view(-1)[5] = float("inf")
    return ws


def _check_packed_against_oracle(ws, packed, table, block, qmax, pow2):
    tab_v = golden_table(table)
    for k, (w, p) in enumerate(zip(ws, packed)):
        s_ref = vo.mx_scale(w, (-1,), block, qmax, pow2)
        assert same_bits(p.scale, s_ref.float())[0], f"tensor {k}: scales differ"
        v_ref = vo.quantize(w, s_ref, None, (-1,), block, tab_v).float()
        got = p.levels[mq.unpack_codes(p).cpu().long().clamp(max=p.levels.numel() - 1)]
        ok = ~torch.isnan(v_ref)
        assert torch.equal(got[ok], v_ref[ok]), f"tensor {k}: codes differ"


@pytest.mark.gpu
@pytest.mark.parametrize("count", [33, 40, 225])
@pytest.mark.parametrize("generic", [False, True])
def test_more_than_32_tensors_take_the_uploaded_descriptors(count, generic, monkeypatch):
    """Above 32 tensors the descriptors and running tile counts travel through the device
    workspace (40 tensors: small CTAs; 225: 1024-thread CTAs with the table staged in shared
    memory, the shape of the whole-model pass); ``generic`` forces the unspecialised kernel, which
    always reads the workspace.  Every tensor is compared with the CPU oracle bit for bit."""
    if generic:
        monkeypatch.setenv("VOYAGER_B200_GENERIC_MX", "1")
    ws = _many_tensors(count, 100 + count)
    packed = mq.quantize_tensors_mx([w.cuda() for w in ws], golden_table("nf4"), 64, 1.0, code_bits=4)
    torch.cuda.synchronize()
    _check_packed_against_oracle(ws, packed, "nf4", 64, 1.0, False)


@pytest.mark.gpu
def test_more_than_32_tensors_float_outputs_and_int8_pow2():
    ws = _many_tensors(45, 7, torch.float32, 1.0)
    q = golden_table("int8")
    outs = mq.quantize_tensors_mx([w.cuda() for w in ws], q, 32, 127.0, True, float_outputs=True)
    torch.cuda.synchronize()
    for k, (w, (s, c)) in enumerate(zip(ws, outs)):
        s_ref, c_ref = vo.quantize_mx(w, q, (-1,), 32, 127.0, True)
        assert same_bits(s, s_ref)[0] and same_bits(c, c_ref)[0], k


@pytest.mark.gpu
@pytest.mark.parametrize("count", [1, 7, 40, 225])
def test_plan_runs_match_the_oracle_and_follow_new_data(count):
    """A prepared pass: one, a few (descriptors in the kernel parameters) and many tensors
    (descriptors uploaded once at creation).  The second run reads the tensors' new contents."""
    ws = _many_tensors(max(count, 5), 300 + count)[:count] if count < 5 else _many_tensors(count, 300 + count)
    dev = [w.cuda() for w in ws]
    plan = mq.MXQuantPlan(dev, golden_table("nf4"), 64, 1.0, code_bits=4)
    side = torch.cuda.Stream()
    plan.run()
    torch.cuda.synchronize()
    _check_packed_against_oracle(ws, plan.results, "nf4", 64, 1.0, False)
    ws2 = [(w.float() * 1.7 + 0.003).to(torch.bfloat16) for w in ws]
    for d, w in zip(dev, ws2):
        d.copy_(w)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):                     # any stream of the device will do
        plan.run()
    torch.cuda.synchronize()
    _check_packed_against_oracle(ws2, plan.results, "nf4", 64, 1.0, False)
    plan.close()


@pytest.mark.gpu
def test_plan_rejects_what_it_cannot_read_in_place():
    x = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    with pytest.raises(ValueError):
        mq.MXQuantPlan([x.t()], golden_table("nf4"), 64, 1.0)
    with pytest.raises(NotImplementedError):
        mq.MXQuantPlan([x[:, :100].contiguous()], golden_table("nf4"), 64, 1.0)
    with pytest.raises(ValueError):
        mq.MXQuantPlan([], golden_table("nf4"), 64, 1.0)


def _check_channel_results(ws, got, tab, qmax, scales=None):
    for k, (w, r) in enumerate(zip(ws, got)):
        s_ref = vo.channel_scale(w, qmax) if scales is None else scales[k].to(w.dtype)
        q_ref = vo.quantize(w, s_ref, None, None, None, tab)
        assert same_bits(r.scale, s_ref)[0], k
        assert same_bits(r.values, q_ref)[0], k
        assert same_bits(r.dequant, vo.dequantize(q_ref, s_ref))[0], k
        ok = ~torch.isnan(q_ref.float())
        lv = r.levels[r.codes.cpu().long().clamp(max=r.levels.numel() - 1)]
        assert torch.equal(lv[ok], q_ref.float()[ok]), k


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["stream", "pipe", "sweep"])
@pytest.mark.parametrize("dtype,table,qmax", [(torch.float32, "posit8_1", 4096.0), (torch.bfloat16, "posit8_1", 4096.0),
                                               (torch.float32, "int8", 127.0), (torch.bfloat16, "fp8_e4m3", 448.0)])
def test_per_channel_kernels_on_awkward_shapes(kernel, dtype, table, qmax, monkeypatch):
    """The two bulk-copy kernels (warps in streaming roles; consumer groups) and the two-sweep kernel on the same awkward set: channel lengths that
    are no multiple of 4 (vectors straddle channels), many short channels per batch, a channel as long
    as a batch, a tensor that starts off a 16-byte boundary, tiny and huge magnitudes (the checked
    division), NaN / Inf / all-zero channels; more than 2^21 elements in total so the staged tables
    are used.  The plan runs twice (second run on changed data)."""
    monkeypatch.setenv("VOYAGER_B200_CHANNEL_KERNEL", kernel)
    g = torch.Generator().manual_seed(17)
    # (96, 1152, 4): channels of 4608 elements, as long as a batch of the streaming kernel
    shapes = [(64, 3, 7, 7), (300, 37), (1024, 64), (96, 1152, 4), (40, 2304), (2000, 1000), (5, 6), (128, 3, 3, 3), (70, 1280),
              (33, 256)]
    ws = [(torch.randn(s, generator=g) * 0.05).to(dtype) for s in shapes]
    ws[1][3] = 0
    ws[2][5, 7] = float("nan")
    ws[2][6, 1] = float("inf")
    ws[4][2] *= 1e-30                               # quotients of tiny values: the corrected reciprocal is not used
    ws[4][3] *= 1e20
    ws[5][7, :5] = torch.tensor([1e-38, -1e-39, 3e-41, 0.0, -0.0]).to(dtype)
    tab = golden_table(table)
    dev = [w.cuda() for w in ws]
    pad = torch.zeros(40 * 2304 + 1, dtype=dtype, device="cuda")          # tensor 4 one element off the allocation start
    pad[1:].copy_(dev[4].reshape(-1))
    dev[4] = pad[1:].view(40, 2304)
    plan = mq.ChannelQuantPlan(dev, tab, qmax, want_values=True, want_codes=True, want_dequant=True)
    _check_channel_results(ws, plan.run(), tab, qmax)
    ws2 = [(w.float() * 1.3).to(dtype) for w in ws]
    for d, w in zip(dev, ws2):
        d.copy_(w)
    _check_channel_results(ws2, plan.run(), tab, qmax)
    assert _status() == 0
    # caller-supplied scales (observer state): the checked division, batch by batch
    scales = [(torch.rand(w.shape[0], *([1] * (w.ndim - 1)), generator=g) + 0.1) / 50 for w in ws2]
    got = mq.quantize_tensors_per_channel(dev, tab, qmax, scales=[s.cuda() for s in scales], want_values=True, want_codes=True)
    _check_channel_results(ws2, got, tab, qmax, scales)
    # a channel longer than a batch of the pipeline: the call falls back to the two-sweep kernel
    big = (torch.randn(300, 9000, generator=g) * 0.05).to(dtype)
    (r,) = mq.quantize_tensors_per_channel([big.cuda()], tab, qmax, want_values=True, want_codes=True)
    _check_channel_results([big], [r], tab, qmax)
    plan.close()


def _status():
    from voyager_compiler_b200 import _lib
    return _lib.lib.vq_channel_status()


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["stream", "pipe"])
def test_pipeline_wait_that_runs_out_is_reported_and_the_context_stays_usable(kernel, monkeypatch):
    """The bounded waits of the bulk-copy pipeline: with one batch left out by the producer (a test hook)
    and a budget of about a millisecond, the consumers of that batch give up, the kernel records it and
    returns in order; the next, untouched launch on the same context is correct again."""
    from voyager_compiler_b200 import _lib
    torch.manual_seed(3)
    ws = [torch.randn(512, 4608) * 0.05, torch.randn(1024, 1024) * 0.05]
    dev = [w.cuda() for w in ws]
    tab = golden_table("posit8_1")
    assert _lib.lib.vq_channel_status() == 0
    monkeypatch.setenv("VOYAGER_B200_CHANNEL_KERNEL", kernel)
    monkeypatch.setenv("VOYAGER_B200_CHANNEL_SKIP_BATCH", "7")
    monkeypatch.setenv("VOYAGER_B200_CHANNEL_WAIT_CYCLES", "2000000")
    broken = mq.ChannelQuantPlan(dev, tab, 4096.0, want_values=True, want_codes=True, want_dequant=True)
    broken.run()
    torch.cuda.synchronize()                                   # returns: nothing hangs
    assert _lib.lib.vq_channel_status() in (21, 22, 31, 32, 33)   # producer or consumer side, whichever gave up first
    assert _lib.lib.vq_channel_status() == 0                   # read once, cleared
    broken.close()
    monkeypatch.delenv("VOYAGER_B200_CHANNEL_SKIP_BATCH")
    monkeypatch.delenv("VOYAGER_B200_CHANNEL_WAIT_CYCLES")
    plan = mq.ChannelQuantPlan(dev, tab, 4096.0, want_values=True, want_codes=True, want_dequant=True)
    _check_channel_results(ws, plan.run(), tab, 4096.0)
    assert _lib.lib.vq_channel_status() == 0
    plan.close()


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["stream", "pipe", "sweep"])
@pytest.mark.parametrize("outputs", [dict(want_values=True, want_codes=False, want_dequant=False),
                                     dict(want_values=False, want_codes=True, want_dequant=False),
                                     dict(want_values=False, want_codes=False, want_dequant=True),
                                     dict(want_values=False, want_codes=False, want_dequant=False, want_amax=True)])
def test_per_channel_kernels_with_every_single_output(kernel, outputs, monkeypatch):
    """One output at a time (the kernels predicate their stores on it), and the maxima / scales alone; large enough
    for the bulk-copy kernels, channel lengths that are and are not multiples of 128."""
    monkeypatch.setenv("VOYAGER_B200_CHANNEL_KERNEL", kernel)
    g = torch.Generator().manual_seed(23)
    ws = [torch.randn(700, 2304, generator=g) * 0.05, torch.randn(512, 576, generator=g) * 0.05, torch.randn(3000, 256, generator=g)]
    ws[0][5] = 0
    tab = golden_table("posit8_1")
    got = mq.quantize_tensors_per_channel([w.cuda() for w in ws], tab, 4096.0, **outputs)
    for w, r in zip(ws, got):
        s_ref = vo.channel_scale(w, 4096.0)
        q_ref = vo.quantize(w, s_ref, None, None, None, tab)
        assert same_bits(r.scale, s_ref)[0]
        if outputs.get("want_amax"):
            assert same_bits(r.amax, w.abs().amax(dim=1, keepdim=True))[0]
        if outputs["want_values"]:
            assert same_bits(r.values, q_ref)[0]
        if outputs["want_dequant"]:
            assert same_bits(r.dequant, vo.dequantize(q_ref, s_ref))[0]
        if outputs["want_codes"]:
            lv = r.levels[r.codes.cpu().long().clamp(max=r.levels.numel() - 1)]
            assert torch.equal(lv, q_ref.float())
    assert _status() == 0
