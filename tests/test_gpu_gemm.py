"""tcgen05 GEMM: plain (TMA-fed) and fused-dequant variants against torch / the CPU oracle."""
import os
import sys

import pytest
import torch

import voyager_compiler_b200 as vb
from voyager_compiler_b200 import _lib, gemm_native
from golden_util import golden_table

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import voyager_oracle as vo  # noqa: E402

pytestmark = pytest.mark.gpu
Q = torch.ops.quantized_ops


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / b.norm()).item()


def _plain(a, b, bias=None):
    M, K = a.shape
    N = b.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    st = torch.zeros(1, dtype=torch.int32, device=a.device)
    rc = _lib.lib.vq_gemm_bf16_tn(a.data_ptr(), b.data_ptr(), bias.data_ptr() if bias is not None else None,
                                  out.data_ptr(), M, N, K, st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "gemm")
    torch.cuda.synchronize()
    assert st.item() == 0, f"kernel reported a wait that ran out: {st.item()}"
    return out


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (384, 768, 4096), (100, 200, 72),
                                   (1, 8, 8), (130, 257, 136), (1024, 2816, 512)])
def test_plain_gemm_matches_fp32_reference(M, N, K):
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    got = _plain(a, b)
    ref = a.float() @ b.float().t()           # plain fp32 reference of the same contraction
    assert _rel(got, ref) <= 4e-3             # bf16 output rounding only (2^-9 per element)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    got = _plain(a, b, bias)
    assert _rel(got, ref + bias.float()) <= 4e-3


def test_plain_gemm_exact_on_small_integers():
    """Integer-valued operands: every product and partial sum is exact in fp32, so any wrong
    descriptor, swizzle or accumulate flag shows up as an exact mismatch."""
    torch.manual_seed(0)
    a = torch.randint(-3, 4, (256, 192), device="cuda").to(torch.bfloat16)
    b = torch.randint(-3, 4, (512, 192), device="cuda").to(torch.bfloat16)
    got = _plain(a, b)
    ref = (a.float() @ b.float().t()).to(torch.bfloat16)
    assert torch.equal(got, ref)


def _mx_operands(M, N, K, seed=4):
    torch.manual_seed(seed)
    x = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.02).to(torch.bfloat16)
    q = golden_table("int8")
    xs, xq = vo.quantize_mx(x, q, (-1,), 32, 127.0, True)
    ws, wq = vo.quantize_mx(w, q, (-1,), 32, 127.0, True)
    return xq, xs, wq, ws


@pytest.mark.parametrize("mode", ["fused", "plain"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 512), (300, 1000, 1024), (2048, 2816, 4096)])
def test_linear_mx_against_oracle(mode, M, N, K):
    xq, xs, wq, ws = _mx_operands(M, N, K)
    want = vo.linear_mx(xq, wq, None, input_scale=xs, weight_scale=ws, block_size=32)
    os.environ["VOYAGER_B200_GEMM"] = mode
    try:
        got = Q.linear_mx(xq.cuda(), wq.cuda(), None, input_scale=xs.cuda(), weight_scale=ws.cuda(), block_size=32)
        torch.cuda.synchronize()
    finally:
        del os.environ["VOYAGER_B200_GEMM"]
    assert gemm_native.gemm_status("cuda") == 0
    assert got.dtype == torch.bfloat16 and got.shape == want.shape
    assert _rel(got, want) <= 1e-2            # tolerance for the bf16 / fp32-accumulate linear


def test_fused_equals_plain_bitwise():
    """int8 x 2^e is exact in bf16, so the fused staging must build the very same operands as
    the dequantize kernel; same MMA order -> identical results."""
    xq, xs, wq, ws = _mx_operands(512, 768, 2048, seed=9)
    outs = {}
    for mode in ("fused", "plain"):
        os.environ["VOYAGER_B200_GEMM"] = mode
        try:
            outs[mode] = Q.linear_mx(xq.cuda(), wq.cuda(), None, input_scale=xs.cuda(), weight_scale=ws.cuda(), block_size=32)
        finally:
            del os.environ["VOYAGER_B200_GEMM"]
    os.environ["VOYAGER_B200_GEMM"], os.environ["VOYAGER_B200_FUSED_STAGING"] = "fused", "regs"
    try:            # the register-staged variant of the CTA-pair kernel (ragged last row tile included: 512 + 100 rows)
        outs["regs"] = Q.linear_mx(xq.cuda(), wq.cuda(), None, input_scale=xs.cuda(), weight_scale=ws.cuda(), block_size=32)
        x2, s2 = torch.cat([xq, xq[:100]]), torch.cat([xs, xs[:100]])
        regs2 = Q.linear_mx(x2.cuda(), wq.cuda(), None, input_scale=s2.cuda(), weight_scale=ws.cuda(), block_size=32)
    finally:
        del os.environ["VOYAGER_B200_GEMM"], os.environ["VOYAGER_B200_FUSED_STAGING"]
    torch.cuda.synchronize()
    assert torch.equal(outs["fused"], outs["plain"])
    assert torch.equal(outs["regs"], outs["plain"])
    assert torch.equal(regs2[:512], outs["plain"]) and torch.equal(regs2[512:], outs["plain"][:100])


def test_fused_with_bias_and_3d_input():
    xq, xs, wq, ws = _mx_operands(6 * 50, 320, 256, seed=11)
    bias = torch.randn(320).to(torch.bfloat16)
    x3, s3 = xq.reshape(6, 50, 256), xs.reshape(6, 50, 8)
    want = vo.linear_mx(x3, wq, bias, input_scale=s3, weight_scale=ws, block_size=32)
    got = Q.linear_mx(x3.cuda(), wq.cuda(), bias.cuda(), input_scale=s3.cuda(), weight_scale=ws.cuda(), block_size=32)
    assert got.shape == (6, 50, 320) and _rel(got, want) <= 1e-2
    assert gemm_native.gemm_status("cuda") == 0


@pytest.mark.parametrize("M,N,K", [(2048, 2304, 4096), (512, 768, 2048), (612, 300, 512), (8192, 1024, 256), (64, 256, 512), (300, 256, 320)])
def test_packed_operands_equal_the_float_code_path_bitwise(M, N, K):
    """int8 bytes + bf16 scales through the packed GEMM (conversion inside the operand staging) against
    the float-code linear_mx: int8 x 2^e is exact in bf16 and the MMA order is the same."""
    from voyager_compiler_b200 import gemm_native, model_quant as mq
    from golden_util import golden_table
    torch.manual_seed(M + N + K)
    q = golden_table("int8")
    x = torch.randn(M, K).to(torch.bfloat16)
    x[0, :32] = 0
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N).to(torch.bfloat16)
    (px,) = mq.quantize_tensors_mx([x.cuda()], q, 32, 127.0, True, code_bits=8)
    (pw,) = mq.quantize_tensors_mx([w.cuda()], q, 32, 127.0, True, code_bits=8)
    got = gemm_native.linear_mx_packed(px, pw, bias.cuda())
    xs, xq = Q.quantize_mx(x.cuda(), q.cuda(), (-1,), 32, 127.0, True)
    ws, wq = Q.quantize_mx(w.cuda(), q.cuda(), (-1,), 32, 127.0, True)
    want = Q.linear_mx(xq, wq, bias.cuda(), input_scale=xs, weight_scale=ws, block_size=32)
    torch.cuda.synchronize()
    assert gemm_native.gemm_status() == 0
    assert torch.equal(got, want)


@pytest.mark.parametrize("table,qmax,pow2", [("int8", 127.0, True), ("int8", 127.0, False), ("fp8_e4m3", 448.0, True)])
@pytest.mark.parametrize("shape,N", [((300, 256), 520), ((2, 65, 136), 96), ((1, 64), 8)])
def test_linear_mx_dynamic_equals_quantize_mx_then_linear_mx(table, qmax, pow2, shape, N):
    """Activation quantized on the fly inside one pass == the quantize_mx + linear_mx node pair, bit for bit,
    and both within the linear's tolerance of the CPU oracle."""
    g = torch.Generator().manual_seed(sum(shape) + N)
    K = shape[-1]
    x = torch.randn(*shape, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    bias = torch.randn(N, generator=g).bfloat16()
    q = golden_table(table)
    ws, wq = vo.quantize_mx(w, q, (-1,), 32, qmax, pow2)
    xs, xq = vo.quantize_mx(x, q, (-1,), 32, qmax, pow2)
    want = vo.linear_mx(xq, wq, bias, input_scale=xs, weight_scale=ws, block_size=32)
    qc, wqc, wsc, bc, xc = q.cuda(), wq.cuda(), ws.cuda(), bias.cuda(), x.cuda()
    s2, q2 = Q.quantize_mx(xc, qc, (-1,), 32, qmax, pow2)
    two_ops = Q.linear_mx(q2, wqc, bc, input_scale=s2, weight_scale=wsc, block_size=32)
    got = gemm_native.linear_mx_dynamic(xc, wqc, bc, qmap=qc, weight_scale=wsc, block_size=32, quant_max=qmax,
                                        force_scale_power_of_two=pow2)
    assert gemm_native.gemm_status("cuda") == 0
    assert got.shape == two_ops.shape == want.shape
    assert torch.equal(got.view(torch.int16), two_ops.view(torch.int16))
    assert _rel(got.float(), want.float()) <= 1e-2


@pytest.mark.gpu
def test_status_word_is_one_per_device_however_the_device_is_named(monkeypatch):
    """``cuda``, ``cuda:0`` and a ``torch.device`` name the same word, so a wait that ran out is
    seen by whoever asks; with VOYAGER_B200_GEMM_CHECK=1 the next native GEMM call raises."""
    from voyager_compiler_b200 import _lib, gemm_native
    torch.cuda.set_device(0)
    word = gemm_native._status_tensor(torch.device("cuda:0"))
    assert gemm_native._status_tensor("cuda") is word and gemm_native._status_tensor(torch.device("cuda")) is word
    word.fill_(3)                                   # what the epilogue role writes when its wait runs out
    assert gemm_native.gemm_status("cuda") == 3
    assert gemm_native.gemm_status("cuda:0") == 0   # read once, cleared
    with pytest.raises(ValueError):
        gemm_native.gemm_status("cpu")
    monkeypatch.setenv("VOYAGER_B200_GEMM_CHECK", "1")
    a = torch.randn(256, 64, device="cuda").bfloat16()
    b = torch.randn(256, 64, device="cuda").bfloat16()
    y = gemm_native.native_mx_gemm(a, b, None, None, None, None, None, None)
    assert y.shape == (256, 256)
    word.fill_(2)
    with pytest.raises(_lib.VoyagerB200Error, match="bounded wait"):
        gemm_native.native_mx_gemm(a, b, None, None, None, None, None, None)


def _no_vendor_gemm(monkeypatch):
    """The contraction must run on this library's kernel: any route into the vendor GEMM fails the test."""
    def boom(*a, **k):
        raise AssertionError("the vendor GEMM was called")
    monkeypatch.setattr(torch, "matmul", boom)
    monkeypatch.setattr(torch.nn.functional, "linear", boom)


def _mx_pair(a_shape, b_shape, seed, b_axis):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(*a_shape, generator=g).to(torch.bfloat16)
    b = (torch.randn(*b_shape, generator=g) * 0.05).to(torch.bfloat16)
    q = golden_table("int8")
    sa, qa = vo.quantize_mx(a, q, (-1,), 32, 127.0, True)
    sb, qb = vo.quantize_mx(b, q, (b_axis,), 32, 127.0, True)
    return qa, sa, qb, sb


@pytest.mark.parametrize("a_shape,b_shape", [
    ((2, 3, 256, 64), (2, 3, 64, 256)),        # attention scores: Q [B,H,S,D] x K^T [B,H,D,S]
    ((2, 3, 256, 256), (2, 3, 256, 64)),       # attention output: P [B,H,S,S] x V [B,H,S,D]
    ((4, 1, 128), (4, 128, 320)),              # decode step: one query row per batch (one-CTA tile)
    ((5, 200, 96), (5, 96, 130)),              # ragged: tiles reach into the next batch and are masked
    ((3, 300, 64), (64, 512)),                 # right operand shared by all batches
    ((300, 64), (64, 512)),
])
def test_matmul_mx_runs_on_the_native_gemm(a_shape, b_shape, monkeypatch):
    """``matmul_mx`` with the right operand in [.., K, N] order and block scales along K (ops/quantized.py:363-432):
    decode + transpose kernel, then the tcgen05 GEMM over all batches in one launch."""
    qa, sa, qb, sb = _mx_pair(a_shape, b_shape, sum(a_shape) + sum(b_shape), -2)
    want = vo.matmul_mx(qa, qb, input_scale=sa, weight_scale=sb, block_size=32)
    before = _lib.launch_count()
    _no_vendor_gemm(monkeypatch)
    got = Q.matmul_mx(qa.cuda(), qb.cuda(), input_scale=sa.cuda(), weight_scale=sb.cuda(), block_size=32)
    torch.cuda.synchronize()
    monkeypatch.undo()
    assert _lib.launch_count() >= before + 3          # decode of a, decode + transpose of b, the GEMM
    assert gemm_native.gemm_status("cuda") == 0
    assert got.shape == want.shape and got.dtype == torch.bfloat16
    assert _rel(got, want) <= 1e-2


def test_matmul_mx_kc_layout_batched_and_plain_operands(monkeypatch):
    """Batched right operand already in [.., N, K] order (weight_layout="kc"), and operands without scales."""
    qa, sa, qb, sb = _mx_pair((2, 2, 160, 64), (2, 2, 288, 64), 5, -1)
    want = vo.matmul_mx(qa, qb, input_scale=sa, weight_scale=sb, block_size=32, weight_layout="kc")
    g = torch.Generator().manual_seed(6)
    a = torch.randn(3, 40, 72, generator=g).bfloat16()
    b = torch.randn(3, 72, 50, generator=g).bfloat16()
    want2 = vo.matmul_mx(a, b)
    _no_vendor_gemm(monkeypatch)
    got = Q.matmul_mx(qa.cuda(), qb.cuda(), input_scale=sa.cuda(), weight_scale=sb.cuda(), block_size=32, weight_layout="kc")
    got2 = Q.matmul_mx(a.cuda(), b.cuda())
    torch.cuda.synchronize()
    monkeypatch.undo()
    assert gemm_native.gemm_status("cuda") == 0
    assert got.shape == want.shape and _rel(got, want) <= 1e-2
    assert got2.shape == want2.shape and _rel(got2, want2) <= 1e-2


def test_linear_mx_ck_weight_runs_on_the_native_gemm(monkeypatch):
    """``linear_mx(..., weight_layout="ck")``: the weight is stored [K, N] with block scales along K
    (ops/quantized.py:330-333); bias and a 3-D activation included; a codebook on the weight."""
    qa, sa, qb, sb = _mx_pair((4, 75, 128), (128, 384), 21, -2)
    bias = torch.randn(384).to(torch.bfloat16)
    want = vo.linear_mx(qa, qb, bias, input_scale=sa, weight_scale=sb, block_size=32, weight_layout="ck")
    code = torch.linspace(-1, 1, 16).to(torch.bfloat16)
    idx = torch.randint(0, 16, (128, 384)).to(torch.bfloat16)
    want_c = vo.linear_mx(qa, idx, None, input_scale=sa, weight_scale=sb, block_size=32, weight_code=code, weight_layout="ck")
    _no_vendor_gemm(monkeypatch)
    dev = [t.cuda() for t in (qa, sa, qb, sb, bias, idx, code)]
    got = Q.linear_mx(dev[0], dev[2], dev[4], input_scale=dev[1], weight_scale=dev[3], block_size=32, weight_layout="ck")
    again = Q.linear_mx(dev[0], dev[2], dev[4], input_scale=dev[1], weight_scale=dev[3], block_size=32, weight_layout="ck")
    got_c = Q.linear_mx(dev[0], dev[5], None, input_scale=dev[1], weight_scale=dev[3], block_size=32, weight_code=dev[6],
                        weight_layout="ck")
    torch.cuda.synchronize()
    monkeypatch.undo()
    assert gemm_native.gemm_status("cuda") == 0
    assert got.shape == want.shape == (4, 75, 384) and _rel(got, want) <= 1e-2
    assert torch.equal(got, again)                    # second call: the decoded weight comes from the cache
    assert _rel(got_c, want_c) <= 1e-2


def test_dequantize_transpose_equals_dequantize_then_transpose():
    g = torch.Generator().manual_seed(8)
    for batch, K, N in ((1, 64, 64), (3, 96, 130), (2, 200, 66), (1, 4096, 1024)):
        x = torch.randn(batch, K, N, generator=g).bfloat16().cuda()
        s = (torch.rand(batch, -(-K // 32), N, generator=g) + 0.5).bfloat16().cuda()
        want = Q.dequantize(x, s, None, (-2,), 32).transpose(-1, -2).contiguous()
        got = gemm_native._decode_transposed("test", x, None, s, 32)
        assert torch.equal(got, want), (batch, K, N)
        assert torch.equal(gemm_native._decode_transposed("test", x, None, None, None), x.transpose(-1, -2).contiguous())


def _mx_pair_f32(a_shape, b_shape, seed, b_axis, pow2=True):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(*a_shape, generator=g)
    b = torch.randn(*b_shape, generator=g) * 0.05
    q = golden_table("int8")
    sa, qa = vo.quantize_mx(a, q, (-1,), 32, 127.0, pow2)
    sb, qb = vo.quantize_mx(b, q, (b_axis,), 32, 127.0, pow2)
    return qa, sa, qb, sb


@pytest.mark.parametrize("pow2,tol", [(True, 1e-5), (False, 2e-3)])
@pytest.mark.parametrize("a_shape,N", [((300, 256), 200), ((2, 70, 132), 520), ((64,), 96)])
def test_fp32_linear_mx_runs_on_the_tensor_cores_as_tf32(a_shape, N, pow2, tol, monkeypatch):
    """fp32 operands (ops/quantized.py:295-348 on fp32 tensors): decoded by this library, contracted as tf32 with
    fp32 accumulation.  Codes times power-of-two scales are exact in tf32, so only the summation order differs
    from the fp32 oracle; arbitrary fp32 scales lose the low 13 bits of every decoded operand."""
    K = a_shape[-1]
    qa, sa, qb, sb = _mx_pair_f32(a_shape, (N, K), 40 + N, -1, pow2)
    bias = torch.randn(N)
    want = vo.linear_mx(qa, qb, bias, input_scale=sa, weight_scale=sb, block_size=32)
    before = _lib.launch_count()
    _no_vendor_gemm(monkeypatch)
    got = Q.linear_mx(qa.cuda(), qb.cuda(), bias.cuda(), input_scale=sa.cuda(), weight_scale=sb.cuda(), block_size=32)
    torch.cuda.synchronize()
    monkeypatch.undo()
    assert _lib.launch_count() >= before + 2
    assert gemm_native.gemm_status("cuda") == 0
    assert got.dtype == torch.float32 and got.shape == want.shape
    assert _rel(got, want) <= tol


@pytest.mark.parametrize("a_shape,b_shape", [((2, 3, 130, 64), (2, 3, 64, 200)), ((3, 90, 64), (64, 300)), ((150, 96), (96, 72))])
def test_fp32_matmul_mx_runs_on_the_tensor_cores_as_tf32(a_shape, b_shape, monkeypatch):
    qa, sa, qb, sb = _mx_pair_f32(a_shape, b_shape, 77, -2)
    want = vo.matmul_mx(qa, qb, input_scale=sa, weight_scale=sb, block_size=32)
    _no_vendor_gemm(monkeypatch)
    got = Q.matmul_mx(qa.cuda(), qb.cuda(), input_scale=sa.cuda(), weight_scale=sb.cuda(), block_size=32)
    torch.cuda.synchronize()
    monkeypatch.undo()
    assert gemm_native.gemm_status("cuda") == 0
    assert got.dtype == torch.float32 and got.shape == want.shape
    assert _rel(got, want) <= 1e-5


def test_fp32_vendor_switch(monkeypatch):
    qa, sa, qb, sb = _mx_pair_f32((64, 128), (96, 128), 3, -1)
    a = Q.linear_mx(qa.cuda(), qb.cuda(), None, input_scale=sa.cuda(), weight_scale=sb.cuda(), block_size=32)
    monkeypatch.setenv("VOYAGER_B200_FP32", "vendor")
    b = Q.linear_mx(qa.cuda(), qb.cuda(), None, input_scale=sa.cuda(), weight_scale=sb.cuda(), block_size=32)
    assert _rel(a, b.cpu()) <= 1e-5


@pytest.mark.parametrize("stores", ["tiles", "rows"])
@pytest.mark.parametrize("M,N,K,ldy,col0,n_out", [(512, 512, 256, 1280, 256, 3), (300, 384, 128, 1024, 512, 2), (1000, 200, 64, 456, 256, 4),
                                                  (256, 256, 64, 256, 0, 8)])
def test_scatter_gemm_writes_its_columns_into_every_output_buffer(M, N, K, ldy, col0, n_out, stores, monkeypatch):
    """``vq_gemm_bf16_tn_scatter`` (the epilogue of the column-parallel linear): the [M, N] result goes to columns
    [col0, col0 + N) of every output buffer, here several buffers on one GPU; whole 128 x 64 sub-tiles by tensor
    stores or one bulk copy per row, partial tiles by plain stores; nothing outside the column range is touched."""
    import ctypes
    monkeypatch.setenv("VOYAGER_B200_SCATTER_STORES", stores)
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).bfloat16().cuda()
    b = (torch.randn(N, K, generator=g) * 0.1).bfloat16().cuda()
    bias = torch.randn(N, generator=g).bfloat16().cuda()
    outs = [torch.full((M, ldy), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(n_out)]
    ptrs = (ctypes.c_void_p * n_out)(*[o.data_ptr() for o in outs])
    st = gemm_native._status_tensor(torch.device("cuda"))
    rc = _lib.lib.vq_gemm_bf16_tn_scatter(a.data_ptr(), b.data_ptr(), bias.data_ptr(), ptrs, n_out, ldy, col0, M, N, K, st.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "scatter")
    torch.cuda.synchronize()
    assert gemm_native.gemm_status("cuda") == 0
    want = (a.float() @ b.float().t() + bias.float()).bfloat16()
    for o in outs:
        assert torch.equal(o[:, col0:col0 + N].view(torch.int16), outs[0][:, col0:col0 + N].view(torch.int16))
        assert bool((o[:, :col0] == 7).all()) and bool((o[:, col0 + N:] == 7).all())
    rel = (outs[0][:, col0:col0 + N].float() - want.float()).norm() / want.float().norm()
    assert rel <= 5e-3, rel
