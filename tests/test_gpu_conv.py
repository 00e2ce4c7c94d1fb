"""conv2d_mx on the library's own GEMM (patch matrix + tcgen05 contraction) against the CPU oracle
(oracle/voyager_oracle.py: conv2d_mx, following ops/quantized.py:239-283), and the patch matrix itself
against torch's unfold, bit for bit."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "oracle"))
import voyager_oracle as vo  # noqa: E402

import voyager_compiler_b200 as vb  # noqa: E402
from voyager_compiler_b200 import _lib  # noqa: E402

pytestmark = pytest.mark.gpu

# (N, C, H, W, O, kh, kw, stride, padding, dilation)
SHAPES = [
    (2, 64, 14, 14, 128, 1, 1, 1, 0, 1),          # pointwise: no patch matrix for NHWC
    (2, 64, 15, 13, 96, 3, 3, 1, 1, 1),
    (3, 32, 16, 16, 64, 3, 3, 2, 1, 1),
    (2, 3, 33, 35, 64, 7, 7, 2, 3, 1),            # K = 147, padded to 152
    (1, 24, 12, 12, 40, 3, 3, 1, 2, 2),           # dilation
    (2, 128, 8, 8, 256, 1, 1, 2, 0, 1),           # strided pointwise (downsample)
    (1, 40, 9, 11, 48, (3, 1), (3, 1), (1, 2), (1, 0), 1),
    (2, 20, 7, 7, 30, 5, 5, 1, 2, 1),             # C not a multiple of 8
]


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def _case(shape, seed):
    N, C, H, W, O, kh, kw, st, pd, dl = shape
    kh = kh[0] if isinstance(kh, tuple) else kh
    kw = kw[1] if isinstance(kw, tuple) else kw
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, C, H, W, generator=g).bfloat16()
    w = (torch.randn(O, C, kh, kw, generator=g) * 0.1).bfloat16()
    b = torch.randn(O, generator=g).bfloat16()
    return x, w, b, _pair(st), _pair(pd), _pair(dl)


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("shape", SHAPES, ids=[str(i) for i in range(len(SHAPES))])
def test_conv2d_mx_matches_oracle(shape, layout):
    x, w, b, st, pd, dl = _case(shape, 11)
    if layout == "nhwc":
        x, w = x.permute(0, 2, 3, 1).contiguous(), w.permute(2, 3, 1, 0).contiguous()
    want = vo.conv2d_mx(x.float(), w.float(), b.float(), st, pd, dl, 1, layout=layout)
    before = _lib.launch_count()
    got = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), st, pd, dl, 1, layout=layout)
    torch.cuda.synchronize()
    assert _lib.launch_count() > before, "no kernel of this library was launched"
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == tuple(want.shape)
    rel = (got.float().cpu().double() - want.double()).norm() / want.double().norm()
    assert rel <= 1e-2, rel            # tolerance of the fp32-accumulate bf16 contraction
    from voyager_compiler_b200.gemm_native import gemm_status
    assert gemm_status("cuda") == 0


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("C,k,s,p", [(64, 3, 1, 1), (48, 1, 1, 0), (96, 1, 2, 0), (40, 3, 2, 1), (20, 3, 1, 1)])
def test_conv2d_mx_with_block_scales(layout, C, k, s, p):
    """Codes and power-of-two block scales along the channel axis, as the MX flow annotates convolutions
    (quantization/quantize_pt2e.py:111-113): axis 1 of NCHW tensors, the last axis of NHWC activations."""
    from golden_util import golden_table
    g = torch.Generator().manual_seed(5)
    N, H, W, O = 2, 10, 10, 96
    x = torch.randn(N, C, H, W, generator=g).bfloat16()
    w = (torch.randn(O, C, k, k, generator=g) * 0.05).bfloat16()
    q = golden_table("int8")
    if layout == "nhwc":
        x, w = x.permute(0, 2, 3, 1).contiguous(), w.permute(2, 3, 1, 0).contiguous()
        ax_x, ax_w = (3,), (2,)
    else:
        ax_x, ax_w = (1,), (1,)
    xs, xq = vo.quantize_mx(x, q, ax_x, 32, 127.0, True)
    ws, wq = vo.quantize_mx(w, q, ax_w, 32, 127.0, True)
    want = vo.conv2d_mx(xq.float(), wq.float(), None, s, p, 1, 1, input_scale=xs.float(), weight_scale=ws.float(), block_size=32,
                        layout=layout)
    got = torch.ops.quantized_ops.conv2d_mx(xq.cuda(), wq.cuda(), None, (s, s), (p, p), (1, 1), 1, input_scale=xs.cuda(), weight_scale=ws.cuda(),
                                            block_size=32, layout=layout)
    rel = (got.float().cpu().double() - want.double()).norm() / want.double().norm()
    assert rel <= 1e-2, rel
    # the cached weight matrix must follow an in-place change of the weight
    wq2 = wq.cuda()
    a = torch.ops.quantized_ops.conv2d_mx(xq.cuda(), wq2, None, (s, s), (p, p), (1, 1), 1, input_scale=xs.cuda(), weight_scale=ws.cuda(),
                                          block_size=32, layout=layout)
    wq2.mul_(2)
    b = torch.ops.quantized_ops.conv2d_mx(xq.cuda(), wq2, None, (s, s), (p, p), (1, 1), 1, input_scale=xs.cuda(), weight_scale=ws.cuda(),
                                          block_size=32, layout=layout)
    assert torch.allclose(b.float(), 2 * a.float(), rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("I,k,scaled", [(64, 3, True), (64, 3, False), (96, 1, True), (40, 3, False), (32, 7, True)])
def test_weight_matrix_one_pass_equals_decode_and_permute(layout, I, k, scaled):
    """The [O, K] weight written by one launch of the patch kernel equals dequantize + permute + pad, bit for bit."""
    from voyager_compiler_b200 import conv_native, ops
    g = torch.Generator().manual_seed(9)
    O = 72
    w = (torch.randn(O, I, k, k, generator=g) * 0.05).bfloat16()
    ws = None
    if scaled:
        ws = torch.exp2(torch.randint(-9, -3, (O, -(-I // 32), k, k), generator=g).float()).bfloat16()
    if layout == "nhwc":
        w = w.permute(2, 3, 1, 0).contiguous()
        ws = None if ws is None else ws.permute(2, 3, 1, 0).contiguous()
    w, ws = w.cuda(), None if ws is None else ws.cuda()
    got = conv_native._weight_matrix_one_pass(w, ws, None, 32 if scaled else None, layout)
    assert got is not None
    wd = ops._decode_operand("conv2d_mx", w, None, ws, 32 if scaled else None)
    want = (wd.permute(0, 2, 3, 1) if layout == "nchw" else wd.permute(3, 0, 1, 2)).reshape(O, -1)
    assert torch.equal(got[:, :want.shape[1]].view(torch.int16), want.contiguous().view(torch.int16))


def test_vendor_switch_and_other_dtypes_agree(monkeypatch):
    x, w, b, st, pd, dl = _case(SHAPES[1], 3)
    a = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), st, pd, dl, 1)
    monkeypatch.setenv("VOYAGER_B200_CONV", "vendor")
    v = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), st, pd, dl, 1)
    rel = (a.float() - v.float()).norm() / v.float().norm()
    assert rel <= 1e-2, rel
    monkeypatch.delenv("VOYAGER_B200_CONV")
    f = torch.ops.quantized_ops.conv2d_mx(x.float().cuda(), w.float().cuda(), b.float().cuda(), st, pd, dl, 1)   # fp32: vendor kernel
    assert f.dtype == torch.float32
    rel = (a.float() - f).norm() / f.norm()
    assert rel <= 1e-2, rel


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("channels_last", [False, True])
@pytest.mark.parametrize("shape", SHAPES, ids=[str(i) for i in range(len(SHAPES))])
def test_patch_matrix_bit_exact(shape, channels_last, dtype):
    x, w, b, st, pd, dl = _case(shape, 23)
    N, C, H, W = x.shape
    kh, kw = w.shape[2], w.shape[3]
    x = x.to(dtype)
    cols = torch.nn.functional.unfold(x.float(), (kh, kw), dilation=dl, padding=pd, stride=st)       # [N, C*kh*kw, L]
    L = cols.shape[-1]
    want = cols.view(N, C, kh * kw, L).permute(0, 3, 2, 1).reshape(N * L, kh * kw * C).to(dtype)
    K = kh * kw * C
    ldk = (K + 7) // 8 * 8 + 8                                    # padding columns must come back zero
    xd = x.cuda()
    if channels_last:
        xd = xd.permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)
    sn, sc, sh, sw = xd.stride()
    out = torch.full((N * L, ldk), 7.0, dtype=dtype, device="cuda")
    _lib.check(_lib.lib.vq_conv_patches(xd.data_ptr(), _lib.VQ_BF16 if dtype == torch.bfloat16 else _lib.VQ_F32, N, H, W, C,
                                        sn, sh, sw, sc, kh, kw, st[0], st[1], pd[0], pd[1], dl[0], dl[1], None, 0, 0, 0, 0, 0, out.data_ptr(), ldk,
                                        torch.cuda.current_stream().cuda_stream), "patches")
    got = out.cpu()
    assert torch.equal(got[:, :K], want)
    assert bool((got[:, K:] == 0).all())


def test_patch_matrix_rejects_bad_arguments():
    x = torch.zeros(1, 4, 4, 8, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(16, 8, dtype=torch.bfloat16, device="cuda")
    rc = _lib.lib.vq_conv_patches(x.data_ptr(), _lib.VQ_BF16, 1, 4, 4, 8, 128, 32, 8, 1, 7, 7, 1, 1, 0, 0, 1, 1, None, 0, 0, 0, 0, 0, out.data_ptr(), 392, None)
    assert rc < 0                                                  # window larger than the image
    rc = _lib.lib.vq_conv_patches(x.data_ptr(), _lib.VQ_BF16, 1, 4, 4, 8, 128, 32, 8, 1, 1, 1, 1, 1, 0, 0, 1, 1, None, 0, 0, 0, 0, 0, out.data_ptr(), 4, None)
    assert rc < 0                                                  # ldk below kh * kw * C
