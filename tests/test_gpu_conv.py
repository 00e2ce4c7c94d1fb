"""conv2d_mx on the library's own tensor-core kernels (implicit GEMM, or patch matrix + contraction for the
channel counts the implicit form does not take) against the CPU oracle (oracle/voyager_oracle.py: conv2d_mx,
following ops/quantized.py:239-283), grouped convolutions included, and the patch matrix itself against
torch's unfold, bit for bit."""
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


# (N, C, H, W, O, k, stride, padding, groups): tile widths 64 / 128 / 256, partial tiles in every direction,
# several tiles per CTA, channel counts below and above one 64-channel step
BIG = [
    (4, 64, 28, 28, 320, 3, 1, 1, 1),             # 128-wide tiles, the last one partial
    (8, 64, 56, 56, 512, 3, 1, 1, 1),             # 256-wide tiles, more tiles than SMs
    (2, 96, 17, 19, 64, 3, 2, 1, 1),              # 64-wide tile; 96 channels = one and a half steps per tap
    (2, 200, 9, 9, 136, 1, 1, 0, 1),              # pointwise through the gather; 200 = 3 steps + 8 channels
    (2, 64, 12, 12, 96, 3, 1, 1, 2),              # two groups of 32 -> 48
    (3, 128, 10, 10, 128, 3, 1, 1, 8),            # eight groups of 16 -> 16
    (2, 48, 14, 14, 48, 5, 2, 2, 6),              # six groups of 8 -> 8
    (1, 512, 7, 7, 512, 3, 1, 1, 1),              # deep K (72 steps), few pixels
]


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("shape", BIG, ids=[str(i) for i in range(len(BIG))])
def test_implicit_gemm_convolution_matches_oracle(shape, layout, monkeypatch):
    N, C, H, W, O, k, st, pd, groups = shape
    g = torch.Generator().manual_seed(31)
    x = torch.randn(N, C, H, W, generator=g).bfloat16()
    w = (torch.randn(O, C // groups, k, k, generator=g) * 0.05).bfloat16()
    b = torch.randn(O, generator=g).bfloat16()
    if layout == "nhwc":
        x = x.permute(0, 2, 3, 1).contiguous()
        if groups == 1:                                          # a grouped convolution keeps its weight OIHW
            w = w.permute(2, 3, 1, 0).contiguous()
    want = vo.conv2d_mx(x.float(), w.float(), b.float(), st, pd, 1, groups, layout=layout)
    before = _lib.launch_count()
    got = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), (st, st), (pd, pd), (1, 1), groups, layout=layout)
    torch.cuda.synchronize()
    launches = _lib.launch_count() - before
    assert launches >= 1
    assert got.dtype == torch.bfloat16 and tuple(got.shape) == tuple(want.shape)
    rel = (got.float().cpu().double() - want.double()).norm() / want.double().norm()
    assert rel <= 1e-2, rel
    from voyager_compiler_b200.gemm_native import gemm_status
    assert gemm_status("cuda") == 0
    if groups == 1:
        # the explicit form (patch matrix in memory) computes the same sums in the same order
        monkeypatch.setenv("VOYAGER_B200_CONV", "patches")
        ref = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), (st, st), (pd, pd), (1, 1), groups, layout=layout)
        rel2 = (got.float() - ref.float()).norm() / ref.float().norm()
        assert rel2 <= 1e-3, rel2


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("C,O,groups,k", [(64, 64, 2, 3), (128, 96, 4, 1), (64, 128, 1, 3)])
def test_implicit_gemm_convolution_with_block_scales_and_groups(layout, C, O, groups, k):
    """MX activations and weights (codes + power-of-two scales per 32 channels... 16 where a group is narrower), the
    activation's scales multiplied in by the gather warps."""
    from golden_util import golden_table
    g = torch.Generator().manual_seed(17)
    N, H, W = 2, 11, 13
    bs = min(32, C // groups)
    x = torch.randn(N, C, H, W, generator=g).bfloat16()
    w = (torch.randn(O, C // groups, k, k, generator=g) * 0.05).bfloat16()
    q = golden_table("int8")
    w_hwio = layout == "nhwc" and groups == 1
    if layout == "nhwc":
        x = x.permute(0, 2, 3, 1).contiguous()
    if w_hwio:
        w = w.permute(2, 3, 1, 0).contiguous()
    xs, xq = vo.quantize_mx(x, q, (3,) if layout == "nhwc" else (1,), bs, 127.0, True)
    ws, wq = vo.quantize_mx(w, q, (2,) if w_hwio else (1,), bs, 127.0, True)
    p = k // 2
    want = vo.conv2d_mx(xq.float(), wq.float(), None, 1, p, 1, groups, input_scale=xs.float(), weight_scale=ws.float(),
                        block_size=bs, layout=layout)
    got = torch.ops.quantized_ops.conv2d_mx(xq.cuda(), wq.cuda(), None, (1, 1), (p, p), (1, 1), groups, input_scale=xs.cuda(),
                                            weight_scale=ws.cuda(), block_size=bs, layout=layout)
    rel = (got.float().cpu().double() - want.double()).norm() / want.double().norm()
    assert rel <= 1e-2, rel


def test_grouped_convolution_with_narrow_groups_uses_the_vendor_kernel():
    """Depthwise and other groups narrower than 8 channels are not taken by the tensor-core kernels."""
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 16, 9, 9, generator=g).bfloat16()
    w = (torch.randn(16, 1, 3, 3, generator=g) * 0.1).bfloat16()
    want = vo.conv2d_mx(x.float(), w.float(), None, 1, 1, 1, 16)
    got = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), None, (1, 1), (1, 1), (1, 1), 16)
    rel = (got.float().cpu().double() - want.double()).norm() / want.double().norm()
    assert rel <= 1e-2, rel


@pytest.mark.parametrize("layout", ["nchw", "nhwc"])
@pytest.mark.parametrize("shape", SHAPES, ids=[str(i) for i in range(len(SHAPES))])
def test_fp32_convolution_runs_on_the_tensor_cores_as_tf32(shape, layout, monkeypatch):
    """fp32 operands: patch matrix + the tf32 contraction (the low 13 bits of every operand are ignored), fp32
    result; no vendor convolution."""
    x, w, b, st, pd, dl = _case(shape, 13)
    x, w, b = x.float() + 0.001 * torch.randn(x.shape), w.float() * 1.003, b.float()      # not bf16-representable
    if layout == "nhwc":
        x, w = x.permute(0, 2, 3, 1).contiguous(), w.permute(2, 3, 1, 0).contiguous()
    want = vo.conv2d_mx(x, w, b, st, pd, dl, 1, layout=layout)

    def boom(*a, **k):
        raise AssertionError("the vendor convolution was called")
    monkeypatch.setattr(torch.ops.aten, "conv2d", boom)
    got = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), st, pd, dl, 1, layout=layout)
    torch.cuda.synchronize()
    monkeypatch.undo()
    assert got.dtype == torch.float32 and tuple(got.shape) == tuple(want.shape)
    rel = (got.cpu().double() - want.double()).norm() / want.double().norm()
    assert rel <= 2e-3, rel
    from voyager_compiler_b200.gemm_native import gemm_status
    assert gemm_status("cuda") == 0


def test_vendor_switch_and_other_dtypes_agree(monkeypatch):
    x, w, b, st, pd, dl = _case(SHAPES[1], 3)
    a = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), st, pd, dl, 1)
    monkeypatch.setenv("VOYAGER_B200_CONV", "vendor")
    v = torch.ops.quantized_ops.conv2d_mx(x.cuda(), w.cuda(), b.cuda(), st, pd, dl, 1)
    rel = (a.float() - v.float()).norm() / v.float().norm()
    assert rel <= 1e-2, rel
    monkeypatch.delenv("VOYAGER_B200_CONV")
    f = torch.ops.quantized_ops.conv2d_mx(x.float().cuda(), w.float().cuda(), b.float().cuda(), st, pd, dl, 1)   # fp32: tf32 contraction
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
