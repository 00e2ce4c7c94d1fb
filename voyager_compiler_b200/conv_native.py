"""``conv2d_mx`` on this library's tensor cores (src/voyager_compiler/ops/quantized.py:239-283).

The convolution is the TN contraction ``patches[M, K] @ weight[O, K]^T``: ``M = N * Ho * Wo`` output
positions, ``K = kh * kw * C`` ordered (kh, kw, c).  Two forms:

* implicit (``vq_conv2d_bf16``): the GEMM kernel's own warps gather the patches from the channels-last
  activation while they stage the operand tiles, so no patch matrix exists in memory; the activation's block
  scales are multiplied in on the way; grouped convolutions run as one launch over (group, tile).  Needs the
  channels per group to be a multiple of 8.
* explicit (``vq_conv_patches`` + ``vq_gemm_bf16_tn``): the patch matrix is written once; used for the channel
  counts the implicit form does not take (a 3-channel stem), ``groups == 1`` only.

An NCHW activation is first made channels-last by ``vq_conv_patches`` (its 1x1 patch matrix, a tiled
transposition with the scaling fused).  The decoded weight matrix is kept for as long as the weight tensor
lives, since a weight is static.  bf16; other dtypes stay on the vendor convolution (``supported`` says which).
"""
from __future__ import annotations

import os
import weakref
from typing import Optional

import torch

from . import _lib
from .gemm_native import _status_tensor

_weight_cache: dict = {}


def weight_layout(layout: str, groups: int) -> str:
    """``"nhwc"`` weights are HWIO, except that a grouped convolution keeps its weight OIHW (ops/layout.py:152-175)."""
    return "nchw" if (layout == "nchw" or groups != 1) else "nhwc"


def implicit_ok(channels: int, groups: int) -> bool:
    """The implicit-GEMM kernel takes the convolution (``VOYAGER_B200_CONV=patches`` forces the explicit form)."""
    return os.environ.get("VOYAGER_B200_CONV", "native") != "patches" and groups >= 1 and channels % groups == 0 \
        and (channels // groups) % 8 == 0


def supported(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], groups: int, layout: str = "nchw") -> bool:
    if os.environ.get("VOYAGER_B200_CONV", "native") == "vendor":
        return False
    if x.dtype != w.dtype or x.ndim != 4 or w.ndim != 4 or groups < 1:
        return False
    if x.dtype == torch.float32:
        # fp32: patch matrix + the tf32 contraction (VOYAGER_B200_FP32=vendor keeps the vendor kernel), one group
        if os.environ.get("VOYAGER_B200_FP32", "tensor") == "vendor" or groups != 1:
            return False
    elif x.dtype != torch.bfloat16:
        return False
    channels = x.shape[1] if layout == "nchw" else x.shape[3]
    outputs = w.shape[0] if weight_layout(layout, groups) == "nchw" else w.shape[3]
    if groups != 1 and not (implicit_ok(channels, groups) and outputs % groups == 0):
        return False
    return bias is None or (bias.dtype == x.dtype and bias.ndim == 1)


def _weight_matrix_one_pass(weight, weight_scale, weight_code, block_size, layout) -> Optional[torch.Tensor]:
    """The [O, K] weight by one launch of the patch kernel (a transposition with the block scales multiplied
    in), for plain or MX-scaled weights without a codebook; None when that form does not apply."""
    if weight_code is not None or not weight.is_contiguous() or weight.data_ptr() % 16 or weight.dtype != torch.bfloat16:
        return None
    dev = weight.device
    if layout == "nchw":
        O, I, kh, kw = weight.shape
        K = kh * kw * I
        if I % 8 or I < 8:                                        # rows of [O * kh * kw, I] must need no padding
            return None
        sc_args = (None, 0, 0, 0, 0, 0)
        if weight_scale is not None:
            if not fusable_scale(weight, weight_scale, block_size, "nchw"):
                return None
            ws = weight_scale.contiguous()
            nb = ws.shape[1]
            sc_args = (ws.data_ptr(), block_size, nb * kh * kw, kw, 1, kh * kw)     # n, h, w, channel block
        wm = torch.empty((O, K), dtype=torch.bfloat16, device=dev)
        # the weight as O "images" of kh x kw pixels (handed over as one row) with I channels: its 1x1 patch matrix
        args = (weight.data_ptr(), _lib.VQ_BF16, O, 1, kh * kw, I, I * kh * kw, kh * kw, 1, kh * kw, 1, 1, 1, 1, 0, 0, 1, 1)
        ldk = I
        if sc_args[0] is not None:
            sc_args = (sc_args[0], sc_args[1], sc_args[2], kh * kw, 1, sc_args[5])
    else:
        kh, kw, I, O = weight.shape
        K = kh * kw * I
        if K < 8:
            return None
        sc_args = (None, 0, 0, 0, 0, 0)
        if weight_scale is not None:
            want = [kh, kw, -(-I // block_size), O] if block_size else None
            if weight_scale.dtype != weight.dtype or list(weight_scale.shape) != want or I % block_size:
                return None
            ws = weight_scale.contiguous()
            sc_args = (ws.data_ptr(), block_size, 0, 0, 1, O)
        Kp = (K + 7) // 8 * 8
        wm = torch.empty((O, Kp), dtype=torch.bfloat16, device=dev)
        # the weight as one image row of O pixels with K strided channels: its 1x1 patch matrix is the transpose
        args = (weight.data_ptr(), _lib.VQ_BF16, 1, 1, O, K, K * O, K * O, 1, O, 1, 1, 1, 1, 0, 0, 1, 1)
        ldk = Kp
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.vq_conv_patches(*args, *sc_args, wm.data_ptr(), ldk, torch.cuda.current_stream(dev).cuda_stream),
                   "conv2d_mx")
    return wm


def _weight_matrix(weight, weight_scale, weight_code, block_size, layout) -> torch.Tensor:
    """Decoded weight as ``[O, ceil8(kh * kw * I)]`` with columns ordered (kh, kw, i), cached per weight."""
    from . import ops
    parts = [t for t in (weight, weight_scale, weight_code) if t is not None]
    key = (tuple((t.data_ptr(), t._version, tuple(t.shape), t.dtype) for t in parts), block_size, layout)
    hit = _weight_cache.get(key)
    if hit is not None and all(r() is t for r, t in zip(hit[0], parts)):
        return hit[1]
    wm = _weight_matrix_one_pass(weight, weight_scale, weight_code, block_size, layout)
    if wm is None:
        wd = ops._decode_operand("conv2d_mx", weight, weight_code, weight_scale, block_size)
        wm = wd.permute(0, 2, 3, 1) if layout == "nchw" else wd.permute(3, 0, 1, 2)       # OIHW / HWIO -> O, kh, kw, I
        O = wm.shape[0]
        wm = wm.reshape(O, -1)
        K = wm.shape[1]
        Kp = (K + 7) // 8 * 8
        if Kp != K:
            wm = torch.nn.functional.pad(wm, (0, Kp - K))
        wm = wm.contiguous()
    if len(_weight_cache) >= 64:
        _weight_cache.pop(next(iter(_weight_cache)))
    _weight_cache[key] = ([weakref.ref(t) for t in parts], wm)
    return wm


def _merged_groups(groups: int, cg: int) -> int:
    """How many neighbouring groups the implicit kernel treats as one: a k-step is 64 channels of one tap, so groups
    narrower than that are merged (their weights become block-diagonal) until a step is full."""
    sg = 1
    while cg * sg * 2 <= 64 and groups % (sg * 2) == 0:
        sg *= 2
    return sg


def _weight_matrix_taps(weight, weight_scale, weight_code, block_size, layout, groups):
    """The decoded weight for the implicit kernel and the group count to run it with.

    ``[O, kh * kw * Cp]``: every tap's channels padded with zeros to ``Cp``, a multiple of 64.  Groups narrower than
    64 channels are merged ``sg`` at a time: the kernel then sees ``groups / sg`` groups of ``sg * Cg`` channels whose
    weight is block-diagonal (output ``o`` of original group ``g`` has its ``Cg`` weights at channel offset
    ``(g % sg) * Cg`` and zeros elsewhere), so that a 64-channel step of the contraction is not mostly padding.
    Cached per weight."""
    parts = [t for t in (weight, weight_scale, weight_code) if t is not None]
    key = (tuple((t.data_ptr(), t._version, tuple(t.shape), t.dtype) for t in parts), block_size, layout, "taps", groups)
    hit = _weight_cache.get(key)
    if hit is not None and all(r() is t for r, t in zip(hit[0], parts)):
        return hit[1]
    layout = weight_layout(layout, groups)
    if layout == "nchw":
        O, Cg, kh, kw = weight.shape
    else:
        kh, kw, Cg, O = weight.shape
    wm = _weight_matrix(weight, weight_scale, weight_code, block_size, layout)[:, :kh * kw * Cg].reshape(O, kh * kw, Cg)
    sg = _merged_groups(groups, Cg) if groups > 1 else 1
    if sg > 1:
        wide = torch.zeros((O, kh * kw, sg, Cg), dtype=wm.dtype, device=wm.device)
        rows = torch.arange(O, device=wm.device)
        wide[rows, :, (rows // (O // groups)) % sg, :] = wm
        wm = wide.reshape(O, kh * kw, sg * Cg)
    cg = sg * Cg
    cols = _lib.lib.vq_conv2d_weight_columns(cg, kh, kw)
    cp = cols // (kh * kw)
    if cp != cg:
        wm = torch.nn.functional.pad(wm, (0, cp - cg))
    wm = wm.reshape(O, cols).contiguous()
    if len(_weight_cache) >= 64:
        _weight_cache.pop(next(iter(_weight_cache)))
    _weight_cache[key] = ([weakref.ref(t) for t in parts], (wm, groups // sg))
    return wm, groups // sg


def fusable_scale(x: torch.Tensor, scale: Optional[torch.Tensor], block_size, layout) -> bool:
    """True when ``scale`` holds one value per block of channels at every pixel of ``x`` (the layout
    ``quantize_mx`` along the channel axis produces), which the patch kernels multiply in on the way."""
    if scale is None or block_size is None or scale.dtype != x.dtype or scale.ndim != 4 or x.ndim != 4:
        return False
    ch = 1 if layout == "nchw" else 3
    want = list(x.shape)
    want[ch] = -(-x.shape[ch] // block_size)
    return list(scale.shape) == want


def _conv2d_implicit(x, weight, bias, stride, padding, dilation, weight_scale, weight_code, block_size, layout, x_scale,
                     groups) -> Optional[torch.Tensor]:
    """The implicit-GEMM form; ``None`` when the activation's strides or the block size rule it out."""
    if layout == "nchw":
        N, C, H, W = x.shape
        sn, sc, sh, sw = x.stride()
    else:
        N, H, W, C = x.shape
        sn, sh, sw, sc = x.stride()
    if weight_layout(layout, groups) == "nchw":
        O, kh, kw = weight.shape[0], weight.shape[2], weight.shape[3]
    else:
        kh, kw, O = weight.shape[0], weight.shape[1], weight.shape[3]
    dev = x.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    sc_args = (None, 0, 0, 0, 0)
    if x_scale is not None:
        if block_size < 8 or block_size & (block_size - 1):
            return None
        x_scale = x_scale.contiguous()
        if layout == "nchw":
            ssn, ssc, ssh, ssw = x_scale.stride()
        else:
            ssn, ssh, ssw, ssc = x_scale.stride()
    with torch.cuda.device(dev):
        if sc != 1:
            # channels strided (NCHW): one tiled pass makes the activation channels-last, scaled on the way
            xt = torch.empty((N, H, W, C), dtype=torch.bfloat16, device=dev)
            pre = (None, 0, 0, 0, 0, 0) if x_scale is None else (x_scale.data_ptr(), block_size, ssn, ssh, ssw, ssc)
            flat = sh == W * sw and (pre[0] is None or pre[3] == W * pre[4])
            h_, w_, sh_ = (1, H * W, H * W * sw) if flat else (H, W, sh)
            ssh_ = (H * W * pre[4] if flat else pre[3])
            _lib.check(_lib.lib.vq_conv_patches(x.data_ptr(), _lib.VQ_BF16, N, h_, w_, C, sn, sh_, sw, sc, 1, 1, 1, 1, 0, 0, 1, 1,
                                                pre[0], pre[1], pre[2], ssh_, pre[4], pre[5], xt.data_ptr(), C, stream), "conv2d_mx")
            x = xt
            sn, sh, sw, sc = H * W * C, W * C, C, 1
        elif x_scale is not None:
            if ssc != 1:
                return None
            sc_args = (x_scale.data_ptr(), block_size, ssn, ssh, ssw)
        if sn % 8 or sh % 8 or sw % 8 or x.data_ptr() % 16:
            return None
        wm, run_groups = _weight_matrix_taps(weight, weight_scale, weight_code, block_size, layout, groups)
        Ho = (H + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
        Wo = (W + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
        if Ho <= 0 or Wo <= 0:
            raise RuntimeError("conv2d_mx: the kernel window is larger than the padded input")
        out = torch.empty((N * Ho * Wo, O), dtype=torch.bfloat16, device=dev)
        bias_c = bias.contiguous() if bias is not None else None
        _lib.check(_lib.lib.vq_conv2d_bf16(
            x.data_ptr(), N, H, W, C, sn, sh, sw, *sc_args, wm.data_ptr(), O, kh, kw, stride[0], stride[1], padding[0], padding[1],
            dilation[0], dilation[1], run_groups, bias_c.data_ptr() if bias_c is not None else None, out.data_ptr(),
            _status_tensor(dev).data_ptr(), stream), "conv2d_mx")
    y = out.view(N, Ho, Wo, O)
    return y.permute(0, 3, 1, 2) if layout == "nchw" else y


def conv2d_mx(x, weight, bias, stride, padding, dilation, weight_scale, weight_code, block_size, layout,
              x_scale: Optional[torch.Tensor] = None, groups: int = 1) -> torch.Tensor:
    """``x``: the activation (bf16, NCHW or NHWC as ``layout`` says, any strides), decoded, or still to be
    multiplied by ``x_scale`` (see :func:`fusable_scale`).  Returns the result in the layout's logical shape;
    for ``"nchw"`` its memory is channels-last (the kernels write [N*Ho*Wo, O])."""
    channels = x.shape[1] if layout == "nchw" else x.shape[3]
    if x.dtype == torch.bfloat16 and implicit_ok(channels, groups):
        y = _conv2d_implicit(x, weight, bias, stride, padding, dilation, weight_scale, weight_code, block_size, layout, x_scale,
                             groups)
        if y is not None:
            return y
    if groups != 1:
        raise NotImplementedError("conv2d_mx: grouped convolutions need channels per group in multiples of 8 and "
                                  "16-byte aligned pixels")
    wm = _weight_matrix(weight, weight_scale, weight_code, block_size, layout)
    dt = _lib.VQ_BF16 if x.dtype == torch.bfloat16 else _lib.VQ_F32
    sc_args = (None, 0, 0, 0, 0, 0)
    if layout == "nchw":
        N, C, H, W = x.shape
        sn, sc, sh, sw = x.stride()
        kh, kw = weight.shape[2], weight.shape[3]
        if x_scale is not None:
            x_scale = x_scale.contiguous()
            ssn, ssc, ssh, ssw = x_scale.stride()
            sc_args = (x_scale.data_ptr(), block_size, ssn, ssh, ssw, ssc)
    else:
        N, H, W, C = x.shape
        sn, sh, sw, sc = x.stride()
        kh, kw = weight.shape[0], weight.shape[1]
        if x_scale is not None:
            x_scale = x_scale.contiguous()
            ssn, ssh, ssw, ssc = x_scale.stride()
            sc_args = (x_scale.data_ptr(), block_size, ssn, ssh, ssw, ssc)
    O, Kp = wm.shape
    K = kh * kw * C
    if (K + 7) // 8 * 8 != Kp:
        raise ValueError("conv2d_mx: the channel counts of input and weight differ")
    Ho = (H + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    Wo = (W + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    if Ho <= 0 or Wo <= 0:
        raise RuntimeError("conv2d_mx: the kernel window is larger than the padded input")
    M = N * Ho * Wo
    dev = x.device
    out = torch.empty((M, O), dtype=x.dtype, device=dev)
    if M and O:
        stream = torch.cuda.current_stream(dev).cuda_stream
        with torch.cuda.device(dev):
            if sc != 1 and C >= 8:
                # channels strided (NCHW): one tiled pass makes the activation channels-last (its 1x1 patch
                # matrix), so that the patch rows below are copied in 16-byte pieces
                # (scaled on the way when the scale was not applied yet); image rows that follow one another in
                # memory are handed over as one long row
                xt = torch.empty((N, H, W, C), dtype=x.dtype, device=dev)
                flat = sh == W * sw and (sc_args[0] is None or sc_args[3] == W * sc_args[4])
                h_, w_, sh_ = (1, H * W, H * W * sw) if flat else (H, W, sh)
                ssh_ = (H * W * sc_args[4] if flat else sc_args[3])
                _lib.check(_lib.lib.vq_conv_patches(x.data_ptr(), dt, N, h_, w_, C, sn, sh_, sw, sc, 1, 1, 1, 1, 0, 0, 1, 1,
                                                    sc_args[0], sc_args[1], sc_args[2], ssh_, sc_args[4], sc_args[5],
                                                    xt.data_ptr(), C, stream), "conv2d_mx")
                x = xt
                sn, sh, sw, sc = x.stride()
                sc_args = (None, 0, 0, 0, 0, 0)
            pointwise = (kh == 1 and kw == 1 and tuple(stride) == (1, 1) and tuple(padding) == (0, 0) and K == Kp
                         and sc == 1 and sw == C and sh == W * C and sn == H * W * C and x.data_ptr() % 16 == 0
                         and sc_args[0] is None)
            if pointwise:
                a = x
            else:
                a = torch.empty((M, Kp), dtype=x.dtype, device=dev)
                _lib.check(_lib.lib.vq_conv_patches(
                    x.data_ptr(), dt, N, H, W, C, sn, sh, sw, sc, kh, kw, stride[0], stride[1], padding[0], padding[1],
                    dilation[0], dilation[1], *sc_args, a.data_ptr(), Kp, stream), "conv2d_mx")
            bias_c = bias.contiguous() if bias is not None else None
            bias_p = bias_c.data_ptr() if bias_c is not None else None
            if x.dtype == torch.bfloat16:
                rc = _lib.lib.vq_gemm_bf16_tn(a.data_ptr(), wm.data_ptr(), bias_p, out.data_ptr(), M, O, Kp,
                                              _status_tensor(dev).data_ptr(), stream)
            else:                                                     # fp32: the tensor cores read the operands as tf32
                rc = _lib.lib.vq_gemm_f32_tn_batched(a.data_ptr(), wm.data_ptr(), bias_p, out.data_ptr(), 1, M, O, Kp, 0, 1,
                                                     _status_tensor(dev).data_ptr(), stream)
            _lib.check(rc, "conv2d_mx")
    y = out.view(N, Ho, Wo, O)
    return y.permute(0, 3, 1, 2) if layout == "nchw" else y
