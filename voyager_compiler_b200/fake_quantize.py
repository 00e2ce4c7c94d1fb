"""Observer + fake-quantize forward on the GPU: the calibration / quantization-aware-training
module of upstream, src/voyager_compiler/quantization/fake_quantize.py.

* :func:`amax` -- ``torch.amax(torch.abs(x))`` per tensor or per channel in one pass
  (``vq_amax``; upstream: an abs pass with a full-size temporary, then a reduce pass, :320-325).
* :func:`fake_quantize` -- ``vmap(x / scale, qmap) * scale`` in one pass (``vq_fake_quantize``;
  ``FakeQuantizeFunction.forward``, :104-115).
* :func:`mx_fake_quantize` -- block scale, quantize and dequantize in one pass (``vq_quantize_mx``
  with its dequantized output; ``MXFakeQuantizeFunction.forward``, :128-153).
* :class:`FusedAmaxObsFakeQuantize` -- the module with the same constructor arguments, buffers
  (``qmap``, ``scale_qmap``, ``amax_history``, ``scale``, ``fake_quant_enabled``,
  ``observer_enabled``) and forward semantics (:216-432); the backward is the straight-through
  estimator.  The amax history is a handful of numbers and is updated with torch operations on the
  device, in upstream's order.  Outlier filtering, the exponent histogram and the group-wise
  affine scheme are not provided and raise ``NotImplementedError``.

CUDA tensors only; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
import math
from enum import Enum
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib, ops, tables
from .qtables import table_handle

__all__ = ["QScheme", "amax", "fake_quantize", "mx_fake_quantize", "FakeQuantizeFunction", "MXFakeQuantizeFunction",
           "FusedAmaxObsFakeQuantize", "quantization_map"]

_DT = {torch.float32: _lib.VQ_F32, torch.bfloat16: _lib.VQ_BF16}


class QScheme(Enum):
    """src/voyager_compiler/quantization/qspec.py:23-27."""
    PER_TENSOR_SYMMETRIC = "per_tensor_symmetric"
    PER_CHANNEL_SYMMETRIC = "per_channel_symmetric"
    MICROSCALING = "microscaling"
    GROUP_WISE_AFFINE = "group_wise_affine"


def _scheme(q) -> Optional[QScheme]:
    if q is None or isinstance(q, QScheme):
        return q
    return QScheme(getattr(q, "value", q))        # upstream's enum member or its string


def quantization_map(dtype: Optional[str], device=None) -> torch.Tensor:
    """The 65 536-entry bf16 value table of an upstream dtype string (``get_quantization_map``,
    fake_quantize.py:30-98; for codebook formats ``values[indices]``, :273-278)."""
    t = torch.from_numpy(tables.build_table(dtype).view(np.int16).copy()).view(torch.bfloat16)
    return t.to(device) if device is not None else t


def _require_cuda(x: torch.Tensor, what: str) -> None:
    if x.device.type != "cuda":
        raise RuntimeError(f"{what}: CUDA tensors only; there is no CPU path")
    if x.dtype not in _DT:
        raise NotImplementedError(f"{what}: dtype {x.dtype} is not supported")


def amax(x: torch.Tensor, ch_axis: Optional[int] = None) -> torch.Tensor:
    """``torch.amax(torch.abs(x))`` (0-d) or, with ``ch_axis``, the maximum over every other axis
    with ``keepdim=True``; in ``x.dtype``."""
    _require_cuda(x, "amax")
    xc = x.contiguous()
    if ch_axis is None:
        outer, ch, inner, shape = 1, 1, xc.numel(), ()
    else:
        a = ch_axis % x.ndim
        outer, ch, inner = math.prod(x.shape[:a]), x.shape[a], math.prod(x.shape[a + 1:])
        shape = tuple(ch if i == a else 1 for i in range(x.ndim))
    out = torch.empty(max(ch, 1), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.vq_amax(xc.data_ptr(), _DT[x.dtype], outer, max(ch, 1), inner, out.data_ptr(),
                                    torch.cuda.current_stream(x.device).cuda_stream), "amax")
    return out[:ch].to(x.dtype).reshape(shape)


def fake_quantize(x: torch.Tensor, scale: torch.Tensor, qmap: torch.Tensor) -> torch.Tensor:
    """``vmap(x / scale, qmap) * scale`` with ``scale`` cast to ``x.dtype`` and broadcast against
    ``x`` (a scalar or a keepdim per-channel tensor)."""
    _require_cuda(x, "fake_quantize")
    xc = x.contiguous()
    s = scale.to(device=x.device, dtype=x.dtype).contiguous()
    out = torch.empty_like(xc)
    if xc.numel():
        lay = ops._layout("fake_quantize", xc.shape, s, None)
        with torch.cuda.device(x.device):
            tab = table_handle(qmap, x.device)
            _lib.check(_lib.lib.vq_fake_quantize(xc.data_ptr(), _DT[x.dtype], xc.numel(), s.data_ptr(), C.byref(lay),
                                                 tab.ptr(), out.data_ptr(),
                                                 torch.cuda.current_stream(x.device).cuda_stream), "fake_quantize")
    return out


def mx_fake_quantize(x: torch.Tensor, qmap: torch.Tensor, axes: Union[int, Sequence[int]], block_size: int,
                     quant_max: float, force_scale_power_of_two: bool = False,
                     scale_qmap: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(scale, quantize_mx codes * expand(scale))``: one launch for one block axis."""
    assert block_size > 0
    _require_cuda(x, "mx_fake_quantize")
    xc = x.contiguous()
    ax = ops._norm_axes(axes, xc.ndim)
    if len(ax) > 1 or xc.numel() == 0:
        sf, q = ops.quantize_mx(xc, qmap, ax, block_size, quant_max, force_scale_power_of_two, scale_qmap)
        return sf, ops.dequantize(q, sf, None, ax, block_size)
    out = torch.empty_like(xc)
    extras = _lib.VqMxExtras()
    extras.dequant = out.data_ptr()
    rule = ops.RULE_POW2 if force_scale_power_of_two else ops.RULE_AMAX_OVER_QMAX
    tab = table_handle(qmap, xc.device)
    sf, _ = ops._mx_call("mx_fake_quantize", xc, ax[0], block_size, quant_max, rule, scale_qmap, tab, False, extras)
    return sf, out


class FakeQuantizeFunction(torch.autograd.Function):
    """fake_quantize.py:101-120."""

    @staticmethod
    def forward(ctx, input, fake_quant_enabled, qmap, scale):
        if fake_quant_enabled[0] == 0:
            return input
        return fake_quantize(input, scale, qmap)

    @staticmethod
    def backward(ctx, grad_output):
        return (grad_output,) + (None,) * 3


class MXFakeQuantizeFunction(torch.autograd.Function):
    """fake_quantize.py:123-159; ``scale`` is resized and overwritten with the block scales."""

    @staticmethod
    def forward(ctx, input, fake_quant_enabled, scale, qmap, axes, block_size, quant_max,
                force_scale_power_of_two=False, scale_qmap=None):
        if fake_quant_enabled[0] == 0:
            return input
        sf, out = mx_fake_quantize(input, qmap, axes, block_size, quant_max, force_scale_power_of_two, scale_qmap)
        scale.resize_(sf.shape).copy_(sf)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        return (grad_output,) + (None,) * 8


class FusedAmaxObsFakeQuantize(torch.nn.Module):
    """fake_quantize.py:216-432 for the symmetric per-tensor, per-channel and microscaling schemes."""

    def __init__(self, dtype: str, qscheme=None, quant_min: Optional[float] = None, quant_max: Optional[float] = None,
                 amax_history_len: Optional[int] = None, ch_axis: Optional[int] = None, block_size: Optional[int] = None,
                 scale_dtype: Optional[str] = None, force_scale_power_of_two: bool = False,
                 record_histogram: bool = False, outlier_threshold: Optional[float] = None,
                 outlier_pct: Optional[float] = None, device: Optional[torch.device] = None, **kwargs) -> None:
        super().__init__()
        if record_histogram or outlier_threshold is not None or outlier_pct is not None:
            raise NotImplementedError("FusedAmaxObsFakeQuantize: histogram recording and outlier filtering are not provided")
        self.dtype = dtype
        self.qscheme = _scheme(qscheme)
        if self.qscheme == QScheme.GROUP_WISE_AFFINE:
            raise NotImplementedError("FusedAmaxObsFakeQuantize: the group-wise affine scheme is not provided")
        self.quant_min = quant_min
        self.quant_max = quant_max
        self.amax_history_len = amax_history_len
        self.ch_axis = ch_axis
        self.block_size = block_size
        self.scale_dtype = scale_dtype
        self.force_scale_power_of_two = force_scale_power_of_two
        kw = {"device": device, "dtype": torch.float}
        self.register_buffer("fake_quant_enabled", torch.tensor([1], dtype=torch.uint8, device=device))
        self.register_buffer("observer_enabled", torch.tensor([1], dtype=torch.uint8, device=device))
        self.register_buffer("qmap", quantization_map(dtype, device), persistent=False)
        self.register_buffer("scale_qmap", quantization_map(scale_dtype, device) if scale_dtype is not None else None,
                             persistent=False)
        self.register_buffer("amax_history", torch.tensor([], **kw))
        self.register_buffer("scale", torch.tensor([1.0], **kw))
        self.register_buffer("zero_point", torch.tensor([1.0], **kw))
        self.observer_enabled[0] = 1 if self.qscheme is not None else 0
        self.is_per_channel = self.qscheme == QScheme.PER_CHANNEL_SYMMETRIC
        # host mirrors of the two switches: reading the device buffers would synchronise every call
        self._fq_on, self._obs_on = True, self.qscheme is not None
        self._fq_host = torch.tensor([1], dtype=torch.uint8)       # what the autograd functions test
        self._amax_cur = None                                      # fp32 scratch of the reduction

    # -- switches (torch.ao.quantization.FakeQuantizeBase interface)
    def enable_fake_quant(self, enabled: bool = True) -> None:
        self.fake_quant_enabled[0] = 1 if enabled else 0
        self._fq_on = bool(enabled)
        self._fq_host[0] = 1 if enabled else 0

    def disable_fake_quant(self) -> None:
        self.enable_fake_quant(False)

    def enable_observer(self, enabled: bool = True) -> None:
        self.observer_enabled[0] = 1 if enabled else 0
        self._obs_on = bool(enabled)

    def disable_observer(self) -> None:
        self.enable_observer(False)

    def calculate_qparams(self):
        return self.scale

    def extra_repr(self) -> str:
        return (f"fake_quant_enabled={self._fq_on}, observer_enabled={self._obs_on}, dtype={self.dtype}, "
                f"amax_history_len={self.amax_history_len}, quant_max={self.quant_max}, qscheme={self.qscheme}, "
                f"ch_axis={self.ch_axis}, block_size={self.block_size}, "
                f"force_scale_power_of_two={self.force_scale_power_of_two}")

    @torch.no_grad()
    def _update_amax_scale(self, x: torch.Tensor) -> None:
        """fake_quantize.py:309-341: the scale is derived from the history BEFORE the current amax
        enters it; 0 / NaN / Inf maxima keep the previous scale.  Two launches: the reduction and
        one kernel for the whole state update."""
        _require_cuda(x, "FusedAmaxObsFakeQuantize")
        xc = x.contiguous()
        if self.is_per_channel:
            a = self.ch_axis % x.ndim
            outer, ch, inner = math.prod(x.shape[:a]), x.shape[a], math.prod(x.shape[a + 1:])
            shape = tuple(ch if i == a else 1 for i in range(x.ndim))
        else:
            outer, ch, inner, shape = 1, 1, xc.numel(), ()
        if self.amax_history.numel() == 0:
            self.amax_history.resize_((self.amax_history_len,) + shape).fill_(0.0)
            self.scale.resize_(shape).fill_(1.0)
        if self._amax_cur is None or self._amax_cur.numel() != ch or self._amax_cur.device != x.device:
            self._amax_cur = torch.empty(ch, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            _lib.check(_lib.lib.vq_amax(xc.data_ptr(), _DT[x.dtype], outer, ch, inner, self._amax_cur.data_ptr(), stream), "amax")
            _lib.check(_lib.lib.vq_observer_update(self._amax_cur.data_ptr(), self.amax_history.data_ptr(),
                                                   self.scale.data_ptr(), self.amax_history_len, ch, float(self.quant_max),
                                                   1 if self.force_scale_power_of_two else 0, stream), "observer update")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.qscheme == QScheme.MICROSCALING:
            if not self._fq_on:
                return x
            return MXFakeQuantizeFunction.apply(x, self._fq_host, self.scale, self.qmap, self.ch_axis,
                                                self.block_size, self.quant_max, self.force_scale_power_of_two,
                                                self.scale_qmap)
        if self._obs_on:
            self._update_amax_scale(x.detach())
        if not self._fq_on:
            return x
        return FakeQuantizeFunction.apply(x, self._fq_host, self.qmap, self.scale)
