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
  device, in upstream's order.  ``record_histogram`` (:369-371) is one counting kernel
  (:func:`exponent_histogram`); outlier filtering (:373-394, :428-430) is a split kernel before and a merge
  kernel after the quantizer (:func:`outlier_split`, :func:`outlier_merge`), the top-k threshold and its
  moving average being torch operations on the device.
* :func:`group_affine_fake_quantize` -- per-block min / max, scale, zero point, round, clamp and dequantize in one
  launch (``vq_group_affine_fake_quantize``; ``GroupWiseAffineFakeQuantFunction.forward``, :160-207).

CUDA tensors only; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from enum import Enum
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import _lib, ops, qtables, tables
from .qtables import table_handle

__all__ = ["QScheme", "amax", "fake_quantize", "mx_fake_quantize", "FakeQuantizeFunction", "MXFakeQuantizeFunction",
           "FusedAmaxObsFakeQuantize", "quantization_map", "exponent_histogram", "outlier_split", "outlier_merge", "group_affine_fake_quantize",
           "GroupWiseAffineFakeQuantFunction"]

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


def _require_same_device(x: torch.Tensor, what: str, **named: Optional[torch.Tensor]) -> None:
    """The kernels take raw addresses: a tensor on another device (a module built without
    ``device=`` and never moved keeps its buffers on the CPU) must be refused on the host, as torch
    refuses mixed devices, before an address of the wrong memory reaches a launch."""
    for name, t in named.items():
        if t is not None and t.device != x.device:
            raise RuntimeError(f"{what}: Expected all tensors to be on the same device, but {name} is on {t.device} "
                               f"and the input on {x.device} (move the module with .to(device))")


def _threshold_arg(x: torch.Tensor, threshold: torch.Tensor, what: str) -> torch.Tensor:
    if not isinstance(threshold, torch.Tensor) or threshold.numel() != 1 or threshold.dtype != torch.float32:
        raise ValueError(f"{what}: the threshold is one fp32 value in a tensor")
    _require_same_device(x, what, threshold=threshold)
    return threshold.contiguous()


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
    _require_same_device(x, "fake_quantize", scale=scale, qmap=qmap)
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


def exponent_histogram(x: torch.Tensor, histogram: torch.Tensor) -> torch.Tensor:
    """``histogram += torch.histc(floor(log2(|x|.float())), 254, min=-126, max=127)`` in place
    (fake_quantize.py:369-371): one counting pass over ``x`` (``vq_exp_histogram``) instead of abs, cast, log2,
    floor and histc passes.  ``histogram``: fp32 [254] on the device of ``x``.  Counts are exact; a bin that
    receives more than 2^24 elements in one call is added as the rounded fp32 count."""
    from .qtables import exp_tables
    _require_cuda(x, "exponent_histogram")
    if histogram.dtype != torch.float32 or histogram.numel() != 254 or not histogram.is_contiguous() or histogram.device != x.device:
        raise ValueError("exponent_histogram: the histogram is a contiguous fp32 tensor of 254 bins on the device of x")
    xc = x.contiguous()
    if xc.numel():
        with torch.cuda.device(x.device):
            ws = torch.empty(256, dtype=torch.int64, device=x.device)     # per call: safe with several streams
            et = exp_tables(torch.float32, 1.0, x.device)         # log2 is taken in fp32 whatever the dtype of x
            _lib.check(_lib.lib.vq_exp_histogram(xc.data_ptr(), _DT[x.dtype], xc.numel(), et.ptr(), histogram.data_ptr(),
                                                 ws.data_ptr(), ws.numel() * 8, torch.cuda.current_stream(x.device).cuda_stream),
                       "exponent_histogram")
    return histogram


def outlier_split(x: torch.Tensor, threshold: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(x.masked_fill(x.abs() >= threshold, 0.0), number of outliers)`` in one pass (fake_quantize.py:388-394).
    ``threshold``: one fp32 value on the device; it is rounded to the dtype of ``x`` for the comparison, as torch
    promotes a scalar.  The count is an int64 tensor on the device (no synchronisation)."""
    threshold = _threshold_arg(x, threshold, "outlier_split")
    _require_cuda(x, "outlier_split")
    xc = x.contiguous()
    out = torch.empty_like(xc)
    count = torch.empty(1, dtype=torch.int64, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.vq_outlier_split(xc.data_ptr(), _DT[x.dtype], xc.numel(), threshold.data_ptr(), out.data_ptr(),
                                             count.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream), "outlier_split")
    return out, count


def outlier_merge(x: torch.Tensor, quantized: torch.Tensor, threshold: torch.Tensor) -> torch.Tensor:
    """``torch.where(x.abs() >= threshold, x, quantized)`` in one pass (fake_quantize.py:428-430)."""
    threshold = _threshold_arg(x, threshold, "outlier_merge")
    _require_same_device(x, "outlier_merge", quantized=quantized)
    _require_cuda(x, "outlier_merge")
    xc, qc = x.contiguous(), quantized.contiguous()
    if qc.dtype != xc.dtype or qc.shape != xc.shape:
        raise ValueError("outlier_merge: the quantized tensor has the shape and dtype of x")
    out = torch.empty_like(xc)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.vq_outlier_merge(xc.data_ptr(), qc.data_ptr(), _DT[x.dtype], xc.numel(), threshold.data_ptr(),
                                             out.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream), "outlier_merge")
    return out


class _OutlierBypass(torch.autograd.Function):
    """Quantizer on the inliers, outliers passed through (fake_quantize.py:388-394, 396-430).  Upstream's graph
    (masked_fill, straight-through quantizer, where) has the identity as its gradient."""

    @staticmethod
    def forward(ctx, x, module):
        with torch.no_grad():
            thr = module._threshold_tensor(x.device)
            inliers, count = outlier_split(x, thr)
            module._note_outliers(count, x.numel())
            return outlier_merge(x, module._quantize(inliers), thr)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


def group_affine_fake_quantize(x: torch.Tensor, axes: Union[int, Sequence[int]], block_size: int, quant_min: float,
                               quant_max: float, scale_qmap: Optional[torch.Tensor] = None
                               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(scale, zero_point, (clamp(round(x / scale + zero_point), quant_min, quant_max) - zero_point) * scale)`` with
    ``scale = (max - min) / (quant_max - quant_min)`` (1 where not positive) and ``zero_point = -min / scale +
    quant_min`` per block of ``block_size`` elements along one axis (fake_quantize.py:160-207).  An axis other than
    the last one is moved there for the launch and back."""
    assert block_size > 0
    _require_cuda(x, "group_affine_fake_quantize")
    ax = ops._norm_axes(axes, x.ndim)
    if len(ax) != 1:
        raise NotImplementedError("group_affine_fake_quantize: blocks along exactly one axis")
    a = ax[0]
    xl = x.movedim(a, -1).contiguous()
    K = xl.shape[-1]
    rows = xl.numel() // K if K else 0
    nb = -(-K // block_size)
    out = torch.empty_like(xl)
    sf = torch.empty(xl.shape[:-1] + (nb,), dtype=x.dtype, device=x.device)
    zp = torch.empty_like(sf)
    if xl.numel():
        with torch.cuda.device(x.device):
            tab = table_handle(scale_qmap, x.device) if scale_qmap is not None else None
            _lib.check(_lib.lib.vq_group_affine_fake_quantize(
                xl.data_ptr(), _DT[x.dtype], rows, K, block_size, float(quant_min), float(quant_max),
                tab.lut16.data_ptr() if tab is not None else None, sf.data_ptr(), zp.data_ptr(), out.data_ptr(),
                torch.cuda.current_stream(x.device).cuda_stream), "group_affine_fake_quantize")
    if a != x.ndim - 1:
        out, sf, zp = out.movedim(-1, a).contiguous(), sf.movedim(-1, a).contiguous(), zp.movedim(-1, a).contiguous()
    return sf, zp, out


class GroupWiseAffineFakeQuantFunction(torch.autograd.Function):
    """fake_quantize.py:160-214; ``scale`` and ``zero_point`` are resized and overwritten with the block values."""

    @staticmethod
    def forward(ctx, input, fake_quant_enabled, scale, zero_point, axes, block_size, quant_min, quant_max, scale_qmap=None):
        if fake_quant_enabled[0] == 0:
            return input
        sf, zp, out = group_affine_fake_quantize(input, axes, block_size, quant_min, quant_max, scale_qmap)
        scale.resize_(sf.shape).copy_(sf)
        zero_point.resize_(zp.shape).copy_(zp)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        return (grad_output,) + (None,) * 8


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
    """fake_quantize.py:216-432: the symmetric per-tensor, per-channel, microscaling and group-wise affine schemes."""

    def __init__(self, dtype: str, qscheme=None, quant_min: Optional[float] = None, quant_max: Optional[float] = None,
                 amax_history_len: Optional[int] = None, ch_axis: Optional[int] = None, block_size: Optional[int] = None,
                 scale_dtype: Optional[str] = None, force_scale_power_of_two: bool = False,
                 record_histogram: bool = False, outlier_threshold: Optional[float] = None,
                 outlier_pct: Optional[float] = None, device: Optional[torch.device] = None, **kwargs) -> None:
        super().__init__()
        assert outlier_pct is None or outlier_threshold is None, "Only one of outlier_pct and outlier_threshold can be set."
        self.dtype = dtype
        self.qscheme = _scheme(qscheme)
        self.quant_min = quant_min
        self.quant_max = quant_max
        self.amax_history_len = amax_history_len
        self.ch_axis = ch_axis
        self.block_size = block_size
        self.scale_dtype = scale_dtype
        self.force_scale_power_of_two = force_scale_power_of_two
        self.record_histogram = record_histogram
        self.outlier_pct = outlier_pct
        kw = {"device": device, "dtype": torch.float}
        self.register_buffer("fake_quant_enabled", torch.tensor([1], dtype=torch.uint8, device=device))
        self.register_buffer("observer_enabled", torch.tensor([1], dtype=torch.uint8, device=device))
        self.register_buffer("qmap", quantization_map(dtype, device), persistent=False)
        self.register_buffer("scale_qmap", quantization_map(scale_dtype, device) if scale_dtype is not None else None,
                             persistent=False)
        self.register_buffer("amax_history", torch.tensor([], **kw))
        self.register_buffer("scale", torch.tensor([1.0], **kw))
        self.register_buffer("zero_point", torch.tensor([1.0], **kw))
        if record_histogram:
            self.register_buffer("histogram", torch.zeros(254, **kw), persistent=False)
        if outlier_pct is not None:
            self.outlier_ema_decay = kwargs.get("outlier_ema_decay", 0.9)
            self.register_buffer("outlier_threshold", torch.tensor([], **kw))
        else:
            self.outlier_threshold = outlier_threshold
        self._thr_dev = None                                       # device copy of a fixed threshold
        self._max_outlier_frac = 0.0
        self._pending_counts = []                                  # (device counter, numel) of forwards not folded in yet
        self.observer_enabled[0] = 1 if self.qscheme is not None else 0
        self.is_per_channel = self.qscheme == QScheme.PER_CHANNEL_SYMMETRIC
        # host mirrors of the two switches: reading the device buffers would synchronise every call
        self._fq_on, self._obs_on = True, self.qscheme is not None
        self._fq_host = torch.tensor([1], dtype=torch.uint8)       # what the autograd functions test
        self._amax_cur = None                                      # fp32 scratch of the reduction
        self._note_switch_versions()

    # The mirrors follow the buffers: a switch written in place (``m.observer_enabled[0] = 0``) or
    # loaded from a checkpoint bumps the buffer's version counter, which costs nothing to compare;
    # only then is the buffer read back (one synchronisation).
    def _note_switch_versions(self) -> None:
        self._switch_versions = (self.fake_quant_enabled._version, self.observer_enabled._version,
                                 id(self.fake_quant_enabled), id(self.observer_enabled))

    def _refresh_switches(self) -> None:
        now = (self.fake_quant_enabled._version, self.observer_enabled._version,
               id(self.fake_quant_enabled), id(self.observer_enabled))
        if now != self._switch_versions:
            self._fq_on = bool(int(self.fake_quant_enabled[0].item()))
            self._obs_on = bool(int(self.observer_enabled[0].item()))
            self._fq_host[0] = 1 if self._fq_on else 0
            self._switch_versions = now

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        """fake_quantize.py:434-463: ``scale`` and ``amax_history`` start empty / one-element and take
        their shape on the first forward, so a checkpoint saved after calibration is loaded by resizing
        them first (``zero_point`` and a learned ``outlier_threshold`` likewise); then the switches'
        host mirrors are refreshed from what was loaded."""
        for name in ("scale", "amax_history", "zero_point", "outlier_threshold"):
            key = prefix + name
            buf = getattr(self, name, None)
            if key in state_dict and isinstance(buf, torch.Tensor):
                buf.resize_(state_dict[key].shape)
            elif strict and name in ("scale", "amax_history"):
                missing_keys.append(key)
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        self._switch_versions = None
        self._refresh_switches()

    # -- switches (torch.ao.quantization.FakeQuantizeBase interface)
    def enable_fake_quant(self, enabled: bool = True) -> None:
        self.fake_quant_enabled[0] = 1 if enabled else 0
        self._fq_on = bool(enabled)
        self._fq_host[0] = 1 if enabled else 0
        self._note_switch_versions()

    def disable_fake_quant(self) -> None:
        self.enable_fake_quant(False)

    def enable_observer(self, enabled: bool = True) -> None:
        self.observer_enabled[0] = 1 if enabled else 0
        self._obs_on = bool(enabled)
        self._note_switch_versions()

    def disable_observer(self) -> None:
        self.enable_observer(False)

    def calculate_qparams(self):
        if self.qscheme == QScheme.GROUP_WISE_AFFINE:
            return self.scale, self.zero_point
        return self.scale

    def extra_repr(self) -> str:
        return (f"fake_quant_enabled={self._fq_on}, observer_enabled={self._obs_on}, dtype={self.dtype}, "
                f"amax_history_len={self.amax_history_len}, quant_max={self.quant_max}, qscheme={self.qscheme}, "
                f"ch_axis={self.ch_axis}, block_size={self.block_size}, "
                f"force_scale_power_of_two={self.force_scale_power_of_two}")

    @torch.no_grad()
    def _update_amax_scale(self, x: torch.Tensor) -> None:
        """fake_quantize.py:309-341: the scale is derived from the history BEFORE the current amax
        enters it; 0 / NaN / Inf maxima keep the previous scale.  One launch: the reduction, whose last
        CTA runs the whole state update (``VOYAGER_B200_OBSERVER=separate``: a memset and two launches)."""
        _require_cuda(x, "FusedAmaxObsFakeQuantize")
        _require_same_device(x, "FusedAmaxObsFakeQuantize", amax_history=self.amax_history, scale=self.scale)
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
        elif tuple(self.amax_history.shape) != (self.amax_history_len,) + shape or tuple(self.scale.shape) != shape:
            # the state was sized by an earlier input (or a checkpoint): the update kernel indexes it
            # with this input's channel count, so a different count must stop here, as the broadcast
            # of upstream's tensor expression does
            raise RuntimeError(f"FusedAmaxObsFakeQuantize: the observer state has shape {tuple(self.amax_history.shape)} "
                               f"(scale {tuple(self.scale.shape)}), this input needs {(self.amax_history_len,) + shape}")
        if not (self.amax_history.is_contiguous() and self.scale.is_contiguous()
                and self.amax_history.dtype == torch.float32 and self.scale.dtype == torch.float32):
            raise RuntimeError("FusedAmaxObsFakeQuantize: amax_history and scale must be contiguous fp32 buffers")
        if self._amax_cur is None or self._amax_cur.numel() != ch + 1 or self._amax_cur.device != x.device:
            # the step's maxima and a ticket: zero now, and left at zero by every fused step
            self._amax_cur = torch.zeros(ch + 1, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            stay = qtables.pow2_stay_table(x.device) if self.force_scale_power_of_two else None
            stay_ptr = stay.data_ptr() if stay is not None else None
            pow2 = 1 if self.force_scale_power_of_two else 0
            if os.environ.get("VOYAGER_B200_OBSERVER") == "separate":
                # the reduction (with its memset) and the state update as launches of their own
                _lib.check(_lib.lib.vq_amax(xc.data_ptr(), _DT[x.dtype], outer, ch, inner, self._amax_cur.data_ptr(), stream), "amax")
                _lib.check(_lib.lib.vq_observer_update(self._amax_cur.data_ptr(), self.amax_history.data_ptr(),
                                                       self.scale.data_ptr(), self.amax_history_len, ch, float(self.quant_max),
                                                       pow2, stay_ptr, stream), "observer update")
                self._amax_cur[:ch].zero_()
            else:
                # one launch: the reduction's last CTA updates the history and the scale and clears the scratch
                _lib.check(_lib.lib.vq_observer_step(xc.data_ptr(), _DT[x.dtype], outer, ch, inner, self._amax_cur.data_ptr(),
                                                     self.amax_history.data_ptr(), self.scale.data_ptr(), self.amax_history_len,
                                                     float(self.quant_max), pow2, stay_ptr, stream), "observer step")

    # -- outlier filtering (fake_quantize.py:373-394)
    @property
    def max_outlier_pct(self) -> float:
        """Largest fraction of elements bypassed in one forward so far.  The counts stay on the device until this
        is read (upstream synchronises on every forward, fake_quantize.py:392-394)."""
        for count, numel in self._pending_counts:
            self._max_outlier_frac = max(self._max_outlier_frac, int(count.item()) / max(numel, 1))
        self._pending_counts.clear()
        return self._max_outlier_frac

    def _threshold_tensor(self, device) -> torch.Tensor:
        if isinstance(self.outlier_threshold, torch.Tensor):
            return self.outlier_threshold
        if self._thr_dev is None or self._thr_dev.device != device:
            self._thr_dev = torch.tensor([float(self.outlier_threshold)], dtype=torch.float32, device=device)
        return self._thr_dev

    def _note_outliers(self, count: torch.Tensor, numel: int) -> None:
        self._pending_counts.append((count, numel))
        if len(self._pending_counts) >= 256:          # bounded: fold (and synchronise) now and then
            _ = self.max_outlier_pct

    @torch.no_grad()
    def _update_outlier_threshold(self, x: torch.Tensor) -> None:
        """The k-th largest magnitude (k = ceil(outlier_pct * numel)) and its moving average: an order statistic
        and two scalar operations, torch calls on the device in upstream's order."""
        flat = x.abs().flatten()
        k = max(1, math.ceil(self.outlier_pct * flat.numel()))
        threshold = torch.topk(flat, k, largest=True, sorted=False).values.min()
        if self.outlier_threshold.numel() == 0:
            self.outlier_threshold.resize_as_(threshold)
            self.outlier_threshold.copy_(threshold)
        else:
            self.outlier_threshold.mul_(self.outlier_ema_decay).add_(threshold * (1.0 - self.outlier_ema_decay))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._refresh_switches()
        _require_same_device(x, "FusedAmaxObsFakeQuantize", qmap=self.qmap, scale=self.scale,
                             fake_quant_enabled=self.fake_quant_enabled)
        if self.record_histogram:
            exponent_histogram(x.detach(), self.histogram)
        if self.outlier_pct is not None and self._obs_on:
            self._update_outlier_threshold(x.detach())
        if self.outlier_threshold is None:
            return self._quantize(x)
        return _OutlierBypass.apply(x, self)

    def _quantize(self, x: torch.Tensor) -> torch.Tensor:
        if self.qscheme == QScheme.MICROSCALING:
            if not self._fq_on:
                return x
            return MXFakeQuantizeFunction.apply(x, self._fq_host, self.scale, self.qmap, self.ch_axis,
                                                self.block_size, self.quant_max, self.force_scale_power_of_two,
                                                self.scale_qmap)
        if self.qscheme == QScheme.GROUP_WISE_AFFINE:
            if not self._fq_on:
                return x
            return GroupWiseAffineFakeQuantFunction.apply(x, self._fq_host, self.scale, self.zero_point, self.ch_axis,
                                                          self.block_size, self.quant_min, self.quant_max, self.scale_qmap)
        if self._obs_on:
            self._update_amax_scale(x.detach())
        if not self._fq_on:
            return x
        return FakeQuantizeFunction.apply(x, self._fq_host, self.qmap, self.scale)
