"""Statistics pass of upstream's learned-codebook fit on the GPU
(src/voyager_compiler/quantization/lcq.py: ``Histogram`` :43-113, ``unit_scale`` :136-150, ``_accumulate``
:601-626).  The fit itself (dynamic program over the three cumulative sums) reads a few kilobytes and stays
on the host, as upstream; what touches every element of every tensor is the accumulation, and that is one
kernel here (``vq_lcq_accumulate``).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import _lib

HISTOGRAM_BINS = 4001                            # lcq.py:40
_DT = {torch.float32: _lib.VQ_F32, torch.bfloat16: _lib.VQ_BF16}


_edge_cache: dict = {}


def _device_edges(quant_min, quant_max, bins, device):
    key = (float(quant_min), float(quant_max), int(bins), str(device))
    e = _edge_cache.get(key)
    if e is None:
        e = torch.linspace(quant_min - 0.5, quant_max + 0.5, bins + 1, dtype=torch.float32).to(device)
        if len(_edge_cache) >= 16:
            _edge_cache.pop(next(iter(_edge_cache)))
        _edge_cache[key] = e
    return e


def accumulate_moments(weight, total, square, quant_min, quant_max, x, block, unit_max, weights):
    """One launch of ``vq_lcq_accumulate`` into the three fp64 ``[bins]`` CUDA tensors of a histogram over
    ``quant_min - 0.5 .. quant_max + 0.5``; ``block == 0``: ``x`` holds normalised values already."""
    if x.device.type != "cuda":
        raise RuntimeError("lcq: CUDA tensors only; there is no CPU path")
    if x.dtype not in _DT:
        x = x.float()
    x = x.contiguous()
    bins = weight.numel()
    edges = _device_edges(quant_min, quant_max, bins, x.device)
    if weights is None:
        wp, nw = None, 0
    else:
        weights = weights.to(device=x.device, dtype=torch.float32).contiguous().reshape(-1)
        wp, nw = weights.data_ptr(), weights.numel()
        if x.numel() % nw:
            raise ValueError("lcq: the weights do not tile the values")
    for m in (weight, total, square):
        if m.dtype != torch.float64 or m.device != x.device or not m.is_contiguous() or m.numel() != bins:
            raise ValueError("lcq: the moments must be contiguous fp64 tensors of equal length on the tensor's device")
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib.vq_lcq_accumulate(
            x.data_ptr(), _DT[x.dtype], x.numel(), block, float(unit_max), wp, nw, edges.data_ptr(), bins,
            weight.data_ptr(), total.data_ptr(), square.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream), "lcq")


def codebook_qmap(entries, device=None) -> torch.Tensor:
    """The bf16 ``[65536]`` lookup table of a codebook on ``device`` (lcq.py:270-291): one launch of
    ``vq_codebook_qmap`` instead of a ``[65536, n]`` distance matrix; ``entries`` is a sequence of numbers or a tensor
    (one on the device is used where it lies, so a fit that ends on the GPU does not come back to the host)."""
    if isinstance(entries, torch.Tensor):
        dev = torch.device(device) if device is not None else entries.device
        cb = entries.detach().to(device=dev, dtype=torch.float32).contiguous().reshape(-1)
    else:
        dev = torch.device(device if device is not None else "cuda")
        cb = torch.tensor(list(entries), dtype=torch.float32, device=dev)
    if dev.type != "cuda":
        raise RuntimeError("lcq.codebook_qmap: CUDA devices only; there is no CPU path")
    table = torch.empty(1 << 16, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.vq_codebook_qmap(cb.data_ptr(), cb.numel(), table.data_ptr(),
                                             torch.cuda.current_stream(dev).cuda_stream), "codebook_qmap")
    return table


class Histogram:
    """Weighted moments of a tensor's normalised values per bin: total weight, weighted sum, weighted sum of
    squares (fp64), between ``quant_min - 0.5`` and ``quant_max + 0.5``; same fields and methods as upstream's
    dataclass, plus :meth:`accumulate`, which also does the normalisation."""

    def __init__(self, quant_min: float, quant_max: float, bins: int = HISTOGRAM_BINS):
        self.quant_min, self.quant_max, self.bins = quant_min, quant_max, bins
        self.weight = self.total = self.square = None

    def edges(self):
        return np.linspace(self.quant_min - 0.5, self.quant_max + 0.5, self.bins + 1)

    def _launch(self, x, block, quant_max, weights):
        if x.device.type != "cuda":
            raise RuntimeError("lcq.Histogram: CUDA tensors only; there is no CPU path")
        if self.weight is None:
            self.weight, self.total, self.square = (torch.zeros(self.bins, dtype=torch.float64, device=x.device) for _ in range(3))
        accumulate_moments(self.weight, self.total, self.square, self.quant_min, self.quant_max, x, block, quant_max, weights)

    def add(self, values: torch.Tensor, weights: Optional[torch.Tensor]):
        """Accumulate normalised ``values`` (flat); ``weights`` is a scalar, or tiles the values (lcq.py:75-105)."""
        self._launch(values, 0, 1.0, weights)

    def accumulate(self, tensor: torch.Tensor, block_size: int, quant_max: float, energy: Optional[torch.Tensor] = None):
        """``unit_scale`` + ``add`` for a tensor whose blocks run along its last axis (lcq.py:601-626): every
        element is divided by its block's ``max(amax, EPS) / quant_max`` and weighted by the energy of its channel."""
        if tensor.numel() < block_size:
            return
        if tensor.shape[-1] % block_size:
            raise ValueError("lcq.Histogram: the last axis must be a whole number of blocks")
        self._launch(tensor.detach(), block_size, quant_max, energy)

    def cumulative(self):
        """The three running sums, with a leading zero, as numpy arrays (lcq.py:107-112)."""
        return tuple(np.concatenate([[0], m.cpu().numpy().cumsum()]) for m in (self.weight, self.total, self.square))
