"""Per-row (per-output-channel) codebook quantization.

Upstream codebooks are per tensor: ``codebook_qmap`` (src/voyager_compiler/quantization/lcq.py:270-291)
turns the sorted levels into a 65 536-entry table and ``vmap`` applies it.  Here every row of a
weight matrix carries its own sorted codebook and one kernel launch searches all rows, with the
same rule per row: clamp to the codebook range, fp32 absolute difference, first minimum wins.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

__all__ = ["row_codebook_quantize", "row_quantile_levels"]

_DT = {torch.float32: _lib.VQ_F32, torch.bfloat16: _lib.VQ_BF16}


def row_quantile_levels(x: torch.Tensor, n_levels: int = 16) -> torch.Tensor:
    """Codebook of every row: its quantiles at (2k+1) / (2 n_levels), k = 0..n_levels-1, linear
    interpolation, fp32 ``[rows, n_levels]``, ascending; bit-identical to
    ``torch.quantile(x.float(), q, dim=-1).T`` evaluated on the CPU.  Rows of up to 8192 elements
    are sorted in shared memory by ``vq_row_quantile``; longer rows go through ``torch.quantile`` on
    the device."""
    if x.device.type != "cuda":
        raise RuntimeError("row_quantile_levels: CUDA tensors only; there is no CPU path")
    if x.ndim != 2:
        raise ValueError("x must be [rows, K]")
    rows, K = x.shape
    if x.dtype in _DT and 1 <= K <= 8192 and 1 <= n_levels <= 256:
        xc = x.contiguous()
        out = torch.empty(rows, n_levels, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib.vq_row_quantile(xc.data_ptr(), _DT[x.dtype], rows, K, n_levels, out.data_ptr(),
                                                torch.cuda.current_stream(x.device).cuda_stream), "row_quantile_levels")
        return out
    q = (2 * torch.arange(n_levels, device=x.device, dtype=torch.float32) + 1) / (2 * n_levels)
    return torch.quantile(x.float(), q, dim=-1).t().contiguous()


def row_codebook_quantize(x: torch.Tensor, levels: torch.Tensor, reference_rule: bool = True,
                          want_indices: bool = True, want_values: bool = True,
                          check_sorted: bool = False) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``(indices uint8, values x.dtype)`` of shape ``x.shape``; ``x`` is ``[rows, K]`` and
    ``levels`` ``[rows, n]`` fp32 with every row ascending.

    ``reference_rule=True``: the element is rounded to bf16 before the search and the returned
    level is rounded to bf16 -- bit-identical to building upstream's table from that row's levels
    and calling ``vmap``.  ``False``: fp32 search, fp32 level."""
    if x.device.type != "cuda":
        raise RuntimeError("row_codebook_quantize: CUDA tensors only; there is no CPU path")
    if x.dtype not in _DT:
        raise NotImplementedError(f"row_codebook_quantize: dtype {x.dtype}")
    if x.ndim != 2 or levels.ndim != 2 or levels.shape[0] != x.shape[0]:
        raise ValueError("x must be [rows, K] and levels [rows, n_levels]")
    if not 1 <= levels.shape[1] <= 256:
        raise ValueError("n_levels must be in [1, 256]")
    if not (want_indices or want_values):
        raise ValueError("nothing to compute")
    if levels.device != x.device:
        raise ValueError("x and levels must live on one device")
    if check_sorted and levels.shape[1] > 1 and not bool((levels[:, 1:] >= levels[:, :-1]).all()):
        raise ValueError("every row of levels must be ascending")
    xc = x.contiguous()
    lv = levels.to(torch.float32).contiguous()
    idx = torch.empty(x.shape, dtype=torch.uint8, device=x.device) if want_indices else None
    val = torch.empty_like(xc) if want_values else None
    work = torch.empty(lv.shape, dtype=torch.float32, device=x.device)      # per-row decision thresholds
    with torch.cuda.device(x.device):
        rc = _lib.lib.vq_row_codebook(
            xc.data_ptr(), _DT[x.dtype], x.shape[0], x.shape[1], lv.data_ptr(), lv.shape[1], 1 if reference_rule else 0,
            idx.data_ptr() if idx is not None else None, val.data_ptr() if val is not None else None,
            work.data_ptr(), work.numel() * 4, torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc, "row_codebook_quantize")
    return idx, val
