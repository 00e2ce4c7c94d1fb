"""GPTQ weight compensation against the deployed microscaling grid, on the GPU
(src/voyager_compiler/quantization/gptq.py: ``compensate_weight`` :184-270, ``block_scale`` :79-137,
``salience_order`` :140-181, ``hessian_inverse_chol`` :30-70).

Upstream walks the input channels one column at a time with a handful of tensor operations per column.
Inside one block of ``block_size`` columns every output row is independent, so ``vq_gptq_block`` gives each
row to a thread and walks the block's columns in registers (scale, optional shrink search, quantize, error,
update of the later columns); what is left per block is one launch and the update of the columns to the
right of it (``addmm_`` with ``alpha=-1``).  A block is reproduced bit for bit; across blocks the result
follows upstream up to the summation order of that fp32 product and of the Cholesky routines, both of
which differ between the CPU and the GPU libraries.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .qtables import table_handle

EPS = 1e-12                                      # quantization/lcq.py:34


DAMPING_STEPS = (1.0, 10.0, 100.0, 1000.0, 10000.0)      # multiples of the requested damping that are tried in turn


def hessian_inverse_chol(hessian: torch.Tensor, tokens: int, damping: float) -> torch.Tensor:
    """Upper Cholesky factor ``U`` of ``inv(H / tokens + lambda * I)`` with ``lambda = damping * mean(diag)``
    (what gptq.py:30-70 computes): the factorisation is attempted with ``lambda`` times 1, 10, ..., 10^4
    until it succeeds; ``LinAlgError`` when even the strongest damping leaves the matrix indefinite.  The
    factorisations are torch's (cuSOLVER) on the device of ``hessian``."""
    mean_h = hessian / max(tokens, 1)
    unit = damping * mean_h.diagonal().mean().clamp_min(EPS)
    eye_diag = torch.ones_like(mean_h.diagonal())
    for step in DAMPING_STEPS:
        trial = mean_h + torch.diag_embed(eye_diag * (step * unit))
        lower, failed = torch.linalg.cholesky_ex(trial)
        if not bool(failed.any()):
            return torch.linalg.cholesky(torch.cholesky_inverse(lower), upper=True)
    raise torch.linalg.LinAlgError("Hessian not positive-definite")


def salience_order(hessian: torch.Tensor, columns: int, within_block: bool, block_size: int) -> Optional[torch.Tensor]:
    """Permutation that puts the blocks with the largest mean ``diag(H)`` first and keeps every block whole;
    with ``within_block`` the columns of a block are ordered by their own ``diag(H)`` too.  ``None`` when the
    width is not a whole number of blocks (gptq.py:140-181)."""
    if columns % block_size:
        return None
    nb = columns // block_size
    dev = hessian.device
    diag = hessian.diagonal().reshape(nb, block_size)
    blocks = torch.argsort(diag.mean(dim=1), descending=True)
    if within_block:
        inner = torch.argsort(diag, dim=1, descending=True)
    else:
        inner = torch.arange(block_size, device=dev).expand(nb, block_size)
    return (torch.arange(nb, device=dev).unsqueeze(1) * block_size + inner)[blocks].reshape(-1)


def walk(weight: torch.Tensor, hinv_chol: torch.Tensor, salience: Optional[torch.Tensor], qmap: torch.Tensor,
         scale_qmap: Optional[torch.Tensor], quant_max: float, block_size: int, shrink: bool = False,
         return_scales: bool = False):
    """The column walk of gptq.py:238-262 on a weight whose columns are already in walking order:
    returns the reconstruction on the grid (fp32 ``[out, in]``), and with ``return_scales`` the scale every
    row used in every block (``[out, ceil(in / block_size)]``)."""
    if weight.device.type != "cuda":
        raise RuntimeError("gptq.walk: CUDA tensors only; there is no CPU path")
    if weight.ndim != 2:
        raise ValueError("gptq.walk: the weight must be [out, in]")
    if block_size > 64:
        raise NotImplementedError("gptq.walk: blocks of up to 64 input channels")
    if shrink and scale_qmap is None:
        raise ValueError("gptq.walk: the shrink search re-encodes the scale and needs its table")
    dev = weight.device
    O, K = weight.shape
    work = weight.float().contiguous().clone()
    hinv = hinv_chol.float().contiguous()
    out = torch.zeros_like(work)
    nblk = (K + block_size - 1) // block_size
    scales = torch.empty((nblk, O), dtype=torch.float32, device=dev) if return_scales else None
    deltas = torch.empty((O, block_size), dtype=torch.float32, device=dev)
    sal = salience.float().contiguous() if salience is not None else None
    tab = table_handle(qmap, dev)
    stab = table_handle(scale_qmap, dev, allow_runs=False) if scale_qmap is not None else None
    stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        for b, start in enumerate(range(0, K, block_size)):
            end = min(start + block_size, K)
            bw = end - start
            d = deltas if bw == block_size else deltas.view(-1)[: O * bw].view(O, bw)
            _lib.check(_lib.lib.vq_gptq_block(
                work.data_ptr(), K, O, start, bw, hinv.data_ptr(), K, sal.data_ptr() if sal is not None else None,
                1 if shrink else 0, float(quant_max), tab.ptr(), stab.ptr() if stab is not None else None,
                out.data_ptr(), K, d.data_ptr(), scales[b].data_ptr() if scales is not None else None, stream), "gptq.walk")
            if end < K:
                work[:, end:].addmm_(d, hinv[start:end, end:], alpha=-1.0)
    return (out, scales.t().contiguous()) if return_scales else out


def compensate_weight(weight, hessian, tokens, fake_quant, damping, act_order=True, within_block=True, shrink=False):
    """The GPTQ-compensated reconstruction of ``weight`` ``[out, in]`` on the grid ``fake_quant`` deploys
    (its ``qmap``, ``scale_qmap``, ``quant_max``, ``block_size`` and ``ch_axis``); same arguments and result as
    upstream's ``compensate_weight`` (gptq.py:184-270).  Steps: walking order of the input channels (most salient
    blocks first), the damped inverse factor in that order, the kernel's column walk, the columns put back."""
    axes = fake_quant.ch_axis
    block_axis = axes[0] if isinstance(axes, (tuple, list)) else axes
    if block_axis % weight.dim() != weight.dim() - 1:
        raise ValueError(f"weight blocks run along axis {block_axis}, but the compensation walks the input channels of a "
                         f"{tuple(weight.shape)} weight")
    order = salience_order(hessian, weight.shape[1], within_block, fake_quant.block_size) if act_order else None
    w_walk, h_walk = (weight, hessian) if order is None else (weight.index_select(1, order), hessian.index_select(0, order).index_select(1, order))
    hinv = hessian_inverse_chol(h_walk, tokens, damping)
    out = walk(w_walk, hinv, h_walk.diagonal().clone(), fake_quant.qmap, fake_quant.scale_qmap, fake_quant.quant_max,
               fake_quant.block_size, shrink)
    if order is None:
        return out
    back = torch.empty_like(order)
    back[order] = torch.arange(order.numel(), device=order.device)
    return out.index_select(1, back)
