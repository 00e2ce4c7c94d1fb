"""CUDA implementations of the ``quantized_ops`` operators, registered on the dispatcher.

Op names, schemas, argument order, defaults and error behaviour are those of
src/voyager_compiler/ops/quantized.py (``vmap`` :98, ``quantize`` :124-172, ``dequantize``
:175-227, ``calculate_mx_qparam`` :435-499, ``quantize_mx`` :502-529, ``linear_mx`` :286-348,
``matmul_mx`` :363-421).  If the upstream package has already defined the ``quantized_ops``
library, only ``CUDA`` kernels are added to it, so its ``convert_pt2e`` / codegen passes keep
their op identities while CUDA tensors run here; otherwise the schemas are defined verbatim
together with shape-only fake kernels.  CPU tensors are never handled by this package.

Every function below validates arguments, picks the layout description and calls the C ABI
(``include/voyager_b200.h``) on the current CUDA stream of the input's device.
"""
from __future__ import annotations

import ctypes as C
import logging
import math
from typing import List, Optional, Sequence, Tuple, Union

import torch

from . import _lib
from .qtables import exp_tables, table_handle

logger = logging.getLogger(__name__)

__all__ = ["vmap", "quantize", "dequantize", "calculate_mx_qparam", "quantize_mx", "linear_mx", "matmul_mx", "conv2d_mx",
           "filter_outlier", "quantize_mx_outlier", "slice_csr_tensor", "spmm_csr", "register", "SCHEMAS"]

_DT = {torch.float32: _lib.VQ_F32, torch.bfloat16: _lib.VQ_BF16}

SCHEMAS = {
    "vmap": "vmap(Tensor self, Tensor other) -> Tensor",
    "quantize": "quantize(Tensor input, Tensor scale, Tensor? zero_point=None, "
                "SymInt[]? axes=None, int? block_size=None, Tensor? qmap=None, "
                "Tensor? output_code=None) -> Tensor",
    "dequantize": "dequantize(Tensor input, Tensor scale, Tensor? zero_point=None, "
                  "SymInt[]? axes=None, int? block_size=None, Tensor? input_qmap=None, "
                  "Tensor? output_qmap=None) -> Tensor",
    "calculate_mx_qparam": "calculate_mx_qparam(Tensor self, SymInt[] axes, int block_size, "
                           "float quant_max, bool force_scale_power_of_two=False, "
                           "Tensor scale_qmap=None) -> Tensor",
    "quantize_mx": "quantize_mx(Tensor self, Tensor qmap, SymInt[] axes, int block_size, "
                   "float quant_max, bool force_scale_power_of_two=False, "
                   "Tensor scale_qmap=None, Tensor output_code=None) -> (Tensor, Tensor)",
    "conv2d_mx": "conv2d_mx(Tensor input, Tensor weight, Tensor? bias=None, "
                 "SymInt[2] stride=1, SymInt[2] padding=0, SymInt[2] dilation=1, "
                 "SymInt groups=1, *, Tensor? input_scale=None, Tensor? weight_scale=None, "
                 "int? block_size=None, Tensor? input_code=None, "
                 'Tensor? weight_code=None, str layout="nchw") -> Tensor',
    "linear_mx": "linear_mx(Tensor input, Tensor weight, Tensor? bias=None, *, "
                 "Tensor? input_scale=None, Tensor? weight_scale=None, "
                 "int? block_size=None, Tensor? input_code=None, Tensor? weight_code=None, "
                 "Tensor? A_data=None, Tensor? A_indices=None, Tensor? A_indptr=None, "
                 'str weight_layout="kc") -> Tensor',
    "matmul_mx": "matmul_mx(Tensor self, Tensor other, *, Tensor? input_scale=None, "
                 "Tensor? weight_scale=None, int? block_size=None, Tensor? input_code=None, "
                 "Tensor? weight_code=None, Tensor? A_data=None, Tensor? A_indices=None, "
                 'Tensor? A_indptr=None, str weight_layout="ck") -> Tensor',
    "filter_outlier": "filter_outlier(Tensor input, float threshold, float max_pct=0.01) "
                      "-> (Tensor, Tensor, Tensor, Tensor)",
    "quantize_mx_outlier": "quantize_mx_outlier(Tensor self, Tensor qmap, SymInt[] axes, "
                           "int block_size, float quant_max, bool force_scale_power_of_two=False, "
                           "Tensor scale_qmap=None, Tensor output_code=None, float? threshold=None, "
                           "float max_pct=0.01, SymInt indptr_offset=0) "
                           "-> (Tensor, Tensor, Tensor, Tensor, Tensor)",
    "slice_csr_tensor": "slice_csr_tensor(Tensor data, Tensor indices, Tensor indptr, int dim=0, "
                        "SymInt? start=None, SymInt? end=None, float size_factor=1.0) "
                        "-> (Tensor, Tensor, Tensor)",
    "spmm_csr": "spmm_csr(Tensor data, Tensor indices, Tensor indptr, Tensor B, "
                "Tensor? B_scale=None, Tensor? B_code=None, int? block_size=None, "
                'str weight_layout="kc") -> Tensor',
}


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(f"{what}: voyager_compiler_b200 only runs CUDA tensors (got {t.device}); there is no CPU path")


def _meta(t: torch.Tensor, dtype=None) -> torch.Tensor:
    return torch.empty(t.shape, dtype=dtype or t.dtype, device="meta")


def _compute_dtype(name: str, x: torch.Tensor, *others: Optional[torch.Tensor]) -> torch.dtype:
    """dtype torch's type promotion gives ``x (op) others``; only widening casts are accepted."""
    d = x.dtype
    for o in others:
        if o is not None:
            d = torch.result_type(_meta(x, d), _meta(o))
    if d not in _DT:
        raise NotImplementedError(f"{name}: dtype {d} is not supported on CUDA (float32 and bfloat16 are)")
    for t in (x, *others):
        if t is None or t.dtype == d:
            continue
        if not (d == torch.float32 and t.dtype in (torch.bfloat16, torch.float16)):
            raise NotImplementedError(
                f"{name}: mixing {t.dtype} with {d} would need a narrowing cast the reference does not perform")
    return d


def _layout(name: str, shape: Sequence[int], scale: torch.Tensor, block_size: Optional[int]):
    """``vq_scale_layout`` for ``scale`` against a tensor of ``shape``: the index rule of ``expand``
    (ops/quantized.py:82-95: left-pad, repeat mismatching dims ``block_size`` times, crop) when
    ``block_size`` is given, plain broadcasting otherwise."""
    lay = _lib.VqScaleLayout()
    shape = list(shape)
    if scale.ndim > len(shape):
        raise NotImplementedError(f"{name}: scale has more dimensions than the input")
    sshape = [1] * (len(shape) - scale.ndim) + list(scale.shape)
    dims = []  # (size, scale size, divisor) of every dim with more than one element
    for d, (n, sz) in enumerate(zip(shape, sshape)):
        if sz == n:
            div = 1
        else:
            grown = sz if block_size is None else min(sz * block_size, n)
            if grown == n:
                div = block_size
            elif grown == 1:
                div = max(n, 1)              # broadcast: every coordinate reads index 0
            else:
                raise RuntimeError(f"{name}: scale of shape {tuple(scale.shape)} with block_size {block_size} "
                                   f"does not cover input of shape {tuple(shape)} (dim {d})")
        if n != 1:
            dims.append((n, sz, div))
    if scale.numel() == 1 or not dims:
        lay.mode = _lib.SCALE_SCALAR
        return lay
    lead = 0
    while lead < len(dims) and dims[lead][1] == dims[lead][0]:
        lead += 1
    rows = math.prod(d[0] for d in dims[:lead])
    rest = dims[lead:]
    if not rest:                                             # one scale per element
        lay.mode, lay.rows, lay.K, lay.block = _lib.SCALE_ROWBLOCK, rows, 1, 1
        return lay
    if all(d[1] == 1 for d in rest):                         # one scale per row of the [rows, K] view
        K = math.prod(d[0] for d in rest)
        lay.mode, lay.rows, lay.K, lay.block = _lib.SCALE_ROWBLOCK, rows, K, K
        return lay
    if len(rest) == 1 and rest[0][1] == -(-rest[0][0] // min(rest[0][2], rest[0][0])):
        # blocks along the contiguous axis, scale rows exactly ceil(K / block) long
        lay.mode, lay.rows, lay.K, lay.block = _lib.SCALE_ROWBLOCK, rows, rest[0][0], rest[0][2]
        return lay
    if len(dims) > 6:
        raise NotImplementedError(f"{name}: more than 6 non-trivial dimensions with a general scale layout")
    lay.mode, lay.ndim = _lib.SCALE_STRIDED, len(dims)
    acc = 1
    for d in range(len(dims) - 1, -1, -1):
        n, sz, div = dims[d]
        lay.size[d], lay.div[d] = n, div
        lay.stride[d] = acc if sz > 1 else 0
        acc *= sz
    return lay


def _prep(t: Optional[torch.Tensor], dtype: torch.dtype) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def vmap(input: torch.Tensor, qmap: torch.Tensor) -> torch.Tensor:
    """``out = qmap[bits(bf16(input))]`` in ``input.dtype`` (ops/quantized.py:101-121)."""
    _require_cuda(input, "vmap")
    src_dtype = input.dtype
    if src_dtype == torch.float16:
        input = input.float()            # exact widening; rounding to bf16 happens once, in the kernel
    if input.dtype not in _DT:
        raise NotImplementedError(f"vmap: dtype {src_dtype} is not supported on CUDA")
    x = input.contiguous()
    out = torch.empty_like(x)
    if x.numel():
        with torch.cuda.device(x.device):
            tab = table_handle(qmap, x.device)
            _lib.check(_lib.lib.vq_lut_map(x.data_ptr(), _DT[x.dtype], x.numel(), tab.ptr(), out.data_ptr(),
                                           _stream(x.device)), "vmap")
    return out if out.dtype == src_dtype else out.to(src_dtype)


def _same_shape_or_expand(name, zp, scale):
    if zp is None or zp.shape == scale.shape:
        return zp
    try:
        return zp.expand_as(scale)
    except RuntimeError:
        raise NotImplementedError(f"{name}: zero_point of shape {tuple(zp.shape)} against scale {tuple(scale.shape)}")


def quantize(input: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
             axes: Optional[Sequence[int]] = None, block_size: Optional[int] = None,
             qmap: Optional[torch.Tensor] = None, output_code: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``vmap(input / scale [+ zero_point], qmap)`` (ops/quantized.py:131-172).  ``axes`` and
    ``output_code`` are accepted and ignored, as upstream does."""
    assert qmap is not None, "qmap must be provided for quantization"
    _require_cuda(input, "quantize")
    dt = _compute_dtype("quantize", input, scale, zero_point)
    x = _prep(input, dt)
    zero_point = _same_shape_or_expand("quantize", zero_point, scale)
    s, z = _prep(scale, dt), _prep(zero_point, dt)
    lay = _layout("quantize", x.shape, s, block_size)
    out = torch.empty_like(x)
    if x.numel():
        with torch.cuda.device(x.device):
            tab = table_handle(qmap, x.device)
            _lib.check(_lib.lib.vq_quantize(x.data_ptr(), _DT[dt], x.numel(), s.data_ptr(),
                                            z.data_ptr() if z is not None else None, C.byref(lay), tab.ptr(),
                                            out.data_ptr(), None, 0, _stream(x.device)), "quantize")
    return out


def dequantize(input: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
               axes: Optional[Sequence[int]] = None, block_size: Optional[int] = None,
               input_qmap: Optional[torch.Tensor] = None, output_qmap: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out_qmap((in_qmap(input) - zero_point) * scale)`` (ops/quantized.py:182-227)."""
    _require_cuda(input, "dequantize")
    dt = _compute_dtype("dequantize", input, scale, zero_point)
    if input_qmap is not None and dt != input.dtype:
        raise NotImplementedError("dequantize: input_qmap with a scale of a wider dtype than the input")
    x = _prep(input, dt)
    zero_point = _same_shape_or_expand("dequantize", zero_point, scale)
    s, z = _prep(scale, dt), _prep(zero_point, dt)
    lay = _layout("dequantize", x.shape, s, block_size)
    out = torch.empty_like(x)
    if x.numel():
        with torch.cuda.device(x.device):
            tin = table_handle(input_qmap, x.device).ptr() if input_qmap is not None else None
            tout = table_handle(output_qmap, x.device).ptr() if output_qmap is not None else None
            _lib.check(_lib.lib.vq_dequantize(x.data_ptr(), _DT[dt], x.numel(), s.data_ptr(),
                                              z.data_ptr() if z is not None else None, C.byref(lay), tin, tout,
                                              out.data_ptr(), _stream(x.device)), "dequantize")
    return out


def _norm_axes(axes, ndim: int) -> List[int]:
    axes = [axes] if isinstance(axes, int) else list(axes)
    return sorted(a + ndim if a < 0 else a for a in axes)


RULE_AMAX_OVER_QMAX, RULE_POW2, RULE_RAW_AMAX = 0, 1, 2


def _mx_call(fn_name, x, axis, block_size, quant_max, rule, scale_qmap, table, want_codes, extras=None):
    """One launch over ``x`` viewed as [outer, L, inner] with blocks along ``axis``."""
    shape = list(x.shape)
    L = shape[axis]
    outer, inner = math.prod(shape[:axis]), math.prod(shape[axis + 1:])
    eff = min(block_size, L) if L > 0 else block_size
    nblk = (L + eff - 1) // eff if L > 0 else 0
    sshape = shape[:axis] + [nblk] + shape[axis + 1:]
    scale = torch.empty(sshape, dtype=x.dtype, device=x.device)
    codes = torch.empty_like(x) if want_codes else None
    if x.numel() == 0:
        return scale, codes
    with torch.cuda.device(x.device):
        exp = exp_tables(x.dtype, quant_max, x.device).ptr() if rule == RULE_POW2 else None
        stab = table_handle(scale_qmap, x.device, allow_runs=False).ptr() if (scale_qmap is not None and rule == RULE_AMAX_OVER_QMAX) else None
        if table is None:
            rc = _lib.lib.vq_mx_scale(x.data_ptr(), _DT[x.dtype], outer, L, inner, block_size, float(quant_max), rule,
                                      exp, stab, scale.data_ptr(), _stream(x.device))
        else:
            rc = _lib.lib.vq_quantize_mx(x.data_ptr(), _DT[x.dtype], outer, L, inner, block_size, float(quant_max),
                                         rule, exp, stab, table.ptr(), scale.data_ptr(),
                                         codes.data_ptr() if codes is not None else None,
                                         C.byref(extras) if extras is not None else None, _stream(x.device))
        _lib.check(rc, fn_name)
    return scale, codes


def calculate_mx_qparam(input: torch.Tensor, axes: Union[int, Sequence[int]], block_size: int, quant_max: float,
                        force_scale_power_of_two: bool = False, scale_qmap: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-block scale (ops/quantized.py:442-499)."""
    assert block_size > 0
    _require_cuda(input, "calculate_mx_qparam")
    if input.dtype not in _DT:
        raise NotImplementedError(f"calculate_mx_qparam: dtype {input.dtype} is not supported on CUDA")
    x = input.contiguous()
    ax = _norm_axes(axes, x.ndim)
    rule = RULE_POW2 if force_scale_power_of_two else RULE_AMAX_OVER_QMAX
    # several block axes: reduce |x| maxima axis by axis, apply the scale rule on the last one
    for a in ax[:-1]:
        x, _ = _mx_call("calculate_mx_qparam", x, a, block_size, quant_max, RULE_RAW_AMAX, None, None, False)
    scale, _ = _mx_call("calculate_mx_qparam", x, ax[-1], block_size, quant_max, rule, scale_qmap, None, False)
    return scale


def quantize_mx(input: torch.Tensor, qmap: torch.Tensor, axes: Sequence[int], block_size: int, quant_max: float,
                force_scale_power_of_two: bool = False, scale_qmap: Optional[torch.Tensor] = None,
                output_code: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(scale, codes)`` in one pass over the input (ops/quantized.py:509-529)."""
    assert block_size > 0
    _require_cuda(input, "quantize_mx")
    if input.dtype not in _DT:
        raise NotImplementedError(f"quantize_mx: dtype {input.dtype} is not supported on CUDA")
    x = input.contiguous()
    ax = _norm_axes(axes, x.ndim)
    if len(ax) > 1:
        scale = calculate_mx_qparam(x, ax, block_size, quant_max, force_scale_power_of_two, scale_qmap)
        return scale, quantize(x, scale, None, ax, block_size, qmap)
    rule = RULE_POW2 if force_scale_power_of_two else RULE_AMAX_OVER_QMAX
    tab = table_handle(qmap, x.device)
    return _mx_call("quantize_mx", x, ax[0], block_size, quant_max, rule, scale_qmap, tab, True)


# ---------------------------------------------------------------------------------------------
# MX GEMMs
# ---------------------------------------------------------------------------------------------
def _decode_operand(name, t, code, scale, block_size):
    """``code[t.long()].to(t.dtype) * expand(scale)`` with this package's kernels."""
    if code is not None:
        n = code.numel()
        lut = torch.zeros(1 << 16, dtype=torch.bfloat16, device=t.device)
        idx = torch.arange(n, dtype=torch.float32, device=t.device).to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
        if t.dtype == torch.float32 and not torch.equal(code.to(torch.bfloat16).to(code.dtype), code):
            raise NotImplementedError(f"{name}: float32 operands need a codebook whose entries are exact in bfloat16")
        lut[idx.long()] = code.to(torch.bfloat16)
        t = vmap(t, lut)
    if scale is not None:
        t = dequantize(t, scale, None, None, block_size)
    return t


# ---------------------------------------------------------------------------------------------
# Outlier side path
# ---------------------------------------------------------------------------------------------
def _filter_outlier(input: torch.Tensor, threshold: float, max_pct: float, indptr_offset: int = 0):
    _require_cuda(input, "filter_outlier")
    if input.dtype not in _DT:
        raise NotImplementedError(f"filter_outlier: dtype {input.dtype} is not supported on CUDA")
    if input.ndim < 2:
        raise ValueError("filter_outlier: the input needs at least two dimensions")
    x = input.contiguous()
    batch_shape, (rows, cols) = tuple(x.shape[:-2]), x.shape[-2:]
    batch = math.prod(batch_shape)
    max_nnz = int(rows * cols * max_pct)
    dev = x.device
    data = torch.empty(batch_shape + (max_nnz,), dtype=x.dtype, device=dev)
    indices = torch.empty(batch_shape + (max_nnz,), dtype=torch.int32, device=dev)
    indptr = torch.empty(batch_shape + (rows + 1,), dtype=torch.int32, device=dev)
    inlier = torch.empty_like(x)
    if batch and rows * cols == 0:                      # empty matrices: empty CSRs
        data.zero_()
        indices.fill_(-1)
        indptr.fill_(int(indptr_offset))
    elif batch:
        with torch.cuda.device(dev):
            need = _lib.lib.vq_filter_outlier_workspace(batch, rows)
            ws = torch.empty(max(need, 4), dtype=torch.uint8, device=dev)
            _lib.check(_lib.lib.vq_filter_outlier(
                x.data_ptr(), _DT[x.dtype], batch, rows, cols, float(threshold), max_nnz, int(indptr_offset),
                data.data_ptr(), indices.data_ptr(), indptr.data_ptr(), inlier.data_ptr(), ws.data_ptr(), ws.numel(),
                _stream(dev)), "filter_outlier")
    return data, indices, indptr, inlier


def filter_outlier(input: torch.Tensor, threshold: float, max_pct: float = 0.01):
    """``(data, indices, indptr, inlier)``: elements with ``|x| > threshold`` leave the tensor as a
    padded CSR per trailing matrix (ops/quantized.py:565-621)."""
    return _filter_outlier(input, threshold, max_pct)


def quantize_mx_outlier(input: torch.Tensor, qmap: torch.Tensor, axes: Sequence[int], block_size: int, quant_max: float,
                        force_scale_power_of_two: bool = False, scale_qmap: Optional[torch.Tensor] = None,
                        output_code: Optional[torch.Tensor] = None, threshold: Optional[float] = None,
                        max_pct: float = 0.01, indptr_offset: int = 0):
    """``(data, indices, indptr, scale, inliers)``: the outlier split followed by ``quantize_mx`` of
    the inliers (ops/quantized.py:650-700)."""
    data, indices, indptr, inlier = _filter_outlier(input, threshold, max_pct, indptr_offset)
    scale, codes = quantize_mx(inlier, qmap, axes, block_size, quant_max, force_scale_power_of_two, scale_qmap)
    return data, indices, indptr, scale, codes


def slice_csr_tensor(data, indices, indptr, dim: int = 0, start=None, end=None, size_factor: float = 1.0):
    """Rows (``dim`` 0) or columns (``dim`` 1) ``[start, end)`` of a padded CSR (ops/quantized.py:745-788) as one
    to three kernel launches of ``vq_slice_csr``: nothing is read back to the host, so the call does not
    synchronise.  The outputs hold ``int(data.shape[0] * size_factor)`` entries padded with 0 / -1; entries beyond
    that capacity are dropped and the row pointers clamped, as upstream does (its warning about dropped entries
    would need the count on the host and is not issued)."""
    _require_cuda(data, "slice_csr_tensor")
    dim = dim + 2 if dim < 0 else dim
    if dim not in (0, 1):
        raise ValueError(f"Cannot slice sparse CSR matrix along dim {dim}")
    if data.dtype not in _DT:
        raise NotImplementedError(f"slice_csr_tensor: dtype {data.dtype} is not supported on CUDA")
    if data.ndim != 1 or indices.ndim != 1 or indptr.ndim != 1 or indices.dtype != torch.int32 or indptr.dtype != torch.int32:
        raise NotImplementedError("slice_csr_tensor: one padded CSR (1-D data / int32 indices / int32 indptr) per call")
    rows = indptr.numel() - 1
    start = 0 if start is None else int(start)
    end = (rows if dim == 0 else (1 << 31) - 1) if end is None else int(end)
    cap = int(data.shape[0] * size_factor)
    d, ix, ip = data.contiguous(), indices.contiguous(), indptr.contiguous()
    new_data = torch.empty(cap, dtype=data.dtype, device=data.device)
    new_indices = torch.empty(cap, dtype=torch.int32, device=data.device)
    new_indptr = torch.empty(end - start + 1 if dim == 0 else rows + 1, dtype=torch.int32, device=data.device)
    with torch.cuda.device(data.device):
        ws = torch.empty(max(_lib.lib.vq_slice_csr_workspace(rows), 4), dtype=torch.uint8, device=data.device) if dim == 1 else None
        _lib.check(_lib.lib.vq_slice_csr(d.data_ptr(), ix.data_ptr(), ip.data_ptr(), _DT[data.dtype], rows, d.numel(), dim, start, end,
                                         cap, new_data.data_ptr(), new_indices.data_ptr(), new_indptr.data_ptr(),
                                         ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                         _stream(data.device)), "slice_csr_tensor")
    return new_data, new_indices, new_indptr


_kn_cache: "dict" = {}


def _decoded_kn(B, B_scale, B_code, block_size, weight_layout):
    """The decoded dense operand of ``spmm_csr`` in [..., K, N] order.  A weight is static, so the
    last few results are kept, keyed by the identity and version counters of the tensors involved
    (weak references: an entry dies with its weight)."""
    import weakref
    parts = [t for t in (B, B_scale, B_code) if t is not None]
    key = (tuple((t.data_ptr(), t._version, tuple(t.shape), t.dtype) for t in parts), block_size, weight_layout)
    hit = _kn_cache.get(key)
    if hit is not None and all(r() is t for r, t in zip(hit[0], parts)):
        return hit[1]
    Bd = _decode_operand("spmm_csr", B, B_code, B_scale, block_size)
    Bt = (Bd.mT if weight_layout == "kc" else Bd).contiguous()
    if len(_kn_cache) >= 8:
        _kn_cache.pop(next(iter(_kn_cache)))
    _kn_cache[key] = ([weakref.ref(t) for t in parts], Bt)
    return Bt


def spmm_csr(data, indices, indptr, B, B_scale=None, B_code=None, block_size=None, weight_layout: str = "kc"):
    """Sparse (padded CSR) x dense with the dense operand decoded like a ``linear_mx`` weight
    (ops/quantized.py:786-862); fp32 accumulation, output in ``B``'s dtype."""
    return _spmm_csr(data, indices, indptr, B, B_scale, B_code, block_size, weight_layout, None)


def _spmm_csr(data, indices, indptr, B, B_scale, B_code, block_size, weight_layout, addend):
    """``spmm_csr``; with ``addend`` (the dense product, overwritten) the sum ``addend + spmm`` in one pass."""
    assert weight_layout in ("kc", "ck"), weight_layout
    _require_cuda(B, "spmm_csr")
    Bt = _decoded_kn(B, B_scale, B_code, block_size, weight_layout)      # [..., K, N]
    if Bt.dtype not in _DT:
        raise NotImplementedError(f"spmm_csr: dtype {Bt.dtype} is not supported on CUDA")
    if data.dtype != Bt.dtype:
        raise NotImplementedError("spmm_csr: the sparse values and the dense operand must share a dtype")
    Bd = Bt
    batch_shape = tuple(indptr.shape[:-1])
    batch = math.prod(batch_shape)
    rows = indptr.shape[-1] - 1
    K, N = Bt.shape[-2], Bt.shape[-1]
    if Bt.ndim > 2 and math.prod(Bt.shape[:-2]) != batch:
        raise ValueError("spmm_csr: batch dimensions of the sparse and the dense operand differ")
    if addend is not None and (addend.dtype != Bd.dtype or tuple(addend.shape) != batch_shape + (rows, N)
                               or not addend.is_contiguous()):
        return addend + _spmm_csr(data, indices, indptr, B, B_scale, B_code, block_size, weight_layout, None)
    out = addend if addend is not None else torch.empty(batch_shape + (rows, N), dtype=Bd.dtype, device=Bd.device)
    if out.numel():
        with torch.cuda.device(Bd.device):
            _lib.check(_lib.lib.vq_spmm_csr(
                data.contiguous().data_ptr(), indices.contiguous().data_ptr(), indptr.contiguous().data_ptr(), Bt.data_ptr(),
                _DT[Bd.dtype], batch, rows, K, N, data.shape[-1], K * N if Bt.ndim > 2 else 0,
                addend.data_ptr() if addend is not None else None, out.data_ptr(),
                _stream(Bd.device)), "spmm_csr")
    return out


def linear_mx(input, weight, bias=None, *, input_scale=None, weight_scale=None, block_size=None, input_code=None,
              weight_code=None, A_data=None, A_indices=None, A_indptr=None, weight_layout="kc"):
    """ops/quantized.py:295-348."""
    assert weight_layout in ("kc", "ck"), weight_layout
    _require_cuda(input, "linear_mx")
    from .gemm import mx_gemm
    dense = mx_gemm("linear_mx", input, weight, bias, input_scale, weight_scale, block_size, input_code, weight_code,
                    b_is_nk=(weight_layout == "kc"))
    if A_data is None:
        return dense
    return _spmm_csr(A_data, A_indices, A_indptr, weight, weight_scale, weight_code, block_size, weight_layout, dense)


def matmul_mx(self, other, *, input_scale=None, weight_scale=None, block_size=None, input_code=None, weight_code=None,
              A_data=None, A_indices=None, A_indptr=None, weight_layout="ck"):
    """ops/quantized.py:371-421."""
    assert weight_layout in ("kc", "ck"), weight_layout
    _require_cuda(self, "matmul_mx")
    from .gemm import mx_gemm
    dense = mx_gemm("matmul_mx", self, other, None, input_scale, weight_scale, block_size, input_code, weight_code,
                    b_is_nk=(weight_layout == "kc"))
    if A_data is None:
        return dense
    return _spmm_csr(A_data, A_indices, A_indptr, other, weight_scale, weight_code, block_size, weight_layout, dense)


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def conv2d_mx(input, weight, bias=None, stride=1, padding=0, dilation=1, groups=1, *, input_scale=None,
              weight_scale=None, block_size=None, input_code=None, weight_code=None, layout="nchw"):
    """ops/quantized.py:239-283: operands are decoded and scaled by this package's kernels (blocks
    along the channel axis go through the strided scale layout).  bf16 convolutions run on this library's
    tensor-core kernels (``conv_native``: implicit GEMM, grouped included, or patch matrix + GEMM; an ``"nchw"``
    result then comes back with channels-last strides), fp32 ones with one group as patch matrix + the tf32
    contraction; grouped fp32 and depthwise convolutions use the vendor kernel, as upstream.
    ``"nhwc"``: NHWC activations, HWIO weight, NHWC result."""
    assert layout in ("nchw", "nhwc"), layout
    _require_cuda(input, "conv2d_mx")
    from . import conv_native
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    native = conv_native.supported(input, weight, bias, groups, layout) and padding[0] >= 0 and padding[1] >= 0
    if native and input_code is None and conv_native.fusable_scale(input, input_scale, block_size, layout):
        # the activation's block scales are multiplied in while the operand tiles are staged: no decoded copy of the input
        return conv_native.conv2d_mx(input, weight, bias, stride, padding, dilation, weight_scale, weight_code, block_size,
                                     layout, x_scale=input_scale, groups=groups)
    x = _decode_operand("conv2d_mx", input, input_code, input_scale, block_size)
    if native:
        return conv_native.conv2d_mx(x, weight, bias, stride, padding, dilation, weight_scale, weight_code, block_size, layout,
                                     groups=groups)
    w = _decode_operand("conv2d_mx", weight, weight_code, weight_scale, block_size)
    if layout == "nhwc":
        x = x.permute(0, 3, 1, 2)
        if groups == 1:
            w = w.permute(3, 2, 0, 1)
        return torch.ops.aten.conv2d(x, w, bias, stride, padding, dilation, groups).permute(0, 2, 3, 1)
    return torch.ops.aten.conv2d(x, w, bias, stride, padding, dilation, groups)


# ---------------------------------------------------------------------------------------------
# dispatcher registration
# ---------------------------------------------------------------------------------------------
_libs = []      # Library handles must stay alive for the registrations to persist
_registered = False


def _op_defined(name: str) -> bool:
    try:
        getattr(torch.ops.quantized_ops, name)
        return True
    except (AttributeError, RuntimeError):
        return False


def _fake_like(x, *others):
    d = x.dtype
    for o in others:
        if o is not None:
            d = torch.promote_types(d, o.dtype) if o.ndim else d
    return torch.empty(x.shape, dtype=d, device=x.device)


def _fake_mx_shape(x, axes, block_size):
    shape = list(x.shape)
    for a in _norm_axes(axes, x.ndim):
        shape[a] = 1 if shape[a] <= block_size else -(-shape[a] // block_size)
    return shape


def _traced(name: str, fn):
    """With ``VOYAGER_B200_NVTX=1`` every dispatcher call of an op runs inside an NVTX range named
    ``quantized_ops::<op>``, so a timeline shows which kernels belong to which graph node; otherwise ``fn``
    itself is registered (no wrapper, no cost)."""
    import os
    if os.environ.get("VOYAGER_B200_NVTX") != "1":
        return fn
    import functools
    label = f"quantized_ops::{name}"

    @functools.wraps(fn)
    def ranged(*args, **kwargs):
        torch.cuda.nvtx.range_push(label)
        try:
            return fn(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()

    return ranged


def register() -> str:
    """Attach the CUDA kernels to ``torch.ops.quantized_ops``.  Returns ``"impl"`` when the upstream
    library definition was found (kernels added to it) or ``"def"`` when this package had to define
    the schemas itself.  Idempotent."""
    global _registered
    if _registered:
        return _registered
    mode = "impl" if _op_defined("quantize") else "def"
    if mode == "def":
        d = torch.library.Library("quantized_ops", "DEF")
        for schema in SCHEMAS.values():
            d.define(schema)
        _libs.append(d)
        m = torch.library.Library("quantized_ops", "IMPL", "Meta")
        m.impl("vmap", lambda x, q: torch.empty(x.shape, dtype=x.dtype, device=x.device))
        m.impl("quantize", lambda x, s, zp=None, axes=None, bs=None, qmap=None, oc=None: _fake_like(x, s, zp))
        m.impl("dequantize", lambda x, s, zp=None, axes=None, bs=None, iq=None, oq=None: _fake_like(x, s, zp))
        m.impl("calculate_mx_qparam", lambda x, axes, bs, qmax, p2=False, sq=None:
               torch.empty(_fake_mx_shape(x, axes, bs), dtype=x.dtype, device=x.device))
        m.impl("quantize_mx", lambda x, q, axes, bs, qmax, p2=False, sq=None, oc=None:
               (torch.empty(_fake_mx_shape(x, axes, bs), dtype=x.dtype, device=x.device),
                torch.empty(x.shape, dtype=x.dtype, device=x.device)))

        def _lin_fake(x, w, b=None, **kw):
            n = w.shape[0] if kw.get("weight_layout", "kc") == "kc" else w.shape[1]
            return torch.empty(list(x.shape[:-1]) + [n], dtype=x.dtype, device=x.device)

        def _mm_fake(a, b, **kw):
            bb = b if kw.get("weight_layout", "ck") == "ck" else b.transpose(-1, -2)
            return torch.empty(list(torch.broadcast_shapes(a.shape[:-2], bb.shape[:-2])) + [a.shape[-2], bb.shape[-1]],
                               dtype=a.dtype, device=a.device)

        def _conv_fake(x, w, b=None, stride=1, padding=0, dilation=1, groups=1, **kw):
            xm, wm = torch.empty(x.shape, device="meta", dtype=x.dtype), torch.empty(w.shape, device="meta", dtype=w.dtype)
            if kw.get("layout", "nchw") == "nhwc":
                xm = xm.permute(0, 3, 1, 2)
                wm = wm.permute(3, 2, 0, 1) if groups == 1 else wm
            y = torch.ops.aten.conv2d(xm, wm, None, _pair(stride), _pair(padding), _pair(dilation), groups)
            return y.permute(0, 2, 3, 1) if kw.get("layout", "nchw") == "nhwc" else y

        m.impl("conv2d_mx", _conv_fake)
        m.impl("linear_mx", _lin_fake)
        m.impl("matmul_mx", _mm_fake)

        # shapes as upstream's register_fake functions give them (ops/quantized.py:624-640, 703-732, 770-783, 865-879)
        def _csr_fake(x, max_pct):
            batch, (r, c) = tuple(x.shape[:-2]), x.shape[-2:]
            nnz = int(r * c * max_pct)
            return (x.new_empty(batch + (nnz,)), x.new_empty(batch + (nnz,), dtype=torch.int32),
                    x.new_empty(batch + (r + 1,), dtype=torch.int32))

        def _filter_fake(x, threshold, max_pct=0.01):
            return (*_csr_fake(x, max_pct), torch.empty_like(x))

        def _qmx_outlier_fake(x, q, axes, bs, qmax, p2=False, sq=None, oc=None, threshold=None, max_pct=0.01, off=0):
            return (*_csr_fake(x, max_pct), x.new_empty(_fake_mx_shape(x, axes, bs)),
                    torch.empty_like(x, memory_format=torch.contiguous_format))

        def _slice_fake(data, indices, indptr, dim=0, start=None, end=None, size_factor=1.0):
            ip = torch.empty_like(indptr)
            return torch.empty_like(data), torch.empty_like(indices), (ip[start:end + 1] if dim in (0, -2) else ip)

        def _spmm_fake(data, indices, indptr, B, B_scale=None, B_code=None, block_size=None, weight_layout="kc"):
            n = B.shape[-1] if weight_layout == "ck" else B.shape[-2]
            return data.new_empty(tuple(indptr.shape[:-1]) + (indptr.shape[-1] - 1, n))

        m.impl("filter_outlier", _filter_fake)
        m.impl("quantize_mx_outlier", _qmx_outlier_fake)
        m.impl("slice_csr_tensor", _slice_fake)
        m.impl("spmm_csr", _spmm_fake)
        _libs.append(m)
    c = torch.library.Library("quantized_ops", "IMPL", "CUDA")
    for name, fn in (("vmap", vmap), ("quantize", quantize), ("dequantize", dequantize),
                     ("calculate_mx_qparam", calculate_mx_qparam), ("quantize_mx", quantize_mx), ("conv2d_mx", conv2d_mx),
                     ("linear_mx", linear_mx), ("matmul_mx", matmul_mx)):
        c.impl(name, _traced(name, fn))
    for name, fn in (("filter_outlier", filter_outlier), ("quantize_mx_outlier", quantize_mx_outlier),
                     ("slice_csr_tensor", slice_csr_tensor), ("spmm_csr", spmm_csr)):
        if _op_defined(name):
            c.impl(name, _traced(name, fn))
    _libs.append(c)
    _registered = mode
    logger.info("quantized_ops CUDA kernels registered (%s mode)", mode)
    return mode
