"""Binding of the tcgen05 MX GEMM kernels (``vq_linear_mx`` fused, ``vq_gemm_bf16_tn`` plain)."""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from . import _lib

_status: Dict[str, torch.Tensor] = {}


def _device_key(device) -> torch.device:
    """``cuda`` without an index means the current device: one status word per physical device,
    whichever way the caller names it."""
    d = torch.device(device)
    if d.type != "cuda":
        raise ValueError(f"the GEMM status word lives on a CUDA device, not on {d}")
    return torch.device("cuda", torch.cuda.current_device() if d.index is None else d.index)


def _status_tensor(device) -> torch.Tensor:
    key = str(_device_key(device))
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _status[key]


def gemm_status(device="cuda") -> int:
    """Non-zero when a bounded wait inside a GEMM kernel on ``device`` ran out since the last
    call (1 producer, 2 MMA issuer, 3 epilogue): the result of that GEMM is then not to be used.
    Synchronises the device and clears the flag.  The ops do not poll it (that would synchronise
    every call); callers check it at a point where they synchronise anyway, or set
    ``VOYAGER_B200_GEMM_CHECK=1`` to have every native GEMM call check it and raise."""
    t = _status_tensor(device)
    v = int(t.item())
    t.zero_()
    return v


def _debug_check(device, what: str) -> None:
    if os.environ.get("VOYAGER_B200_GEMM_CHECK") == "1":
        v = gemm_status(device)
        if v:
            raise _lib.VoyagerB200Error(f"{what}: a bounded wait inside the GEMM kernel ran out (role {v}); the result is invalid")


def _mode() -> str:
    """``plain`` (default): operands dequantised by this package's dequantize kernel, then the
    TMA-fed tcgen05 GEMM.  ``fused``: dequantisation inside the GEMM's operand staging (no
    dequantised copy in HBM; slower on a one-CTA 128x256 tile because the staging warps cannot keep
    enough loads in flight).  ``cublas``: dequantize kernel + the vendor GEMM (for A/B timing)."""
    return os.environ.get("VOYAGER_B200_GEMM", "plain")


def _is_rows_by_kblocks(scale, rows, K, block) -> bool:
    return scale is not None and scale.dtype == torch.bfloat16 and tuple(scale.shape) == (rows, K // block)


def native_supported(a, b, bias, a_scale, b_scale, block_size, a_code, b_code, b_is_nk) -> bool:
    if _mode() == "cublas" or not b_is_nk:
        return False
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or b.ndim != 2 or a.ndim < 1:
        return False
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.ndim != 1 or bias.shape[0] != b.shape[0]):
        return False
    K = a.shape[-1]
    return K == b.shape[1] and K % 8 == 0 and K > 0


_decoded_weights: Dict[tuple, tuple] = {}


def _weight_cache_entries() -> int:
    """How many decoded weights are kept between calls (``VOYAGER_B200_WEIGHT_CACHE``, default 8; 0 disables)."""
    try:
        return max(0, int(os.environ.get("VOYAGER_B200_WEIGHT_CACHE", "8")))
    except ValueError:
        return 8


def _decoded_weight(name, b, b_code, b_scale, block_size):
    """``deq(b)`` of a 2-D ``[N, K]`` linear weight.  Weights are static buffers of the converted graph, so
    the last few decoded copies are kept, keyed by the identity, address and version counter of the tensors
    involved (weak references: an entry is never used for another tensor that reuses the address; an
    in-place update of the weight bumps its version and misses)."""
    import weakref
    from . import ops

    limit = _weight_cache_entries()
    if b_scale is None and b_code is None:
        return b.contiguous()
    if limit == 0:
        return ops._decode_operand(name, b, b_code, b_scale, block_size).contiguous()
    parts = [t for t in (b, b_scale, b_code) if t is not None]
    key = tuple((id(t), t.data_ptr(), t._version) for t in parts) + (block_size,)
    hit = _decoded_weights.get(key)
    if hit is not None and all(r() is t for r, t in zip(hit[0], parts)):
        return hit[1]
    db = ops._decode_operand(name, b, b_code, b_scale, block_size).contiguous()
    while len(_decoded_weights) >= limit:
        _decoded_weights.pop(next(iter(_decoded_weights)))
    _decoded_weights[key] = ([weakref.ref(t) for t in parts], db)
    return db


def native_mx_gemm(a, b, bias, a_scale, b_scale, block_size, a_code, b_code):
    from . import ops

    K = a.shape[-1]
    N = b.shape[0]
    lead = a.shape[:-1]
    M = 1
    for d in lead:
        M *= d
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    if M == 0 or N == 0:
        return out.reshape(*lead, N)
    a2 = a.reshape(M, K)
    a_sc2 = a_scale.reshape(M, -1) if a_scale is not None and a_scale.ndim >= 2 else a_scale
    stream = torch.cuda.current_stream(a.device).cuda_stream
    bias_c = bias.contiguous() if bias is not None else None
    with torch.cuda.device(a.device):
        st = _status_tensor(a.device)
        fused = (_mode() == "fused" and a_code is None and b_code is None and block_size == 32 and K % 64 == 0
                 and _is_rows_by_kblocks(a_sc2, M, K, 32) and _is_rows_by_kblocks(b_scale, N, K, 32))
        if fused:
            ac, bc = a2.contiguous(), b.contiguous()
            asc, bsc = a_sc2.contiguous(), b_scale.contiguous()
            rc = _lib.lib.vq_linear_mx(ac.data_ptr(), asc.data_ptr(), bc.data_ptr(), bsc.data_ptr(),
                                       bias_c.data_ptr() if bias_c is not None else None, out.data_ptr(), M, N, K, 32,
                                       st.data_ptr(), stream)
            _lib.check(rc, "linear_mx")
        else:
            da = ops._decode_operand("linear_mx", a2, a_code, a_sc2, block_size).contiguous()
            db = _decoded_weight("linear_mx", b, b_code, b_scale, block_size)
            rc = _lib.lib.vq_gemm_bf16_tn(da.data_ptr(), db.data_ptr(), bias_c.data_ptr() if bias_c is not None else None,
                                          out.data_ptr(), M, N, K, st.data_ptr(), stream)
            _lib.check(rc, "linear_mx")
    _debug_check(a.device, "linear_mx")
    return out.reshape(*lead, N)


def native_kn_supported(a, b, bias) -> bool:
    """Right operand in ``[.., K, N]`` order (``matmul_mx``, ``"ck"`` weights): bf16, K a multiple of 8, N even,
    and batch dimensions that are either equal on both sides or absent on the right."""
    if _mode() == "cublas":
        return False
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.ndim < 2 or b.ndim < 2:
        return False
    K, N = b.shape[-2], b.shape[-1]
    if a.shape[-1] != K or K % 8 or K == 0 or N % 2:
        return False
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.ndim != 1 or bias.shape[0] != N):
        return False
    if b.ndim == 2 or all(d == 1 for d in b.shape[:-2]):
        return True
    return tuple(a.shape[:-2]) == tuple(b.shape[:-2])


_kn_weights: Dict[tuple, tuple] = {}


def _decode_transposed(name, b, b_code, b_scale, block_size):
    """``[batch, N, K]`` bf16: ``deq(b)`` of a ``[batch, K, N]`` operand, transposed by the decode kernel."""
    from . import ops

    K, N = b.shape[-2], b.shape[-1]
    batch = b.numel() // (K * N) if K * N else 0
    x = b.contiguous()
    if b_code is not None:
        x = ops._decode_operand(name, x, b_code, None, None)
    sc, rows = None, 0
    if b_scale is not None:
        want = tuple(b.shape[:-2]) + (-(-K // block_size) if block_size else 0, N)
        if block_size and block_size % 2 == 0 and b_scale.dtype == torch.bfloat16 and tuple(b_scale.shape) == want:
            sc, rows = b_scale.contiguous(), want[-2]
        else:                                                        # any other scale placement: the general decode first
            x = ops.dequantize(x, b_scale, None, None, block_size)
    out = torch.empty((batch, N, K), dtype=torch.bfloat16, device=b.device)
    if out.numel():
        with torch.cuda.device(b.device):
            rc = _lib.lib.vq_dequantize_transpose(x.data_ptr(), sc.data_ptr() if sc is not None else None, batch, K, N,
                                                  block_size or 0, rows, out.data_ptr(),
                                                  torch.cuda.current_stream(b.device).cuda_stream)
            _lib.check(rc, name)
    return out


def native_batched_nk_supported(a, b) -> bool:
    """``matmul_mx(..., weight_layout="kc")`` on batched operands: right operand ``[.., N, K]`` with the batch
    dimensions of the left one."""
    if _mode() == "cublas" or a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.ndim < 3 or b.ndim < 3:
        return False
    K = a.shape[-1]
    return K == b.shape[-1] and K % 8 == 0 and K > 0 and tuple(a.shape[:-2]) == tuple(b.shape[:-2])


def native_mx_gemm_batched_nk(name, a, b, a_scale, b_scale, block_size, a_code, b_code):
    from . import ops

    K, M, N = a.shape[-1], a.shape[-2], b.shape[-2]
    da = ops._decode_operand(name, a, a_code, a_scale, block_size).contiguous()
    db = ops._decode_operand(name, b, b_code, b_scale, block_size).contiguous()
    out = torch.empty(tuple(a.shape[:-1]) + (N,), dtype=torch.bfloat16, device=a.device)
    batch = out.numel() // (M * N) if M * N else 0
    if out.numel():
        with torch.cuda.device(a.device):
            rc = _lib.lib.vq_gemm_bf16_tn_batched(da.data_ptr(), db.data_ptr(), out.data_ptr(), batch, M, N, K, 0, 0,
                                                  _status_tensor(a.device).data_ptr(), torch.cuda.current_stream(a.device).cuda_stream)
            _lib.check(rc, name)
        _debug_check(a.device, name)
    return out


def native_mx_gemm_kn(name, a, b, bias, a_scale, b_scale, block_size, a_code, b_code):
    """``deq(a) @ deq(b)`` with ``b`` in ``[.., K, N]`` order on the tcgen05 GEMM: ``b`` is decoded into
    ``[batch, N, K]`` by one kernel, ``a`` by the dequantize kernel, and one persistent launch walks
    the output tiles of all batches.  A 2-D ``b`` (a ``"ck"`` weight) is shared by every row of ``a``;
    its decoded form is kept between calls, keyed by the identity and version of its tensors."""
    import weakref
    from . import ops

    K, N = b.shape[-2], b.shape[-1]
    shared_b = b.ndim == 2 or all(d == 1 for d in b.shape[:-2])
    lead = tuple(a.shape[:-1])
    if shared_b:
        parts = [t for t in (b, b_scale, b_code) if t is not None]
        key = tuple((id(t), t._version, t.data_ptr()) for t in parts) + (block_size,)
        hit = _kn_weights.get(key)
        if hit is not None and all(r() is t for r, t in zip(hit[0], parts)):
            bt = hit[1]
        else:
            bt = _decode_transposed(name, b.reshape(K, N), b_code, b_scale.reshape(-1, N) if b_scale is not None and b_scale.ndim >= 2 else b_scale,
                                    block_size)
            if len(_kn_weights) >= 8:
                _kn_weights.pop(next(iter(_kn_weights)))
            _kn_weights[key] = ([weakref.ref(t) for t in parts], bt)
        batch, M = 1, a.numel() // K
    else:
        bt = _decode_transposed(name, b, b_code, b_scale, block_size)
        batch, M = bt.shape[0], a.shape[-2]
    da = ops._decode_operand(name, a, a_code, a_scale, block_size).contiguous()
    out = torch.empty(lead + (N,), dtype=torch.bfloat16, device=a.device)
    if out.numel() == 0:
        return out
    stream = torch.cuda.current_stream(a.device).cuda_stream
    with torch.cuda.device(a.device):
        st = _status_tensor(a.device)
        if batch == 1:
            bias_c = bias.contiguous() if bias is not None else None
            rc = _lib.lib.vq_gemm_bf16_tn(da.data_ptr(), bt.data_ptr(), bias_c.data_ptr() if bias_c is not None else None,
                                          out.data_ptr(), M, N, K, st.data_ptr(), stream)
        else:
            rc = _lib.lib.vq_gemm_bf16_tn_batched(da.data_ptr(), bt.data_ptr(), out.data_ptr(), batch, M, N, K, 0, 0,
                                                  st.data_ptr(), stream)
        _lib.check(rc, name)
    _debug_check(a.device, name)
    if batch > 1 and bias is not None:
        out = out + bias
    return out


def linear_mx_dynamic(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *, qmap: torch.Tensor,
                      weight_scale: Optional[torch.Tensor] = None, block_size: int = 32, quant_max: float = 127.0,
                      force_scale_power_of_two: bool = True, scale_qmap: Optional[torch.Tensor] = None,
                      weight_code: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``linear_mx`` on an activation that is quantized on the fly: the value of

        s, q = quantize_mx(x, qmap, (-1,), block_size, quant_max, force_scale_power_of_two, scale_qmap)
        linear_mx(q, weight, bias, input_scale=s, weight_scale=weight_scale, block_size=block_size, weight_code=weight_code)

    (the node pair the converter emits for a dynamically quantized linear, ops/quantized.py:502-529 and :286-348)
    without the round trip of codes and scales through HBM: one pass writes ``codes * scale`` of the
    activation straight into the GEMM's left operand (the MX fake-quantize form of the quantize kernel), the
    weight is decoded as ``linear_mx`` decodes it, then the tcgen05 GEMM runs.  Bit-identical to the two ops.
    The one-pass form takes bf16 ``x`` of shape [..., K] and ``weight`` [N, K] with K a multiple of 8;
    anything else runs as the two ops."""
    from . import fake_quantize, ops

    if x.device.type != "cuda":
        raise RuntimeError("linear_mx_dynamic: CUDA tensors only; there is no CPU path")
    if not native_supported(x, weight, bias, None, weight_scale, block_size, None, weight_code, True):
        # shapes / dtypes the one-pass form does not take (fp32 operands, K not a multiple of 8): the two ops
        s, q = ops.quantize_mx(x, qmap, (-1,), block_size, quant_max, force_scale_power_of_two, scale_qmap)
        return ops.linear_mx(q, weight, bias, input_scale=s, weight_scale=weight_scale, block_size=block_size,
                             weight_code=weight_code)
    K, N = x.shape[-1], weight.shape[0]
    lead = x.shape[:-1]
    M = x.numel() // K if K else 0
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    if M == 0 or N == 0:
        return out.reshape(*lead, N)
    _, da = fake_quantize.mx_fake_quantize(x.reshape(M, K), qmap, -1, block_size, quant_max, force_scale_power_of_two, scale_qmap)
    bias_c = bias.contiguous() if bias is not None else None
    with torch.cuda.device(x.device):
        db = _decoded_weight("linear_mx", weight, weight_code, weight_scale, block_size)
        rc = _lib.lib.vq_gemm_bf16_tn(da.data_ptr(), db.data_ptr(), bias_c.data_ptr() if bias_c is not None else None,
                                      out.data_ptr(), M, N, K, _status_tensor(x.device).data_ptr(),
                                      torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc, "linear_mx_dynamic")
    _debug_check(x.device, "linear_mx_dynamic")
    return out.reshape(*lead, N)


def linear_mx_packed(x, w, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``deq(x) @ deq(w).T (+ bias)`` in bf16 for two :class:`~voyager_compiler_b200.model_quant.PackedMX`
    operands with 8-bit integer codes and blocks of 32 along the last axis (``quantize_tensors_mx(...,
    code_bits=8)`` through an integer table): the GEMM reads the packed bytes and converts inside its
    operand staging.  Shapes the packed kernel does not take (M <= 128, K not a multiple of 256) are
    dequantised by ``dequantize_packed`` and multiplied by the TMA-fed GEMM."""
    from . import model_quant as mq

    for t, nm in ((x, "x"), (w, "w")):
        if t.code_bits != 8 or t.block != 32:
            raise NotImplementedError(f"linear_mx_packed: {nm} needs 8-bit codes and blocks of 32")
        lv = t.levels
        if lv.numel() != 256 or float(lv[1]) != 1.0 or float(lv[255]) != -1.0:
            raise NotImplementedError(f"linear_mx_packed: {nm} must hold two's-complement integer codes")
    K = x.shape[-1]
    if len(w.shape) != 2 or w.shape[1] != K:
        raise ValueError("linear_mx_packed: w must be [N, K] with the K of x")
    N = w.shape[0]
    lead = tuple(x.shape[:-1])
    M = 1
    for d in lead:
        M *= d
    dev = x.codes.device
    out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    if M == 0 or N == 0:
        return out.reshape(*lead, N)
    bias_c = bias.to(torch.bfloat16).contiguous() if bias is not None else None
    stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        st = _status_tensor(dev)
        if M > 128 and K % 256 == 0:
            xs = x.scale.to(torch.bfloat16).reshape(M, K // 32).contiguous()
            ws = w.scale.to(torch.bfloat16).reshape(N, K // 32).contiguous()
            rc = _lib.lib.vq_linear_mx_packed(x.codes.data_ptr(), xs.data_ptr(), w.codes.data_ptr(), ws.data_ptr(),
                                              bias_c.data_ptr() if bias_c is not None else None, out.data_ptr(), M, N, K, 32,
                                              st.data_ptr(), stream)
            _lib.check(rc, "linear_mx_packed")
        else:
            da = mq.dequantize_packed(x, torch.bfloat16).reshape(M, K)
            db = mq.dequantize_packed(w, torch.bfloat16)
            rc = _lib.lib.vq_gemm_bf16_tn(da.data_ptr(), db.data_ptr(), bias_c.data_ptr() if bias_c is not None else None,
                                          out.data_ptr(), M, N, K, st.data_ptr(), stream)
            _lib.check(rc, "linear_mx_packed")
    return out.reshape(*lead, N)


def f32_supported(a, b, bias, b_is_nk: bool) -> bool:
    """fp32 operands go to the tensor cores as tf32 (``vq_gemm_f32_tn_batched``) unless ``VOYAGER_B200_FP32=vendor``.
    Shapes: a 2-D right operand shared by every row of ``a``, or equal batch dimensions on both sides."""
    if os.environ.get("VOYAGER_B200_FP32", "tensor") == "vendor" or _mode() == "cublas":
        return False
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.ndim < 1 or b.ndim < 2 or not a.is_cuda:
        return False
    K = a.shape[-1]
    if K <= 0 or K % 4 or K != (b.shape[-1] if b_is_nk else b.shape[-2]):
        return False
    N = b.shape[-2] if b_is_nk else b.shape[-1]
    if bias is not None and (bias.dtype != torch.float32 or bias.ndim != 1 or bias.shape[0] != N):
        return False
    return b.ndim == 2 or (a.ndim == b.ndim and a.shape[:-2] == b.shape[:-2])


def native_f32_gemm(name, a, b, bias, a_scale, b_scale, block_size, a_code, b_code, b_is_nk: bool) -> torch.Tensor:
    """``deq(a) @ deq(b)^T`` (``b_is_nk``) or ``deq(a) @ deq(b)`` for fp32 operands: decoded by this package's kernels
    (the 2-D linear weight kept between calls), a ``[.., K, N]`` right operand made ``[.., N, K]`` by one copy, then the
    tf32 tensor-core contraction with fp32 accumulation and an fp32 result."""
    from . import ops

    dev = a.device
    da = ops._decode_operand(name, a, a_code, a_scale, block_size).contiguous()
    if b_is_nk and b.ndim == 2:
        db = _decoded_weight(name, b, b_code, b_scale, block_size)
    else:
        db = ops._decode_operand(name, b, b_code, b_scale, block_size)
        db = (db if b_is_nk else db.transpose(-1, -2)).contiguous()
    K = da.shape[-1]
    N = db.shape[-2]
    if db.ndim == 2:
        batch, M, b_shared, lead = 1, da.numel() // K, 1, da.shape[:-1]
    else:
        M, b_shared, lead = da.shape[-2], 0, da.shape[:-1]
        batch = da.numel() // (M * K) if M else 0
    out = torch.empty((*lead, N), dtype=torch.float32, device=dev)
    if out.numel() == 0:
        return out
    fused_bias = bias is not None and batch == 1
    bias_c = bias.contiguous() if fused_bias else None
    with torch.cuda.device(dev):
        rc = _lib.lib.vq_gemm_f32_tn_batched(da.data_ptr(), db.data_ptr(), bias_c.data_ptr() if bias_c is not None else None,
                                             out.data_ptr(), batch, M, N, K, 0, b_shared, _status_tensor(dev).data_ptr(),
                                             torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(rc, name)
    _debug_check(dev, name)
    return out if bias is None or fused_bias else out + bias
