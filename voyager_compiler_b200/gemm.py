"""MX-quantized GEMM: ``Y = deq(A) @ deq(B)^T`` for ``linear_mx`` / ``matmul_mx``
(src/voyager_compiler/ops/quantized.py:295-348, :371-421).

``deq(T) = code[T] * expand(scale)`` is formed in the operand dtype (one rounding to bf16 for
bf16 operands), the product accumulates in fp32 and the result is stored in the operand dtype.
bf16 operands run on this library's tcgen05 GEMM in every layout: ``[N, K]`` weights directly,
``[.., K, N]`` right operands (``matmul_mx``, ``"ck"`` linear weights) through the decode kernel that
writes them transposed.  fp32 operands are decoded by this package's kernels and contracted by the same
tensor cores as tf32 (the low 13 bits of an operand are ignored: exact for MX-decoded values with
power-of-two scales; fp32 accumulation and result); ``VOYAGER_B200_FP32=vendor`` keeps the vendor fp32 GEMM.
"""
from __future__ import annotations

from typing import Optional

import torch


def mx_gemm(name: str, a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], a_scale, b_scale, block_size,
            a_code, b_code, b_is_nk: bool) -> torch.Tensor:
    """``a``: [..., M, K]; ``b``: [N, K] when ``b_is_nk`` (linear's weight) else [..., K, N]."""
    from . import ops
    from .gemm_native import (f32_supported, native_batched_nk_supported, native_f32_gemm, native_kn_supported, native_mx_gemm,
                              native_mx_gemm_batched_nk, native_mx_gemm_kn, native_supported)

    if native_supported(a, b, bias, a_scale, b_scale, block_size, a_code, b_code, b_is_nk):
        return native_mx_gemm(a, b, bias, a_scale, b_scale, block_size, a_code, b_code)
    if not b_is_nk and native_kn_supported(a, b, bias):
        return native_mx_gemm_kn(name, a, b, bias, a_scale, b_scale, block_size, a_code, b_code)
    if b_is_nk and bias is None and native_batched_nk_supported(a, b):
        return native_mx_gemm_batched_nk(name, a, b, a_scale, b_scale, block_size, a_code, b_code)
    if f32_supported(a, b, bias, b_is_nk):
        return native_f32_gemm(name, a, b, bias, a_scale, b_scale, block_size, a_code, b_code, b_is_nk)
    # K not a multiple of 8 (4 for fp32), batch shapes that only broadcast, mixed dtypes: operands are decoded by this
    # package's dequantize kernel and multiplied by the vendor GEMM.
    da = ops._decode_operand(name, a, a_code, a_scale, block_size)
    db = ops._decode_operand(name, b, b_code, b_scale, block_size)
    if b_is_nk:
        return torch.nn.functional.linear(da, db, bias)
    out = torch.matmul(da, db)
    return out if bias is None else out + bias
