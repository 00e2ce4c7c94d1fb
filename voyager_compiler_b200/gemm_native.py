"""Binding of the tcgen05 MX GEMM kernel (filled in with the kernel)."""
from __future__ import annotations


def native_supported(a, b, bias, a_scale, b_scale, block_size, a_code, b_code, b_is_nk) -> bool:
    return False


def native_mx_gemm(a, b, bias, a_scale, b_scale, block_size, a_code, b_code):
    raise NotImplementedError
