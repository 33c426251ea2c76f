"""Oracle: integer GEMM and the quantized linear.  Test infrastructure only."""
from __future__ import annotations

import torch

from .quant import unpack_i4, unpack_ui4, sym_dequant, sym_dequant_moe

__all__ = ["matmul_i4", "w4a4_linear", "matmul_grouped_ref"]


def matmul_i4(a_packed: torch.Tensor, b_packed: torch.Tensor, a_unsigned: bool = False) -> torch.Tensor:
    """int32 unpack(A) @ unpack(B)^T (signrot/kernels/gemm.cu:7-85).  Evaluated in fp32 by
    BLAS, which is exact here: every partial sum is an integer of magnitude <= 64*K < 2^24
    (signed) or <= 120*K (unsigned A; exact for K <= 139810), else in fp64."""
    a = (unpack_ui4(a_packed) if a_unsigned else unpack_i4(a_packed))
    b = unpack_i4(b_packed)
    k = a.shape[-1]
    dt = torch.float32 if (120 if a_unsigned else 64) * k < 2 ** 24 else torch.float64
    return (a.to(dt) @ b.to(dt).T).to(torch.int32)


def w4a4_linear(a_packed, a_scale_h, w_packed, w_scale_h, a_zero=None, w_sum=None, bias_h=None):
    """Linear4bit.forward on packed input (signrot/nn/linear.py:36-50)."""
    acc = matmul_i4(a_packed, w_packed, a_unsigned=a_zero is not None)
    if a_zero is not None:
        acc = acc - a_zero.to(torch.int32).reshape(-1, 1) * w_sum.to(torch.int32).reshape(1, -1)
    out = sym_dequant(acc, a_scale_h, w_scale_h)
    if bias_h is not None:
        out = (out.float() + bias_h.float()).half()
    return out


def matmul_grouped_ref(a_list, b_list, a_unsigned=False):
    """Per-problem dense GEMMs: what the grouped kernel must equal bit for bit
    (benchmarks/test_grouped_gemm.py:76-91)."""
    return [matmul_i4(a, b, a_unsigned) for a, b in zip(a_list, b_list)]
