"""Oracle: the online rotation.  Test infrastructure only."""
from __future__ import annotations

import math

import torch

__all__ = ["fwht", "rotate", "rotate_heads", "had_scale_f32"]


def had_scale_f32(n: int) -> torch.Tensor:
    """1/sqrt(n) as the reference evaluates it: fp32 (signrot/functional/hadamard.py:81)."""
    return (1.0 / torch.tensor(n).sqrt()).float()


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Walsh-Hadamard transform over the last dimension (a power of two),
    Sylvester order, radix-2 butterflies in x's dtype -- the transform
    fast_hadamard_transform.hadamard_transform applies (un-vendored dependency; contract
    restated from its call sites signrot/functional/hadamard.py:81,85 and pinned by the
    reference's own butterfly signrot/functional/hadamard.py:43-65)."""
    n = x.shape[-1]
    assert n & (n - 1) == 0
    y = x.reshape(-1, n).clone()
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        a, b = y[:, :, 0, :], y[:, :, 1, :]
        y = torch.stack((a + b, a - b), dim=2)
        h *= 2
    return y.reshape(x.shape)


def _round(v: torch.Tensor, dtype) -> torch.Tensor:
    return v.to(dtype).float() if dtype != torch.float32 else v


def rotate(x: torch.Tensor, hadK: torch.Tensor | None = None, K: int = 1, sign: torch.Tensor | None = None,
           fp32_mode: bool = False, cast_in_to_f16: bool = False, out_dtype=None) -> torch.Tensor:
    """OnlineHadamard.forward (signrot/nn/hadamard.py:26-42) = matmul_hadU_cuda
    (signrot/functional/hadamard.py:78-87) * had_adj_sign, with the reference's rounding
    points: the Walsh-Hadamard sums are fp32, scaled by 1/sqrt(n) and rounded to the tensor
    dtype; the had-K factor is a matmul in that dtype (fp32 accumulation, rounded again); the
    +-1 sign is exact.  fp32_mode: no rounding until the final cast."""
    n = x.shape[-1]
    work = x.dtype
    if cast_in_to_f16 and x.dtype == torch.bfloat16:
        x = x.to(torch.float16)  # fake_quant/quant_utils.py:284
        work = torch.float16
    if fp32_mode:
        work = torch.float32
    out_dtype = out_dtype or x.dtype
    xf = x.float().reshape(-1, K, n // K)
    z = fwht(xf) * had_scale_f32(n)
    z = _round(z, work)
    if K > 1:
        h = hadK.float()
        z = torch.matmul(h.view(1, K, K), z)
        z = _round(z, work)
    z = z.reshape(-1, n)
    if sign is not None:
        z = z * sign.float()
    return z.to(out_dtype).reshape(x.shape)


def rotate_heads(x: torch.Tensor, heads: int, fp32_mode: bool = False, cast_in_to_f16: bool = False) -> torch.Tensor:
    """o_proj input rotation (fake_quant/quant_utils.py:287-291): [-1, heads, head_dim] ->
    transpose -> Hadamard over heads (scale 1/sqrt(heads)) -> transpose back."""
    n = x.shape[-1]
    d = n // heads
    if cast_in_to_f16 and x.dtype == torch.bfloat16:
        x = x.to(torch.float16)
    t = x.reshape(-1, heads, d).transpose(1, 2)
    t = rotate(t.contiguous(), None, 1, None, fp32_mode=fp32_mode)
    return t.transpose(1, 2).reshape(x.shape)
