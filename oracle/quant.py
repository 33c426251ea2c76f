"""Oracle: nibble packing, per-token quantizers, dequant.  Test infrastructure only."""
from __future__ import annotations

import torch

__all__ = ["pack_i4", "unpack_i4", "unpack_ui4", "sym_quant_codes", "sym_quant", "sym_quant_dynamic",
           "asym_quant_codes", "asym_quant_dynamic", "sym_dequant", "sym_dequant_moe", "kv_quant_pack",
           "kv_dequant", "sum_i4", "matmul_colrow", "pack_codes"]


def pack_codes(q: torch.Tensor) -> torch.Tensor:
    """Integer codes (any sign) -> uint8, element 2j in the low nibble of byte j
    (signrot/functional/quantization.py:45-53, kernels/include/int4.h:79-99)."""
    nib = (q.to(torch.int16) & 15).to(torch.uint8)
    if nib.shape[-1] % 2:
        nib = torch.nn.functional.pad(nib, (0, 1))
    return nib[..., 0::2] | (nib[..., 1::2] << 4)


def pack_i4(q: torch.Tensor) -> torch.Tensor:
    assert bool(((q >= -8) & (q <= 7)).all())
    return pack_codes(q)


def unpack_ui4(x: torch.Tensor) -> torch.Tensor:
    """uint8 -> int32 nibbles, unsigned (quantization.py:82-101)."""
    lo, hi = (x & 15).to(torch.int32), (x >> 4).to(torch.int32)
    return torch.stack((lo, hi), dim=-1).reshape(*x.shape[:-1], x.shape[-1] * 2)


def unpack_i4(x: torch.Tensor) -> torch.Tensor:
    """uint8 -> int32 nibbles, sign-extended (quantization.py:56-79)."""
    u = unpack_ui4(x)
    return torch.where(u >= 8, u - 16, u)


def _rint_codes(quot_h: torch.Tensor) -> torch.Tensor:
    """`__half2int_rn` on an fp16 quotient: round half to even, NaN -> 0, +-inf saturate."""
    f = quot_h.float()
    r = torch.round(f)  # ties to even
    r = torch.where(torch.isnan(r), torch.zeros_like(r), r)
    return r.clamp(-2.0 ** 31, 2.0 ** 31 - 1)


def sym_quant_codes(x_h: torch.Tensor, scale_h: torch.Tensor) -> torch.Tensor:
    """clamp(half2int_rn(x / s), -8, 7) per row (signrot/kernels/quant.cu:38-41, fused.cu:105-106).
    x_h fp16 [rows, cols], scale_h fp16 [rows] or [rows, 1]."""
    quot = (x_h.float() / scale_h.float().reshape(-1, 1)).half()
    return _rint_codes(quot).clamp(-8, 7).to(torch.int32)


def sym_quant(x_h, scale_h):
    """Packed codes for a given scale (kernel.sym_quant, functional/kernel.py:94-98)."""
    return pack_codes(sym_quant_codes(x_h, scale_h))


def sym_quant_dynamic(x_h: torch.Tensor, clip: float = 1.0, sign: torch.Tensor | None = None,
                      expert_ids: torch.Tensor | None = None):
    """Per-row amax -> scale = rn_h(amax / 7) [-> rn_h(scale * clip)] -> codes
    (signrot/kernels/fused.cu:83-110; nn/quantization.py:23-28; MoE sign: moe.cu:53-101).
    Returns (codes int32 [rows, cols], scale fp16 [rows, 1])."""
    x_h = x_h.reshape(-1, x_h.shape[-1])
    if sign is not None:
        s = sign if expert_ids is None else sign[expert_ids.long()]
        x_h = (x_h.float() * s.float()).half()
    amax = x_h.float().abs().amax(dim=-1, keepdim=True)
    scale = (amax / 7.0).half()
    if clip != 1.0:
        scale = (scale.float() * torch.tensor(clip, dtype=torch.float32)).half()
    return sym_quant_codes(x_h, scale), scale


def asym_quant_codes(x_h, scale_h, zero_h, lo: int, hi: int):
    """clamp(half2int_rn(x / s) + int(zero), lo, hi) (quant.cu:155-156, 202-203; fused.cu:191-192)."""
    quot = (x_h.float() / scale_h.float().reshape(-1, 1)).half()
    z = _rint_codes(zero_h.reshape(-1, 1))
    return (_rint_codes(quot) + z).clamp(lo, hi).to(torch.int32)


def asym_quant_dynamic(x_h: torch.Tensor, clip: float = 1.0, sign=None, expert_ids=None):
    """Per-row min/max -> scale, zero -> unsigned codes (signrot/kernels/fused.cu:156-198;
    nn/quantization.py:67-76).  Returns (codes, scale fp16 [rows,1], zero fp16 [rows,1])."""
    x_h = x_h.reshape(-1, x_h.shape[-1])
    if sign is not None:
        s = sign if expert_ids is None else sign[expert_ids.long()]
        x_h = (x_h.float() * s.float()).half()
    hmin = x_h.amin(dim=-1, keepdim=True)
    hmax = x_h.amax(dim=-1, keepdim=True)
    if clip != 1.0:
        c = torch.tensor(clip, dtype=torch.float32)
        hmin, hmax = (hmin.float() * c).half(), (hmax.float() * c).half()
    diff = (hmax.float() - hmin.float()).half()
    scale = (diff.float() / 15.0).half()
    ratio = (-hmin.float() / scale.float()).half()
    zero = torch.round(ratio.float()).half()
    return asym_quant_codes(x_h, scale, zero, 0, 15), scale, zero


def sym_dequant(acc: torch.Tensor, scale_row_h: torch.Tensor, scale_col_h: torch.Tensor) -> torch.Tensor:
    """rn_h((float(acc) * s_row) * s_col) (signrot/kernels/quant.cu:84-87)."""
    v = acc.to(torch.float32) * scale_row_h.float().reshape(-1, 1)
    return (v * scale_col_h.float().reshape(1, -1)).half()


def sym_dequant_moe(acc, scale_row_h, w_scales_h, expert_ids, zero_row=None, w_sum=None):
    """Expert-indexed dequant with exact int32 zero correction (signrot/kernels/moe.cu:216-225)."""
    e = expert_ids.long()
    a = acc.to(torch.int64)
    if zero_row is not None:
        a = a - zero_row.to(torch.int64).reshape(-1, 1) * w_sum.to(torch.int64)[e]
    v = a.to(torch.float32) * scale_row_h.float().reshape(-1, 1)
    return (v * w_scales_h.float()[e]).half()


def kv_quant_pack(x_h: torch.Tensor):
    """KV-cache quantizer (signrot/kernels/fused.cu:236-261; torch twin
    signrot/transformers/kv_cache.py:47-58).  Returns (packed uint8 [..., d/2], param fp16
    [..., 2] = (scale, zero))."""
    hmin = x_h.amin(dim=-1, keepdim=True)
    hmax = x_h.amax(dim=-1, keepdim=True)
    diff = (hmax.float() - hmin.float()).half()
    diff = torch.clamp(diff.float(), min=1e-5).half()
    scale = (diff.float() / 15.0).half()
    zero = -hmin
    shifted = (x_h.float() + zero.float()).half()
    scaled = (shifted.float() / scale.float()).half()
    q = torch.round(scaled.float()).clamp(0, 15).to(torch.int32)
    return pack_codes(q), torch.cat([scale, zero], dim=-1)


def kv_dequant(packed: torch.Tensor, param_h: torch.Tensor) -> torch.Tensor:
    """float(code) * scale - zero in fp32 (kernels/include/flashinfer/quantization.cuh:76)."""
    return unpack_ui4(packed).float() * param_h[..., 0:1].float() - param_h[..., 1:2].float()


def sum_i4(packed: torch.Tensor, signed: bool = True) -> torch.Tensor:
    """Row sums of 4-bit values (signrot/kernels/quant.cu:233-350)."""
    u = unpack_i4(packed) if signed else unpack_ui4(packed)
    return u.sum(dim=-1, keepdim=True).to(torch.int32)


def matmul_colrow(a_col_i8: torch.Tensor, b_row_i32: torch.Tensor) -> torch.Tensor:
    """Rank-1 int32 product (signrot/kernels/quant.cu:352-383)."""
    return (a_col_i8.to(torch.int32).reshape(-1, 1) * b_row_i32.to(torch.int32).reshape(1, -1))
