"""Integer/fake-quant helpers of `signrot.functional.quantization`
(signrot/functional/quantization.py:5-101): nibble packing and the floating-point
quantize/dequantize formulas.  Pure tensor code that runs on whatever device its inputs
live on; it is host-side/offline code, not part of the GPU hot path."""
from __future__ import annotations

import torch


def two_compl(x, bits: int):
    """Two's-complement representation of signed integers in `bits` bits."""
    return torch.where(x < 0, x + (1 << bits), x)


def get_minq_maxq(bits: int, sym: bool):
    """(minq, maxq) as 0-d tensors: [-2^(b-1), 2^(b-1)-1] symmetric, [0, 2^b-1] otherwise."""
    if sym:
        maxq = torch.tensor(2 ** (bits - 1) - 1)
        return -maxq - 1, maxq
    return torch.tensor(0), torch.tensor(2 ** bits - 1)


def asym_quant(x, scale, zero, maxq):
    scale, zero = scale.to(x.device), zero.to(x.device)
    return torch.clamp(torch.round(x / scale) + zero, 0, maxq), scale, zero


def asym_dequant(q, scale, zero):
    return scale * (q - zero)


def asym_quant_dequant(x, scale, zero, maxq):
    return asym_dequant(*asym_quant(x, scale, zero, maxq))


def sym_quant(x, scale, maxq, minq=None):
    scale = scale.to(x.device)
    lo = -(maxq + 1) if minq is None else minq
    return torch.clamp(torch.round(x / scale), lo, maxq), scale


def sym_dequant(q, scale):
    return scale * q


def sym_quant_dequant(x, scale, maxq, minq=None):
    return sym_dequant(*sym_quant(x, scale, maxq, minq=minq))


def pack_i4(q):
    """Signed integers in [-8, 7] -> uint8 with element 2j in the low nibble of byte j."""
    assert torch.is_signed(q), 'The tensor to be packed should be signed int'
    assert bool(((q >= -8) & (q <= 7)).all())
    nib = two_compl(q.to(torch.int8), 4).to(torch.uint8)
    return nib[..., 0::2] | (nib[..., 1::2] << 4)


def _unpack_nibbles(x, signed: bool, dtype):
    assert x.dtype == torch.uint8, 'The tensor to be unpacked should be stored in uint8'
    lo = (x & 0x0F).to(torch.int16)
    hi = (x >> 4).to(torch.int16)
    both = torch.stack((lo, hi), dim=-1).reshape(*x.shape[:-1], x.shape[-1] * 2)
    if signed:
        both = torch.where(both >= 8, both - 16, both)
    return both.to(dtype)


def unpack_i4(x: torch.Tensor, dtype=torch.int32):
    """Inverse of pack_i4 (sign-extended)."""
    return _unpack_nibbles(x, True, dtype)


def unpack_ui4(x: torch.Tensor):
    """Unsigned nibbles as int32."""
    return _unpack_nibbles(x, False, torch.int32)
