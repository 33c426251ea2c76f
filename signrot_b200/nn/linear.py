"""4-bit linear layers (signrot/nn/linear.py:7-135).

`forward` on a PackedQuantizedTensor runs one fused kernel (GEMM, zero correction, dequant,
bias); `forward_unfused` keeps the reference's operator chain (matmul -> colrow -> dequant)
for equivalence tests."""
from __future__ import annotations

import torch

from ..functional import kernel
from ..functional import quantization as qz


def _round_pack(weight: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    return qz.pack_i4((weight / scales.to(weight.device, weight.dtype)).round().to(torch.int8))


class Linear4bit(torch.nn.Module):
    """Symmetric per-channel int4 weights; activations arrive packed (signed codes, or unsigned
    codes plus zeros)."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.float16):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer('weight_scales', torch.zeros((out_features, 1), requires_grad=False))
        self.register_buffer('weight', torch.ones((out_features, in_features // 2), dtype=torch.uint8,
                                                  requires_grad=False))
        if bias:
            self.register_buffer('bias', torch.zeros((out_features), dtype=dtype))
        else:
            self.bias = None

    def _weight_sum(self):
        if not hasattr(self, 'weight_sum'):
            self.register_buffer('weight_sum', kernel.sum_i4(self.weight), persistent=False)
        return self.weight_sum

    def forward(self, x):
        if not isinstance(x, kernel.PackedQuantizedTensor):
            # float input: dequantize the weight and use a dense linear (linear.py:31-34)
            w = qz.sym_dequant(qz.unpack_i4(self.weight), self.weight_scales)
            return torch.nn.functional.linear(x, w, self.bias)
        wsum = self._weight_sum() if x.zeros_x is not None else None
        return kernel.w4a4_linear(x, self.weight, self.weight_scales, wsum, self.bias)

    def forward_unfused(self, x: kernel.PackedQuantizedTensor):
        q, s, z = x.quantized_x, x.scales_x, x.zeros_x
        if z is not None:
            acc = kernel.matmul_ui4_si4(q, self.weight)
            acc -= kernel.matmul_colrow_i8_i32(z, self._weight_sum().mT)
        else:
            acc = kernel.matmul_si4_si4(q, self.weight)
        out = kernel.sym_dequant(acc, s, self.weight_scales)
        return out + self.bias if self.bias is not None else out

    @staticmethod
    def from_float(module: torch.nn.Linear, weight_scales=None):
        """Packs `round(W / scale)`; W is expected to hold already-quantized values."""
        W = module.weight.data
        new = Linear4bit(module.in_features, module.out_features, bias=module.bias is not None,
                         dtype=W.dtype).to(W.dtype)
        if weight_scales is not None:
            assert weight_scales.shape == (module.out_features, 1), 'weight_scales should have shape (out_features, 1)'
            new.weight_scales.copy_(weight_scales.to(W.dtype))
            new.weight.copy_(_round_pack(W, weight_scales).cpu())
            if module.bias is not None:
                new.bias.copy_(module.bias)
        return new


def linear4bit_from_float_rtn(module: torch.nn.Linear, sign=None, mse=False) -> Linear4bit:
    """A float Linear on the GPU -> Linear4bit in one kernel: per-channel symmetric RTN (optionally
    with the MSE clipping search), SignRot sign refold, packing.  The route through the reference
    is rtn_fwrd (fake_quant/gptq_utils.py:411-465) -> ActQuantWrapper.enable_kernel
    (fake_quant/quant_utils.py:214-276) -> Linear4bit.from_float."""
    W = module.weight.data
    new = Linear4bit(module.in_features, module.out_features, bias=module.bias is not None, dtype=torch.float16)
    new = new.to(W.device)
    packed, scales = kernel.rtn_pack(W, sign=sign, mse=mse)
    new.weight = packed
    new.weight_scales = scales
    if module.bias is not None:
        new.bias = module.bias.data.to(torch.float16)
    return new


class AsymSymmLinear4bit(torch.nn.Module):
    """Variant whose activation codes are signed and whose zero term is always subtracted
    (linear.py:75-135)."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.float16):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer('weight', torch.ones((out_features, in_features // 2), dtype=torch.uint8,
                                                  requires_grad=False))
        self.register_buffer('weight_scales', torch.zeros((out_features, 1), requires_grad=False))
        self.register_buffer('weight_sum', torch.ones((out_features, 1), dtype=torch.int32, requires_grad=False))
        if bias:
            self.register_buffer('bias', torch.zeros((out_features), dtype=dtype))
        else:
            self.bias = None

    def forward(self, x):
        assert type(x) == kernel.PackedQuantizedTensor
        acc = kernel.matmul_si4_si4(x.quantized_x, self.weight)
        zeros = kernel.matmul_colrow_i8_i32(x.zeros_x, self.weight_sum.to(torch.int32).mT)
        out = kernel.sym_dequant(acc - zeros, x.scales_x, self.weight_scales)
        if self.bias is not None:
            out += self.bias
        return out

    @staticmethod
    def from_float(module: torch.nn.Linear, weight_scales=None):
        W = module.weight.data
        new = AsymSymmLinear4bit(module.in_features, module.out_features, bias=module.bias is not None,
                                 dtype=W.dtype).to(W.dtype)
        if weight_scales is not None:
            assert weight_scales.shape == (module.out_features, 1), 'weight_scales should have shape (out_features, 1)'
            new.weight_scales.copy_(weight_scales.to(W.dtype))
            packed = _round_pack(W, weight_scales)
            new.weight.copy_(packed.cpu())
            new.weight_sum.copy_(qz.unpack_i4(packed).sum(dim=-1, keepdim=True).to(torch.int32).cpu())
            if module.bias is not None:
                new.bias.copy_(module.bias)
        return new
