"""Weightless RMSNorm (signrot/nn/normalization.py:7-30); the scale vector is folded into the
following linears offline."""
import torch

from ..functional import kernel


class RMSNorm(torch.nn.Module):
    def __init__(self, mean_dim: int, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.mean_dim = mean_dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype == torch.float16:
            return kernel.rmsnorm(x, self.eps, self.mean_dim)
        return self.forward_reference(x)

    def forward_reference(self, x: torch.Tensor) -> torch.Tensor:
        dt = x.dtype
        xf = x.to(torch.float32) if dt == torch.float16 else x
        var = xf.pow(2).sum(-1, keepdim=True) / self.mean_dim
        return (xf * torch.rsqrt(var + self.eps)).to(dt)
