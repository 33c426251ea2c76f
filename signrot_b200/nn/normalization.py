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
        # other dtypes stay in their own precision, as the reference's module does for them
        inv_rms = torch.rsqrt(x.square().sum(dim=-1, keepdim=True) / self.mean_dim + self.eps)
        return x * inv_rms
