"""Oracle: RMSNorm, rotary embedding, SwiGLU.  Test infrastructure only."""
from __future__ import annotations

import torch

__all__ = ["rmsnorm", "rope_qk", "swiglu"]


def rmsnorm(x_h: torch.Tensor, eps: float, mean_dim: int) -> torch.Tensor:
    """rn_h(x * rsqrt(sum(x^2)/mean_dim + eps)), fp32 (signrot/kernels/fused.cu:288-301;
    nn/normalization.py:24-30)."""
    xf = x_h.float()
    var = xf.pow(2).sum(-1, keepdim=True) / mean_dim
    return (xf * torch.rsqrt(var + eps)).half()


def rope_qk(q_h, k_h, cos_h, sin_h):
    """HF rotate-half rotary embedding with fp16 rounding of each product before the add
    (signrot/kernels/fused.cu:343-348).  q [B,T,Hq,D], k [B,T,Hk,D], cos/sin [B or 1, T, D]."""
    def one(x):
        d = x.shape[-1] // 2
        c, s = cos_h.unsqueeze(2), sin_h.unsqueeze(2)
        rot = torch.cat((-x[..., d:], x[..., :d]), dim=-1)
        return ((x.float() * c.float()).half().float() + (rot.float() * s.float()).half().float()).half()
    return one(q_h), one(k_h)


def swiglu(g_h, u_h):
    """rn_h(rn_h(g / (1 + exp(-g))) * u) (signrot/kernels/fused.cu:378-380)."""
    g = g_h.float()
    s = (g / (1.0 + torch.exp(-g))).half()
    return (s.float() * u_h.float()).half()
