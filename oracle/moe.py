"""Oracle: the sparse mixture-of-experts block.  Test infrastructure only."""
from __future__ import annotations

import torch

from . import quant as Q
from . import gemm as G
from . import hadamard as H
from . import misc as M

__all__ = ["moe_route", "moe_block"]


def moe_route(router_logits: torch.Tensor, top_k: int, norm_topk_prob: bool, dtype=torch.float16):
    """fp32 softmax -> top-k -> optional renormalisation -> cast, then the stable sort of the
    (token, choice) rows by expert (signrot/nn/moe.py:167-182).  Returns (routing weights
    [tokens, top_k] in `dtype`, selected experts [tokens, top_k], perm [rows], counts int32 [E])."""
    probs = torch.softmax(router_logits, dim=1, dtype=torch.float)
    weights, selected = torch.topk(probs, top_k, dim=-1)
    if norm_topk_prob:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    flat = selected.reshape(-1)
    perm = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=router_logits.shape[1]).to(torch.int32)
    return weights.to(dtype), selected, perm, counts


def moe_block(x_h, router_logits, top_k, norm_topk_prob, w_gate, s_gate, w_up, s_up, w_down, s_down,
              sign_down=None, hadK=None, K=1, clip: float = 1.0):
    """SignRotMoEBlock.forward, symmetric codes (signrot/nn/moe.py:160-236), through the integer
    oracle: one quantization per token shared by its experts and by gate/up, per-expert int4 GEMM +
    dequant (:138-157), SwiGLU, rotation of the routed rows, per-expert sign, quantizer, down GEMM,
    un-permute and `(y * w).sum(1)` in the activation dtype.  x_h fp16 [tokens, hidden];
    w_* packed uint8 [E, n, k/2]; s_* fp16 [E, n].  Returns fp16 [tokens, hidden]."""
    tokens, hidden = x_h.shape
    weights, selected, perm, counts = moe_route(router_logits, top_k, norm_topk_prob, x_h.dtype)
    tok = perm // top_k
    eid = selected.reshape(-1)[perm]
    codes, scale = Q.sym_quant_dynamic(x_h, clip)
    q_a, s_a = Q.pack_codes(codes)[tok], scale[tok]

    def per_expert(q, s, w, s_w):
        out = torch.empty((q.shape[0], w.shape[1]), dtype=torch.float16)
        row = 0
        for e, m in enumerate(counts.tolist()):
            if m:
                out[row:row + m] = G.w4a4_linear(q[row:row + m], s[row:row + m], w[e], s_w[e].view(-1, 1))
                row += m
        return out
    inter = M.swiglu(per_expert(q_a, s_a, w_gate, s_gate), per_expert(q_a, s_a, w_up, s_up))
    h = H.rotate(inter, hadK, K, None)
    if sign_down is not None:
        h = h * sign_down[eid].to(h.dtype)
    c2, s2 = Q.sym_quant_dynamic(h, clip)
    y = per_expert(Q.pack_codes(c2), s2, w_down, s_down)
    inv = torch.argsort(perm)
    y = y[inv].view(tokens, top_k, hidden)
    return (y * weights.unsqueeze(-1)).sum(dim=1)
