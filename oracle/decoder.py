"""Oracle: a Llama-shaped decoder stack over the integer path, prefill then decode steps, on the CPU.
Test infrastructure only.

Follows the reference's kernel-mode model: `kernel_attention_forward` and `kernel_mlp_forward`
(fake_quant/kernel_utils.py:86-161, 352-363) over `ActQuantWrapper.kernel_quantize/kernel_matmul`
(fake_quant/quant_utils.py:278-296), the paged int4 cache's `update` (signrot/transformers/
kv_cache.py:295-415: Hadamard(128) on K, `kv_quant_pack` on K and V, original fp16 K/V handed to
the dense prefill attention) and its decode stub (`:153-170`: Hadamard on q, attention over the
dequantized cache).  Every operator is the restatement kept in this package."""
from __future__ import annotations

import torch

from . import quant as Q
from . import gemm as G
from . import hadamard as H
from . import misc as M
from .attention import PagedCacheRef, decode_attention_ref

__all__ = ["DecoderRef"]


class DecoderRef:
    """`state` holds CPU tensors:
      embed [V, hid] fp16, lm_head [V, hid] fp16, layers: list of dicts with packed weights
      `wq wk wv wo wg wu wd` (uint8 [N, K/2]), scales `sq ... sd` (fp16 [N, 1]) and `sign_d`
      (int8 [ffn] or None).
    `cfg`: hidden, heads, kv_heads, head_dim, ffn, eps, theta, hadK (ffn's Kronecker factor or
    None), K."""

    def __init__(self, state, cfg, batch, page_size, max_len):
        self.s, self.c = state, cfg
        self.batch = batch
        pages = (max_len + page_size - 1) // page_size
        self.cache = PagedCacheRef(batch, len(state["layers"]), cfg["kv_heads"], page_size, pages, hadamard=True)
        self.length = 0

    @staticmethod
    def _linear(x_h, w, s):
        rows = x_h.reshape(-1, x_h.shape[-1])
        codes, sc = Q.sym_quant_dynamic(rows, 1.0)
        out = G.w4a4_linear(Q.pack_codes(codes), sc, w, s)
        return out.reshape(*x_h.shape[:-1], -1)

    def _rotary(self, start, t):
        d, theta = self.c["head_dim"], self.c["theta"]
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        ang = torch.arange(start, start + t, dtype=torch.float32)[:, None] * inv[None, :]
        emb = torch.cat((ang, ang), dim=-1)
        return emb.cos().half()[None], emb.sin().half()[None]

    def forward(self, input_ids):
        """input_ids int64 [B, T]: T > 1 is the prefill (empty cache), T == 1 a decode step.
        Returns fp16 logits [B, T, V]."""
        c = self.c
        B, T = input_ids.shape
        Hq, Hk, D = c["heads"], c["kv_heads"], c["head_dim"]
        prefill = self.length == 0
        cos, sin = self._rotary(self.length, T)
        x = self.s["embed"][input_ids]                                # [B, T, hid] fp16
        for li, L in enumerate(self.s["layers"]):
            h = M.rmsnorm(x, c["eps"], c["hidden"])
            rows = h.reshape(-1, c["hidden"])
            codes, sc = Q.sym_quant_dynamic(rows, 1.0)                # one quantization for q/k/v
            pk = Q.pack_codes(codes)
            q = G.w4a4_linear(pk, sc, L["wq"], L["sq"]).reshape(B, T, Hq, D)
            k = G.w4a4_linear(pk, sc, L["wk"], L["sk"]).reshape(B, T, Hk, D)
            v = G.w4a4_linear(pk, sc, L["wv"], L["sv"]).reshape(B, T, Hk, D)
            q, k = M.rope_qk(q, k, cos, sin)
            self.cache.append(li, k, v)
            if prefill:
                g = Hq // Hk
                attn = torch.nn.functional.scaled_dot_product_attention(
                    q.transpose(1, 2).float(), k.transpose(1, 2).repeat_interleave(g, dim=1).float(),
                    v.transpose(1, 2).repeat_interleave(g, dim=1).float(), is_causal=True)
                attn = attn.transpose(1, 2).reshape(B, T, Hq * D).half()
            else:
                kf, vf = self.cache.dense(li)
                attn = decode_attention_ref(q.reshape(B, Hq, D), kf, vf, hadamard_q=True).half().reshape(B, 1, Hq * D)
            o = self._linear(H.rotate_heads(attn, Hq), L["wo"], L["so"])
            x = x + o
            h2 = M.rmsnorm(x, c["eps"], c["hidden"])
            rows = h2.reshape(-1, c["hidden"])
            codes, sc = Q.sym_quant_dynamic(rows, 1.0)                # one quantization for gate/up
            pk = Q.pack_codes(codes)
            gate = G.w4a4_linear(pk, sc, L["wg"], L["sg"])
            up = G.w4a4_linear(pk, sc, L["wu"], L["su"])
            m = M.swiglu(gate, up)
            m = H.rotate(m, c["hadK"], c["K"], L["sign_d"])
            x = x + self._linear(m, L["wd"], L["sd"]).reshape(B, T, c["hidden"])
        self.length += T
        hn = M.rmsnorm(x, c["eps"], c["hidden"])
        return (hn.float() @ self.s["lm_head"].float().T).half()
