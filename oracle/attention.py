"""Oracle: int4 paged KV cache and decode attention.  Test infrastructure only."""
from __future__ import annotations

import math

import torch

from .quant import kv_quant_pack, kv_dequant
from .hadamard import fwht

__all__ = ["PagedCacheRef", "decode_attention_ref", "had128"]


def had128(x_h: torch.Tensor) -> torch.Tensor:
    """Hadamard over head_dim in fp16 with scale 1/sqrt(n) given as a double
    (signrot/transformers/kv_cache.py:70-73)."""
    n = x_h.shape[-1]
    s = torch.tensor(1.0 / math.sqrt(n), dtype=torch.float32)
    return (fwht(x_h.float()) * s).half()


class PagedCacheRef:
    """Dense stand-in for the paged cache: keeps quantized K/V per (layer, request, head,
    position) and reproduces the paged layout of signrot/transformers/kv_cache.py:185-196,
    417-433 (physical page of (b, j) = j * batch + b) on request."""

    def __init__(self, batch, layers, heads, page_size, max_pages, hadamard=True):
        self.batch, self.layers, self.heads, self.page_size = batch, layers, heads, page_size
        self.hadamard = hadamard
        self.data = torch.zeros((max_pages * batch, layers, 2, heads, page_size, 64), dtype=torch.uint8)
        self.param = torch.zeros((max_pages * batch, layers, 2, heads, page_size, 2), dtype=torch.float16)
        self.length = [0] * layers

    def append(self, layer, k_h, v_h):
        """k_h, v_h fp16 [batch, T, heads, 128] (kv_cache.py:308-320)."""
        if self.hadamard:
            k_h = had128(k_h)
        kq, kp = kv_quant_pack(k_h)
        vq, vp = kv_quant_pack(v_h)
        T = k_h.shape[1]
        start = self.length[layer]
        page, slot, head = self._slots(start, T)
        self.data[page, layer, 0, head, slot] = kq
        self.data[page, layer, 1, head, slot] = vq
        self.param[page, layer, 0, head, slot] = kp
        self.param[page, layer, 1, head, slot] = vp
        self.length[layer] = start + T

    def _slots(self, start, count):
        """Index tensors (physical page [B, T, 1], slot [1, T, 1], head [1, 1, H]) of positions
        start .. start + count - 1 of every request."""
        pos = torch.arange(start, start + count)
        b = torch.arange(self.batch)
        page = ((pos // self.page_size)[None, :] * self.batch + b[:, None])[:, :, None]
        slot = (pos % self.page_size)[None, :, None]
        head = torch.arange(self.heads)[None, None, :]
        return page, slot, head

    def specs(self, layer):
        n = self.length[layer]
        pages = (n + self.page_size - 1) // self.page_size
        last = n % self.page_size
        if n != 0 and last == 0:
            last = self.page_size
        indptr = torch.arange(self.batch + 1, dtype=torch.int32) * pages
        idx = (torch.arange(pages, dtype=torch.int32) * self.batch).unsqueeze(0) + \
            torch.arange(self.batch, dtype=torch.int32).unsqueeze(1)
        return indptr, idx.reshape(-1).contiguous(), torch.full((self.batch,), last, dtype=torch.int32)

    def dense(self, layer):
        """Dequantized K, V as fp32 [batch, heads, length, 128]."""
        n = self.length[layer]
        page, slot, head = self._slots(0, n)
        k = kv_dequant(self.data[page, layer, 0, head, slot], self.param[page, layer, 0, head, slot])
        v = kv_dequant(self.data[page, layer, 1, head, slot], self.param[page, layer, 1, head, slot])
        return k.permute(0, 2, 1, 3).contiguous(), v.permute(0, 2, 1, 3).contiguous()


def decode_attention_ref(q_h: torch.Tensor, k_f: torch.Tensor, v_f: torch.Tensor, hadamard_q: bool = True):
    """fp32 softmax attention of one query per (request, q head) over the dequantized cache
    (benchmarks/test_split_decode.py:22-46; kernel arithmetic: include/flashinfer/decode.cuh:93-125,
    state.cuh:68-94).  q_h fp16 [B, Hq, 128]; k_f, v_f fp32 [B, Hkv, T, 128]; q head h reads KV
    head h // (Hq / Hkv).  Returns fp32 [B, Hq, 128]."""
    if hadamard_q:
        q_h = had128(q_h)
    B, Hq, D = q_h.shape
    g = Hq // k_f.shape[1]
    k = k_f.repeat_interleave(g, dim=1)
    v = v_f.repeat_interleave(g, dim=1)
    logits = torch.einsum("bhd,bhtd->bht", q_h.float(), k) / math.sqrt(D)
    p = torch.softmax(logits, dim=-1)
    return torch.einsum("bht,bhtd->bhd", p, v)
