"""int4 paged KV cache with the interface of `signrot.transformers.kv_cache`
(signrot/transformers/kv_cache.py:12-521).

Layout (same as the reference): `pages` uint8 [pages, layers, 2, heads, page_size, head_dim/2],
`scales` fp16 [pages, layers, 2, heads, page_size, 2] = (scale, zero); the physical page of
(request b, logical page j) is j * batch_size + b.

What differs from the reference is how the work is done, not what is stored or returned:
  * `update` runs ONE kernel per layer that rotates K (Hadamard over head_dim), quantizes K
    and V and writes their page slots (the reference chains a Hadamard, two quantizers and an
    append/init kernel, kv_cache.py:308-415);
  * a GQA cache keeps its `num_heads` KV heads once; the decode kernel serves all the query
    heads of a group from one read (the reference repeats every KV head `group_size` times,
    kv_cache.py:346-353).  `group_size` is therefore only the q-per-kv ratio here.
"""
from __future__ import annotations

import functools
import os
import math
from typing import Any, Dict, Optional

import torch

from .. import _lib
from .._lib import ptr, require_cuda, run
from ..functional import kernel as _kernel
from ..functional.quantization import get_minq_maxq

import sys as _sys


class _PlainCache:
    def __init__(self, *a, **k):
        pass


def _hf_cache_base():
    """Hugging Face's `Cache` when the application has already imported transformers (so that
    `isinstance(cache, Cache)` checks in HF model code pass), else a plain base class.  The
    kernels never need transformers, and importing it here would cost seconds on every start."""
    mod = _sys.modules.get("transformers.cache_utils")
    if mod is None and "transformers" in _sys.modules:
        try:
            import importlib
            mod = importlib.import_module("transformers.cache_utils")
        except Exception:
            mod = None
    return getattr(mod, "Cache", _PlainCache) if mod is not None else _PlainCache


_HFCache = _hf_cache_base()


# ----------------------------------------------------------------------------- torch references

def asym_quantize_and_pack_i4(x, clip_factor_a_max=torch.tensor(1.0), clip_factor_a_min=torch.tensor(1.0),
                              lac: bool = False, quantize: bool = True):
    """Torch statement of the KV quantizer (kv_cache.py:12-58); the non-`lac` branch is what
    `kv_quant_pack` computes."""
    _, maxq = get_minq_maxq(bits=4, sym=False)
    xmax = torch.amax(x, dim=-1, keepdim=True)
    xmin = torch.amin(x, dim=-1, keepdim=True)
    if lac:
        zeros = torch.zeros_like(xmax)
        xmax, xmin = torch.maximum(xmax, zeros) * clip_factor_a_max, torch.minimum(xmin, zeros) * clip_factor_a_min
        both_zero = (xmin == 0) & (xmax == 0)
        xmin = torch.where(both_zero, torch.full_like(xmin, -1.0), xmin)
        xmax = torch.where(both_zero, torch.full_like(xmax, 1.0), xmax)
        scale = (xmax - xmin) / maxq
        zero = torch.round((-1.0 * xmin) / scale)
        q = torch.clamp((x / scale).round() + zero, 0, maxq)
    else:
        scale = (xmax - xmin).clamp(min=1e-5) / maxq
        zero = -xmin
        q = torch.clamp(torch.round((x + zero) / scale), 0, maxq)
    if not quantize:
        return scale * (q - zero), scale, zero
    q = q.to(dtype=torch.uint8)
    return q[..., 0::2] | (q[..., 1::2] << 4), scale, zero


def unpack_i4_and_asym_dequantize(q, scale, zero, lac: bool = False):
    assert q.dtype == torch.uint8
    q = torch.stack((q & 0x0F, (q >> 4) & 0x0F), dim=-1).view(*q.shape[:-1], q.shape[-1] * 2)
    return scale * (q - zero) if lac else q * scale - zero


def matmul_had_cuda(X, dtype):
    """Hadamard over the last dimension in `dtype`, cast back (kv_cache.py:70-73)."""
    n = X.shape[-1]
    y = _kernel.hadamard(X.to(dtype), None, 1, scale=float(1 / math.sqrt(n)))
    return y.to(X.dtype).view(X.shape)


# ----------------------------------------------------------------------------- kernel wrappers

def _geometry(kv_data):
    if kv_data.dim() != 6:
        raise RuntimeError("kv_data must be a 6D tensor")
    return kv_data.size(1), kv_data.size(3), kv_data.size(4), kv_data.size(5) * 2


def init_kv_i4(kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, k, v, k_param, v_param,
               seqlen_indptr, layer_idx):
    """Scatter a whole quantized prompt per request into its pages (kv_cache.py:76-86)."""
    dev = require_cuda("init_kv_i4", kv_data, kv_indptr, kv_indices, last_page_offset, k, v, seqlen_indptr)
    L, H, P, D = _geometry(kv_data)
    batch = last_page_offset.size(0)
    if kv_indptr.size(0) != batch + 1 or seqlen_indptr.size(0) != batch + 1:
        raise RuntimeError("CHECK_EQ(kv_indptr.size(0), batch_size + 1) failed.")
    run(dev, "sr_init_kv_i4", ptr(kv_data), ptr(kv_param), ptr(kv_indptr), ptr(kv_indices), ptr(last_page_offset),
        ptr(k), ptr(v), ptr(k_param.contiguous()), ptr(v_param.contiguous()), ptr(seqlen_indptr), k.size(0), L,
        int(layer_idx), H, P, D, batch)


def append_kv_i4(kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, k, v, k_param, v_param, layer_idx):
    """Write one quantized token per request into its slot (kv_cache.py:89-99)."""
    dev = require_cuda("append_kv_i4", kv_data, kv_indptr, kv_indices, last_page_offset, k, v)
    L, H, P, D = _geometry(kv_data)
    batch = k.size(0)
    if kv_indptr.size(0) != batch + 1 or last_page_offset.size(0) != batch:
        raise RuntimeError("CHECK_EQ(kv_indptr.size(0), batch_size + 1) failed.")
    run(dev, "sr_append_kv_i4", ptr(kv_data), ptr(kv_param), ptr(kv_indptr), ptr(kv_indices), ptr(last_page_offset),
        ptr(k), ptr(v), ptr(k_param.contiguous()), ptr(v_param.contiguous()), L, int(layer_idx), H, P, D, batch)


def batch_decode_i4(o, q, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, layer_idx, tmp=None,
                    num_chunks=1, hadamard_q=False, counters=None):
    """Decode attention of one new token per request over the int4 cache (kv_cache.py:101-107).
    o, q: fp16 [batch, q_heads, 128]; q_heads may be a multiple of the cache's head count.
    `counters` (int32 [batch * kv_heads], zero): the split-KV merge runs inside the attention kernel
    instead of as a second launch; the kernel leaves the counters zero."""
    dev = require_cuda("batch_decode_i4", o, q, kv_data, kv_indptr, kv_indices, last_page_offset, tmp, counters)
    if o.dim() != 3 or q.dim() != 3 or o.shape != q.shape:
        raise RuntimeError("o and q must be [B, N, D] tensors of the same shape")
    if kv_data.dtype != torch.uint8 or kv_param.dtype != torch.float16:
        raise RuntimeError("kv_data must be uint8 and kv_param fp16")
    L, H, P, D = _geometry(kv_data)
    batch, hq = o.size(0), o.size(1)
    if kv_indptr.size(0) != batch + 1 or last_page_offset.size(0) != batch:
        raise RuntimeError("CHECK_EQ(kv_indptr.size(0), batch_size + 1) failed.")
    if tmp is not None and num_chunks > 1:
        if tmp.dtype != torch.float32 or tmp.numel() != batch * hq * num_chunks * (D + 4):
            raise RuntimeError("tmp must be fp32 [batch, heads, chunks, head_dim + 4]")
    else:
        tmp, num_chunks = None, 1
    if counters is not None and num_chunks > 1:
        if counters.dtype != torch.int32 or counters.numel() < batch * H:
            raise RuntimeError("counters must be int32 [batch * kv_heads]")
        run(dev, "sr_batch_decode_i4_merged", ptr(o), ptr(q), ptr(kv_data), ptr(kv_param), ptr(kv_indptr),
            ptr(kv_indices), ptr(last_page_offset), L, int(layer_idx), hq, H, P, D, batch, ptr(tmp), int(num_chunks),
            ptr(counters), int(bool(hadamard_q)))
        return
    run(dev, "sr_batch_decode_i4", ptr(o), ptr(q), ptr(kv_data), ptr(kv_param), ptr(kv_indptr), ptr(kv_indices),
        ptr(last_page_offset), L, int(layer_idx), hq, H, P, D, batch, ptr(tmp), int(num_chunks), int(bool(hadamard_q)))


def kv_append_quant(kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, k, v, layer_idx, hadamard_k=True):
    """k, v fp16 [batch, new_tokens, heads, 128] -> rotate K, quantize both, write the slots of
    the last `new_tokens` positions of every request."""
    dev = require_cuda("kv_append_quant", kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, k, v)
    L, H, P, D = _geometry(kv_data)
    if k.dtype != torch.float16 or v.dtype != torch.float16 or k.shape != v.shape or k.dim() != 4:
        raise RuntimeError("kv_append_quant expects fp16 [B, T, H, D] k and v of the same shape")
    if k.size(2) != H or k.size(3) != D:
        raise RuntimeError("kv_append_quant: k/v heads or head_dim do not match the cache")
    run(dev, "sr_kv_append_quant", ptr(kv_data), ptr(kv_param), ptr(kv_indptr), ptr(kv_indices),
        ptr(last_page_offset), ptr(k), ptr(v), k.size(0), k.size(1), L, int(layer_idx), H, P, D,
        int(bool(hadamard_k)))


def _token_stride(name, t, heads, D):
    """Element stride between consecutive tokens of a [B, T, H, D] tensor whose heads are dense
    (it may be a column range of a wider projection output)."""
    if t.dtype != torch.float16 or t.dim() != 4 or t.size(2) != heads or t.size(3) != D:
        raise RuntimeError(f"rope_kv_append expects fp16 [B, T, {heads}, {D}] {name}")
    B, T = t.size(0), t.size(1)
    # the stride of a size-1 dimension carries no information
    stride = t.stride(1) if T > 1 else (t.stride(0) if B > 1 else heads * D)
    if t.stride(3) != 1 or (heads > 1 and t.stride(2) != D) or (B > 1 and T > 1 and t.stride(0) != T * stride):
        raise RuntimeError(f"rope_kv_append: {name} must have dense heads and a uniform token stride")
    return stride


def rope_kv_append(kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, q, k, v, cos, sin, layer_idx,
                   hadamard_k=True, want_k=False):
    """Rotary embedding on q and k, then the fused K/V append, in one launch.  q/k/v fp16
    [B, T, H, D], possibly column ranges of one fused projection output; cos/sin fp16
    [1 or B, T, D].  Returns (rotated q, contiguous; rotated k or None)."""
    dev = require_cuda("rope_kv_append", kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, q, k, v, cos, sin,
                       strided=(q, k, v))
    L, H, P, D = _geometry(kv_data)
    B, T, hq = q.size(0), q.size(1), q.size(2)
    qs, ks, vs = _token_stride("q", q, hq, D), _token_stride("k", k, H, D), _token_stride("v", v, H, D)
    if k.shape[:2] != (B, T) or v.shape[:2] != (B, T):
        raise RuntimeError("rope_kv_append: q, k and v must agree on batch and sequence")
    cos, sin = cos.contiguous(), sin.contiguous()
    if cos.dtype != torch.float16 or cos.shape != sin.shape or cos.dim() != 3 or cos.size(1) != T or cos.size(2) != D \
            or cos.size(0) not in (1, B):
        raise RuntimeError("rope_kv_append expects fp16 cos/sin of shape [1 or B, T, head_dim]")
    q_out = torch.empty((B, T, hq, D), dtype=torch.float16, device=dev)
    k_out = torch.empty((B, T, H, D), dtype=torch.float16, device=dev) if want_k else None
    run(dev, "sr_rope_kv_append", ptr(kv_data), ptr(kv_param), ptr(kv_indptr), ptr(kv_indices), ptr(last_page_offset),
        ptr(q), ptr(k), ptr(v), qs, ks, vs, ptr(cos), ptr(sin), cos.size(0), ptr(q_out), ptr(k_out), B, T, L,
        int(layer_idx), hq, H, P, D, int(bool(hadamard_k)))
    return q_out, k_out


def rope_decode_i4(o, q, k, v, cos, sin, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, layer_idx, tmp=None,
                   num_chunks=1, hadamard_q=False, hadamard_k=True):
    """`rope_kv_append` for one new token per request and `batch_decode_i4` in one launch, with the bits of the
    two calls.  q [B, 1, Hq, D], k / v [B, 1, H, D] fp16 before the rotary embedding (column ranges of a fused
    projection are fine); cos / sin fp16 [1 or B, 1, D]; o fp16 [B, Hq, D].  The page tables already count the new
    token.  Needs page_size % 16 == 0."""
    dev = require_cuda("rope_decode_i4", o, kv_data, kv_param, kv_indptr, kv_indices, last_page_offset, q, k, v, cos, sin,
                       tmp, strided=(q, k, v))
    L, H, P, D = _geometry(kv_data)
    B, hq = q.size(0), q.size(2)
    if q.size(1) != 1 or k.shape[:2] != (B, 1) or v.shape[:2] != (B, 1):
        raise RuntimeError("rope_decode_i4: one new token per request")
    qs, ks, vs = _token_stride("q", q, hq, D), _token_stride("k", k, H, D), _token_stride("v", v, H, D)
    cos, sin = cos.contiguous(), sin.contiguous()
    if cos.dtype != torch.float16 or cos.shape != sin.shape or cos.dim() != 3 or cos.size(1) != 1 or cos.size(2) != D \
            or cos.size(0) not in (1, B):
        raise RuntimeError("rope_decode_i4 expects fp16 cos/sin of shape [1 or B, 1, head_dim]")
    if o.shape != (B, hq, D) or o.dtype != torch.float16 or not o.is_contiguous():
        raise RuntimeError("rope_decode_i4: o must be a contiguous fp16 [B, q_heads, head_dim] tensor")
    if tmp is not None and num_chunks > 1:
        if tmp.dtype != torch.float32 or tmp.numel() != B * hq * num_chunks * (D + 4):
            raise RuntimeError("tmp must be fp32 [batch, heads, chunks, head_dim + 4]")
    else:
        tmp, num_chunks = None, 1
    run(dev, "sr_rope_decode_i4", ptr(o), ptr(q), ptr(k), ptr(v), qs, ks, vs, ptr(cos), ptr(sin), cos.size(0),
        ptr(kv_data), ptr(kv_param), ptr(kv_indptr), ptr(kv_indices), ptr(last_page_offset), L, int(layer_idx), hq, H, P, D,
        B, ptr(tmp), int(num_chunks), int(bool(hadamard_q)), int(bool(hadamard_k)))


# ----------------------------------------------------------------------------- cache object

class _AttentionStub:
    """Decode-time attention over the cache; returned (bound) by `update` (kv_cache.py:144-170)."""

    def __init__(self, hadamard_dtype):
        self.hadamard_dtype = hadamard_dtype
        self.num_chunks = 1
        self.tmp = None
        self.counters = None     # arrival counters of the in-kernel split-KV merge (zero between calls)

    def forward(self, q, num_kv_heads, attention_kwargs, layer_idx):
        bsz, q_len, hq, hd = q.shape
        assert q_len == 1
        q = q.reshape(bsz, hq, hd)
        if q.dtype != torch.float16:
            q = q.to(torch.float16)
        q = q.contiguous()
        out = torch.empty_like(q)
        # the Hadamard on q (kv_cache.py:157-158) is applied inside the decode kernel
        batch_decode_i4(out, q, **attention_kwargs, layer_idx=layer_idx, tmp=self.tmp, num_chunks=self.num_chunks,
                        hadamard_q=self.hadamard_dtype is not None, counters=self.counters)
        return out.unsqueeze(1)

    def forward_rope(self, q, k, v, cos, sin, attention_kwargs, layer_idx, hadamard_k):
        """The decode step's attention from the projections before the rotary embedding: rotary embedding, K/V
        append and attention in one launch (`rope_decode_i4`)."""
        bsz, q_len, hq, hd = q.shape
        assert q_len == 1
        out = torch.empty((bsz, hq, hd), dtype=torch.float16, device=q.device)
        rope_decode_i4(out, q, k, v, cos, sin, **attention_kwargs, layer_idx=layer_idx, tmp=self.tmp,
                       num_chunks=self.num_chunks, hadamard_q=self.hadamard_dtype is not None, hadamard_k=hadamard_k)
        return out.unsqueeze(1)


def decode_split(batch_size, kv_heads, max_pages, device):
    """Chunks per (request, KV head) of the split-KV decode: about two CTAs per SM, at most one per page
    (the kernel shares a request's 16-token blocks out evenly, whatever the count)."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    per_sm = int(os.environ.get("SIGNROT_B200_DECODE_CTAS_PER_SM", "2"))
    chunks = max(1, per_sm * sms // (batch_size * kv_heads))     # two 8-warp CTAs fit an SM: no second wave
    if chunks < 8:
        # 2 or 4 chunks merge inside a thread-block cluster (no second launch); other cluster sizes are slow to place
        chunks = 1 << (chunks.bit_length() - 1)
    return min(chunks, max(1, max_pages))


class MultiLayerPagedKVCache4Bit(_HFCache):
    def __init__(self, batch_size, page_size, max_seq_len, device, n_layers, num_heads, head_dim,
                 disable_quant=False, hadamard_dtype=torch.float16, group_size=1, lac=False, decode_chunks=None):
        self.decode_chunks = decode_chunks
        self.fuse_decode = True      # decode steps: rotary embedding + K/V append + attention in one launch (same bits as two)
        if disable_quant:
            raise NotImplementedError("the unquantized fp16 cache (a baseline knob of the reference) is not built")
        if lac:
            raise NotImplementedError("learned activation clipping is unused in the reference and not built")
        if head_dim != 128:
            raise RuntimeError(f"CHECK_EQ(head_dim, 128) failed. {head_dim} vs 128")
        self.lac = lac
        self.disable_quant = False
        self.page_size = page_size
        self.batch_size = batch_size
        self.max_seq_len = max_seq_len
        self.device = torch.device(device)
        self.hadamard_dtype = hadamard_dtype
        self.group_size = group_size
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.length = 0
        max_pages = self.page_cnt_from_length(max_seq_len)
        self.pages = torch.empty((max_pages * batch_size, n_layers, 2, num_heads, page_size, head_dim // 2),
                                 dtype=torch.uint8, device=device)
        self.scales = torch.empty((max_pages * batch_size, n_layers, 2, num_heads, page_size, 2),
                                  dtype=torch.float16, device=device)
        self._needs_init = [True] * n_layers
        self._stub = _AttentionStub(hadamard_dtype)

        # index tensors: allocated once, refreshed in place, so addresses captured by a CUDA
        # graph stay valid for the whole decode
        self._kv_indices_full = torch.empty(self.pages.shape[0], device=device, dtype=torch.int32)
        self._spec_page_cnt = None
        self._last_page_offset = torch.empty(batch_size, device=device, dtype=torch.int32)
        self._indptr_base = torch.arange(batch_size + 1, device=device, dtype=torch.int32)
        self._kv_indptr_buf = torch.empty(batch_size + 1, device=device, dtype=torch.int32)
        self._specs_frozen = False
        self._spec_cache = {"kv_data": self.pages, "kv_param": self.scales, "kv_indptr": self._kv_indptr_buf,
                            "kv_indices": self._kv_indices_full, "last_page_offset": self._last_page_offset}
        self._configure_decode_split(max_pages)

    def _configure_decode_split(self, max_pages):
        """Fixed number of sequence chunks per (request, KV head) so that about two CTAs per SM
        are in flight; bounded by the page count (a chunk is an equal share of the request's 16-token blocks; a page range in the
        CUDA-core kernel that takes page sizes which are not multiples of 16).  `decode_chunks`
        pins the number (a tensor-parallel shard uses the split of the unsharded head count, so
        that its fp32 merge order, and with it every output bit, is that of one GPU)."""
        if self.decode_chunks is not None:
            chunks = max(1, min(int(self.decode_chunks), max(1, max_pages)))
        else:
            chunks = decode_split(self.batch_size, self.num_heads, max_pages, self.device)
        self._stub.num_chunks = chunks
        if chunks > 1:
            self._stub.tmp = torch.empty((self.batch_size, self.num_heads * self.group_size, chunks,
                                          self.head_dim + 4), dtype=torch.float32, device=self.device)
            # measured on B200 (batch 8, context 2100): the counter-based in-kernel merge costs 5 us per layer
            # more than the separate merge launch (one CTA merges four heads one after the other behind
            # device-wide fences), so it is opt-in
            if os.environ.get("SIGNROT_B200_DECODE_MERGE", "separate") == "fused":
                self._stub.counters = torch.zeros(self.batch_size * self.num_heads, dtype=torch.int32,
                                                  device=self.device)

    def page_cnt_from_length(self, length):
        return (length + self.page_size - 1) // self.page_size

    def _ensure_page_cnt_per_batch(self, pages_per_request):
        need = pages_per_request * self.batch_size
        have = self.pages.shape[0]
        if need <= have:
            return
        # a pool that grows re-lays every request's pages (physical page = j * batch + b needs no
        # move: new pages get higher j), but the tensors move, so captured graphs become invalid
        grow_to = max(need, have * 2)
        extra = grow_to - have
        self.pages = torch.cat([self.pages, torch.empty((extra, *self.pages.shape[1:]), dtype=self.pages.dtype,
                                                        device=self.device)], dim=0)
        self.scales = torch.cat([self.scales, torch.empty((extra, *self.scales.shape[1:]), dtype=self.scales.dtype,
                                                          device=self.device)], dim=0)
        self._kv_indices_full = torch.empty(self.pages.shape[0], device=self.device, dtype=torch.int32)
        self._spec_page_cnt = None
        self._spec_cache.update(kv_data=self.pages, kv_param=self.scales, kv_indices=self._kv_indices_full)

    @property
    def seen_tokens(self):
        return self.length

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs: Optional[Dict[str, Any]] = None):
        """key/value_states [B, T, kv_heads, 128].  Prefill (first call per layer) returns the
        original K/V for the caller's dense attention; decode returns a callable that attends a
        query [B, 1, q_heads, 128] to the cache (kv_cache.py:295-415)."""
        bsz, added, heads, hd = key_states.shape
        cache_kwargs = cache_kwargs or {}
        if cache_kwargs.get("attention_mask") is not None:
            raise NotImplementedError("padded (masked) prefill is not supported by the fused append")
        specs, first = self._advance(bsz, added, layer_idx)
        k16 = key_states if key_states.dtype == torch.float16 else key_states.to(torch.float16)
        v16 = value_states if value_states.dtype == torch.float16 else value_states.to(torch.float16)
        kv_append_quant(**specs, k=k16.contiguous(), v=v16.contiguous(), layer_idx=layer_idx,
                        hadamard_k=self.hadamard_dtype is not None)
        if first:
            return key_states, value_states
        return functools.partial(self._stub.forward, num_kv_heads=heads, attention_kwargs=specs,
                                 layer_idx=layer_idx)

    def _advance(self, bsz, added, layer_idx):
        """Host-side bookkeeping of one `update`: length, pages, index tensors, first-call flag."""
        assert bsz == self.batch_size
        if layer_idx == 0:
            new_len = self.length + added
            self._ensure_page_cnt_per_batch(self.page_cnt_from_length(new_len))
            self.length = new_len
        specs = self.get_cache_specs_for_flash_infer(None)
        first = self._needs_init[layer_idx]
        if first:
            self._needs_init[layer_idx] = False
        else:
            assert added == 1
        return specs, first

    def update_with_rope(self, query_states, key_states, value_states, cos, sin, layer_idx: int, defer_append=False):
        """`rope_qk` + `update` in one launch (kernel_utils.py:118-141 of the reference's glue calls
        them back to back).  q/k/v are the projections BEFORE the rotary embedding, fp16
        [B, T, H, 128], possibly column ranges of one fused projection.  Returns
        (rotated q, what `update` returns: (rotated k, v) on the first call of a layer, the
        attention callable afterwards).

        `defer_append`: the caller promises to call the returned attention callable, with the returned q, before
        anything else touches the cache.  A decode step then runs as ONE launch (`rope_decode_i4`): the callable
        rotates q, appends the new K / V and attends; the q handed back is the unrotated one."""
        bsz, added, heads, hd = key_states.shape
        specs, first = self._advance(bsz, added, layer_idx)
        if (defer_append and not first and added == 1 and self.page_size % 16 == 0 and self._stub.counters is None
                and query_states.dtype == torch.float16 and self.fuse_decode):
            # decode: the attention kernel rotates q, appends the new K / V and attends in one launch; the caller hands
            # the returned q (unrotated) to the returned callable
            return query_states, functools.partial(self._stub.forward_rope, k=key_states, v=value_states, cos=cos, sin=sin,
                                                   attention_kwargs=specs, layer_idx=layer_idx,
                                                   hadamard_k=self.hadamard_dtype is not None)
        q_rot, k_rot = rope_kv_append(**specs, q=query_states, k=key_states, v=value_states, cos=cos, sin=sin,
                                      layer_idx=layer_idx, hadamard_k=self.hadamard_dtype is not None, want_k=first)
        if first:
            return q_rot, (k_rot, value_states)
        return q_rot, functools.partial(self._stub.forward, num_kv_heads=heads, attention_kwargs=specs,
                                        layer_idx=layer_idx)

    def _set_page_cnt(self, page_cnt: int):
        torch.mul(self._indptr_base, page_cnt, out=self._kv_indptr_buf)
        if self._spec_page_cnt == page_cnt:
            return
        self._spec_page_cnt = page_cnt
        j = torch.arange(page_cnt, device=self.device, dtype=torch.int32) * self.batch_size
        b = torch.arange(self.batch_size, device=self.device, dtype=torch.int32)
        self._kv_indices_full[: page_cnt * self.batch_size].copy_((j.unsqueeze(0) + b.unsqueeze(1)).reshape(-1))

    def refresh_specs(self, length: int | None = None):
        """Rewrites the index tensors for a uniform-length batch from the host-side length: two
        small in-place writes, no device->host sync.  A CUDA-graph runner calls this between
        replays (the graph itself must not contain these writes)."""
        if length is None:
            length = self.length
        page_cnt = self.page_cnt_from_length(length)
        last = length % self.page_size
        if length != 0 and last == 0:
            last = self.page_size
        self._last_page_offset.fill_(last)
        self._set_page_cnt(page_cnt)
        return self._spec_cache

    def device_step_state(self):
        """Device-resident (token count int32 [1], position int64 [1]) of the decode step, for a captured
        graph whose first node is `advance_on_device`.  Created on first use; the count is set from the
        host-side length by `sync_device_length`."""
        if getattr(self, "_len_dev", None) is None:
            self._len_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._pos_dev = torch.zeros(1, dtype=torch.int64, device=self.device)
        return self._len_dev, self._pos_dev

    def sync_device_length(self):
        self.device_step_state()[0].fill_(self.length)

    def advance_on_device(self):
        """One launch: position of the token about to be appended and the page tables of the sequence that
        includes it, from the device-resident count, which it then increments (the device twin of
        `refresh_specs(length + 1)`; capturable).  Returns the position tensor."""
        length, position = self.device_step_state()
        _lib.run(self.device, "sr_decode_advance", _lib.ptr(length), _lib.ptr(position), _lib.ptr(self._kv_indptr_buf),
                 _lib.ptr(self._kv_indices_full), _lib.ptr(self._last_page_offset), self.batch_size, self.page_size,
                 self.pages.shape[0] // self.batch_size)
        self._spec_page_cnt = None      # the host-side copy of the page count is stale now
        return position

    def capacity(self) -> int:
        """Tokens per request the allocated pages hold."""
        return (self.pages.shape[0] // self.batch_size) * self.page_size

    def freeze_specs(self, frozen=True):
        """While frozen, `update` does not touch the index tensors (graph capture/replay)."""
        self._specs_frozen = frozen

    def get_cache_specs_for_flash_infer(self, attention_mask):
        if attention_mask is not None:
            raise NotImplementedError("padded (masked) prefill is not supported")
        return self._spec_cache if self._specs_frozen else self.refresh_specs()

    def reset(self):
        """Rewind to empty without reallocating; captured graphs stay valid."""
        self.length = 0
        self._needs_init = [True] * len(self._needs_init)

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return self.length

    def get_max_length(self) -> Optional[int]:
        return None

    def to_legacy_cache(self):
        return self


class HFCacheAdapter(_HFCache):
    """Thin adapter that lets HF model code drive the paged cache (kv_cache.py:500-521)."""

    def __init__(self, inner):
        try:
            super().__init__()
        except Exception:
            pass
        self.inner = inner

    def get_usable_length(self, kv_seq_len: int, layer_idx: int) -> int:
        return self.inner.get_usable_length(kv_seq_len, layer_idx)

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        return self.inner.get_seq_length()

    def get_max_length(self):
        return self.inner.get_max_length()

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs=None):
        return self.inner.update(key_states, value_states, layer_idx, cache_kwargs)

    def to_legacy_cache(self):
        if hasattr(self.inner, "to_legacy_cache"):
            return self.inner.to_legacy_cache()
        return self
