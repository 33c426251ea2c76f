"""Decode-graph glue around the quantized-linear path: the kernel branch of the activation-quantized
linear wrapper, attention and MLP forwards that share one quantization between sibling
projections, a Llama-shaped decoder stack over those pieces, and a CUDA-graph runner for the decode
step.

Reference counterparts:
  * `KernelLinear`             `ActQuantWrapper.enable_kernel / kernel_quantize / kernel_matmul /
                               shares_kernel_input_with` (fake_quant/quant_utils.py:214-314)
  * `kernel_attention_forward` fake_quant/kernel_utils.py:86-161
  * `kernel_mlp_forward`       fake_quant/kernel_utils.py:352-363
  * `build_paged_cache`        fake_quant/kernel_utils.py:64-83
  * `GraphedDecoder`, `try_graph_decoder`   fake_quant/kernel_utils.py:164-292 (same job, different mechanism:
                               the per-step bookkeeping is a device node of the graph)

The reference patches these functions onto a Hugging Face model.  Here the same functions drive a
small self-contained decoder (`KernelDecoderModel`: embedding, N decoder layers, final norm, fp16
lm_head) so that the path can be run and measured without model files; a Hugging Face layer whose
projections are `KernelLinear` objects can be driven by the same two forwards.

What differs from the reference by design:
  * a projection with an online rotation quantizes through ONE launch (`kernel.rotate_quant`:
    rotation, +-1 sign, per-token scale, int4 codes) instead of Hadamard kernel(s) + quantizer;
  * the cache takes K/V straight from the projections (`update` runs the fused
    Hadamard + quantize + page-scatter kernel) and attends grouped-query heads without repeating
    the cached heads;
  * prefill attention (dense, fp16, outside the path) is `scaled_dot_product_attention`.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass

import torch

from .. import nn as snn
from ..functional import kernel
from .kv_cache import MultiLayerPagedKVCache4Bit

# the cache allocates whole pages; a small page also gives the decode kernel several pages per
# sequence to split its work across (fake_quant/kernel_utils.py:57-61)
DEFAULT_PAGE_SIZE = 256


# ----------------------------------------------------------------------------- linear wrapper

class KernelLinear(torch.nn.Module):
    """Online rotation (optional) -> activation quantizer -> int4 linear.

    `online_full_had`: Hadamard over the whole input (down_proj), with the optional +-1
    `had_adj_sign` of the SignRot adjustment.  `online_partial_had`: Hadamard across heads,
    identity within a head (o_proj); `had_dim` is the head size as in the reference."""

    def __init__(self, in_features, out_features, *, bias=False, online_full_had=False, online_partial_had=False,
                 had_dim=0, had_adj=False, fp32_had=False, asym=False, clip_ratio=1.0):
        super().__init__()
        assert not (online_full_had and online_partial_had)
        assert not had_adj or online_full_had, "had_adj is only supported on online_full_had layers"
        self.online_full_had = online_full_had
        self.online_partial_had = online_partial_had
        self.had_dim = had_dim
        self.fp32_had = fp32_had
        self.use_kernel = True
        self.kernel_hadamard = None
        if online_full_had:
            self.kernel_hadamard = snn.OnlineHadamard(in_features, force_fp32=fp32_had, had_adj=had_adj)
        elif online_partial_had:
            assert had_dim > 0 and in_features % had_dim == 0
            self.kernel_hadamard = snn.OnlineHadamard(in_features // had_dim, force_fp32=fp32_had)
        self.kernel_quantizer = (snn.AsymQuantizer if asym else snn.Quantizer)(clip_ratio=clip_ratio)
        self.kernel_module = snn.Linear4bit(in_features, out_features, bias=bias)

    @property
    def in_features(self):
        return self.kernel_module.in_features

    @property
    def out_features(self):
        return self.kernel_module.out_features

    @property
    def _asym(self):
        return isinstance(self.kernel_quantizer, snn.AsymQuantizer)

    def kernel_quantize(self, x) -> kernel.PackedQuantizedTensor:
        """Rotation (+ sign) and activation quantization only, so that siblings reading the same
        activation can share it."""
        had = self.kernel_hadamard
        if had is None:
            return self.kernel_quantizer(x if x.dtype == torch.float16 else x.to(torch.float16))
        if self.fp32_had:
            # fp32 rotation keeps the reference's operator chain (one rounding after the transform)
            x = x.to(torch.float16)
            if self.online_full_had:
                x = had(x)
            else:
                x = kernel.hadamard_heads(x, x.shape[-1] // self.had_dim, fp32_mode=True)
            return self.kernel_quantizer(x)
        if x.dtype not in (torch.float16, torch.bfloat16):
            x = x.to(torch.float16)
        clip = self.kernel_quantizer.clip_ratio
        if self.online_full_had:
            sign = had.had_adj_sign
            if sign is not None and not had._had_adj_ready_cached:
                raise RuntimeError("Dynamic hadamard adjustment not implemented yet.")
            return kernel.rotate_quant(x, had.had_rem_dim, had.rem_dim, sign=sign, clip_ratio=clip, asym=self._asym)
        return kernel.rotate_quant(x, heads=x.shape[-1] // self.had_dim, clip_ratio=clip, asym=self._asym)

    def kernel_matmul(self, packed_x, x_dtype):
        out = self.kernel_module(packed_x)
        return out if out.dtype == x_dtype else out.to(x_dtype)

    def shares_kernel_input_with(self, other) -> bool:
        return (getattr(other, "use_kernel", False) and self.use_kernel
                and not (self.online_full_had or self.online_partial_had)
                and not (other.online_full_had or other.online_partial_had)
                and type(self.kernel_quantizer) is type(other.kernel_quantizer)
                and self.kernel_quantizer.clip_ratio == other.kernel_quantizer.clip_ratio
                and self.in_features == other.in_features)

    def forward(self, x):
        return self.kernel_matmul(self.kernel_quantize(x), x.dtype)


def _shares_input(first, *others):
    shares = getattr(first, "shares_kernel_input_with", None)
    return shares is not None and all(shares(o) for o in others)


# ----------------------------------------------------------------------------- layer forwards

def kernel_attention_forward(self, hidden_states, position_embeddings, attention_mask=None, past_key_values=None,
                             cache_position=None, packed_input=None, **kwargs):
    """Attention over the paged int4 cache.  `self` carries q_proj/k_proj/v_proj/o_proj,
    `head_dim`, `layer_idx` (and optionally q_norm/k_norm).  Returns (output, None).

    `packed_input`: the already quantized activation (the caller fused the quantizer with the
    normalisation in front of it); `hidden_states` then only gives shape and dtype.  When the
    module carries `qkv_fused` (see `fuse_projections_`), the three projections are one GEMM and
    q/k/v are column ranges of its output; with a cache that offers `update_with_rope`, the rotary
    embedding, the K rotation, the K/V quantizers and the page scatter are one launch."""
    input_shape = hidden_states.shape[:-1]
    hidden_shape = (*input_shape, -1, self.head_dim)
    dtype = hidden_states.dtype

    if _shares_input(self.q_proj, self.k_proj, self.v_proj):
        packed = packed_input if packed_input is not None else self.q_proj.kernel_quantize(hidden_states)
        fused = getattr(self, "qkv_fused", None)
        if fused is not None:
            qkv = fused(packed)
            if qkv.dtype != dtype:
                qkv = qkv.to(dtype)
            nq, nk = self.q_proj.out_features, self.k_proj.out_features
            query_states = qkv[..., :nq].unflatten(-1, (-1, self.head_dim))
            key_states = qkv[..., nq:nq + nk].unflatten(-1, (-1, self.head_dim))
            value_states = qkv[..., nq + nk:].unflatten(-1, (-1, self.head_dim))
        else:
            query_states = self.q_proj.kernel_matmul(packed, dtype).view(hidden_shape)
            key_states = self.k_proj.kernel_matmul(packed, dtype).view(hidden_shape)
            value_states = self.v_proj.kernel_matmul(packed, dtype).view(hidden_shape)
    else:
        assert packed_input is None
        query_states = self.q_proj(hidden_states).view(hidden_shape)
        key_states = self.k_proj(hidden_states).view(hidden_shape)
        value_states = self.v_proj(hidden_states).view(hidden_shape)
    if hasattr(self, "q_norm"):
        query_states = self.q_norm(query_states)
        key_states = self.k_norm(key_states)

    # the KV kernels and the decode kernel are fp16-only
    if query_states.dtype != torch.float16:
        query_states, key_states = query_states.to(torch.float16), key_states.to(torch.float16)
        value_states = value_states.to(torch.float16)
    cos, sin = position_embeddings
    if cos.dtype != torch.float16:
        cos, sin = cos.to(torch.float16), sin.to(torch.float16)

    if past_key_values is not None and attention_mask is None and hasattr(past_key_values, "update_with_rope") \
            and getattr(self, "fuse_rope_append", True):
        # the callable this returns is called right below: a decode step may leave rotation and append to it
        query_states, cache_out = past_key_values.update_with_rope(query_states, key_states, value_states, cos, sin,
                                                                   self.layer_idx, defer_append=True)
    else:
        query_states, key_states = query_states.contiguous(), key_states.contiguous()
        kernel.rope_qk(query_states, key_states, cos, sin)     # in place
        if past_key_values is not None:
            cache_out = past_key_values.update(key_states, value_states, self.layer_idx,
                                               {"attention_mask": attention_mask})
        else:
            cache_out = (key_states, value_states)

    if isinstance(cache_out, tuple):
        # prefill: the cache stored the rotated int4 K/V and handed back the fp16 originals
        key_states, value_states = cache_out
        attn_output = torch.nn.functional.scaled_dot_product_attention(
            query_states.transpose(1, 2), key_states.transpose(1, 2), value_states.transpose(1, 2),
            is_causal=True, enable_gqa=key_states.shape[2] != query_states.shape[2]).transpose(1, 2)
    else:
        attn_output = cache_out(query_states)

    attn_output = attn_output.reshape(*input_shape, -1)
    if attn_output.dtype != dtype:
        attn_output = attn_output.to(dtype)
    return self.o_proj(attn_output), None


def kernel_mlp_forward(self, x, packed_input=None):
    """SwiGLU MLP: one quantization for gate and up, fused silu*mul, rotation + quantization of
    the product in one launch inside down_proj.  With `gate_up_fused` (see `fuse_projections_`)
    the two projections and the activation are one launch for up to 32 rows."""
    if _shares_input(self.gate_proj, self.up_proj):
        packed = packed_input if packed_input is not None else self.gate_proj.kernel_quantize(x)
        fused = getattr(self, "gate_up_fused", None)
        if fused is not None:
            wsum = fused._weight_sum() if packed.zeros_x is not None else None
            inter = kernel.w4a4_swiglu(packed, fused.weight, fused.weight_scales, wsum, fused.bias)
        else:
            gate = self.gate_proj.kernel_matmul(packed, torch.float16)
            up = self.up_proj.kernel_matmul(packed, torch.float16)
            inter = kernel.swiglu(gate, up)
    else:
        assert packed_input is None
        inter = kernel.swiglu(self.gate_proj(x).to(torch.float16), self.up_proj(x).to(torch.float16))
    out = self.down_proj(inter)
    return out if out.dtype == x.dtype else out.to(x.dtype)


def _stack_linears(linears):
    """One Linear4bit whose weight is the row-wise concatenation of `linears`' weights; the
    originals' buffers become views of it, so nothing is stored twice and state_dict keeps the
    per-projection names."""
    mods = [lin.kernel_module for lin in linears]
    if any(m.bias is not None for m in mods) and not all(m.bias is not None for m in mods):
        return None
    k = mods[0].in_features
    fused = snn.Linear4bit(k, sum(m.out_features for m in mods), bias=mods[0].bias is not None)
    fused.weight = torch.cat([m.weight for m in mods], dim=0).contiguous()
    fused.weight_scales = torch.cat([m.weight_scales.to(torch.float16) for m in mods], dim=0).contiguous()
    if mods[0].bias is not None:
        fused.bias = torch.cat([m.bias for m in mods], dim=0).contiguous()
    row = 0
    for m in mods:
        m.weight = fused.weight[row:row + m.out_features]
        m.weight_scales = fused.weight_scales[row:row + m.out_features]
        if m.bias is not None:
            m.bias = fused.bias[row:row + m.out_features]
        if hasattr(m, "weight_sum"):
            del m.weight_sum
        row += m.out_features
    return fused


def fuse_projections_(layer):
    """Concatenates q/k/v into one GEMM and gate/up into one (SwiGLU-fused for decode) where the
    siblings share their quantized input.  Call after the weights are loaded and on their final
    device (moving the module afterwards would split the views again; call it once more then)."""
    at = layer.self_attn
    if _shares_input(at.q_proj, at.k_proj, at.v_proj):
        object.__setattr__(at, "qkv_fused", _stack_linears([at.q_proj, at.k_proj, at.v_proj]))
    mlp = getattr(layer, "mlp", None)
    if hasattr(mlp, "gate_proj") and _shares_input(mlp.gate_proj, mlp.up_proj) \
            and mlp.gate_proj.out_features == mlp.up_proj.out_features:
        object.__setattr__(mlp, "gate_up_fused", _stack_linears([mlp.gate_proj, mlp.up_proj]))
    return layer


# ----------------------------------------------------------------------------- decoder stack

@dataclass
class DecoderConfig:
    """Geometry of the stack; the defaults are Llama-3-8B's."""
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    num_local_experts: int = 0        # > 0: every MLP is a sparse block of that many experts
    num_experts_per_tok: int = 2
    norm_topk_prob: bool = True
    a_asym: bool = False
    a_clip_ratio: float = 1.0
    had_adj: bool = True              # SignRot sign vector on down_proj's rotation
    fp32_had: bool = False            # online rotations in fp32, one rounding after the transform (OnlineHadamard force_fp32)
    attention_bias: bool = False      # q/k/v projections carry a bias (Qwen-style checkpoints)
    fuse_edges: bool = True           # fused launches across the path's edges (same bits as the separate ones)


class KernelAttention(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        q_out, kv_out = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
        kw = dict(asym=cfg.a_asym, clip_ratio=cfg.a_clip_ratio)
        self.head_dim = cfg.head_dim
        self.layer_idx = layer_idx
        self.q_proj = KernelLinear(cfg.hidden_size, q_out, bias=cfg.attention_bias, **kw)
        self.k_proj = KernelLinear(cfg.hidden_size, kv_out, bias=cfg.attention_bias, **kw)
        self.v_proj = KernelLinear(cfg.hidden_size, kv_out, bias=cfg.attention_bias, **kw)
        self.o_proj = KernelLinear(q_out, cfg.hidden_size, online_partial_had=True, had_dim=cfg.head_dim,
                                   fp32_had=cfg.fp32_had, **kw)

    forward = kernel_attention_forward


class KernelMLP(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        kw = dict(asym=cfg.a_asym, clip_ratio=cfg.a_clip_ratio)
        self.gate_proj = KernelLinear(cfg.hidden_size, cfg.intermediate_size, **kw)
        self.up_proj = KernelLinear(cfg.hidden_size, cfg.intermediate_size, **kw)
        self.down_proj = KernelLinear(cfg.intermediate_size, cfg.hidden_size, online_full_had=True,
                                      had_adj=cfg.had_adj, fp32_had=cfg.fp32_had, **kw)

    forward = kernel_mlp_forward


class KernelDecoderLayer(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int):
        super().__init__()
        self.input_layernorm = snn.RMSNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)
        self.post_attention_layernorm = snn.RMSNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)
        self.self_attn = KernelAttention(cfg, layer_idx)
        self.mlp = KernelMLP(cfg) if cfg.num_local_experts == 0 else None   # sparse block attached later
        self.fuse_edges = cfg.fuse_edges
        self.self_attn.fuse_rope_append = cfg.fuse_edges

    def _fusable(self, x):
        return (self.fuse_edges and x.dtype == torch.float16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384)

    def forward(self, hidden_states, position_embeddings, past_key_values=None, delta=None):
        """`delta`: the previous layer's MLP output, not yet added to the residual stream (the add
        is fused into this layer's first normalisation).  Returns (hidden, delta) in the same form."""
        at, mlp = self.self_attn, self.mlp
        q = at.q_proj.kernel_quantizer
        if self._fusable(hidden_states) and _shares_input(at.q_proj, at.k_proj, at.v_proj):
            # residual add + RMSNorm + quantizer of q/k/v: one launch
            hidden_states, packed = kernel.add_rmsnorm_quant(
                hidden_states, delta, self.input_layernorm.eps, self.input_layernorm.mean_dim, q.clip_ratio,
                asym=isinstance(q, snn.AsymQuantizer))
            attn, _ = at(hidden_states, position_embeddings, past_key_values=past_key_values, packed_input=packed)
        else:
            if delta is not None:
                hidden_states = hidden_states + delta
            attn, _ = at(self.input_layernorm(hidden_states), position_embeddings, past_key_values=past_key_values)
        norm2 = self.post_attention_layernorm
        if self._fusable(hidden_states) and hasattr(mlp, "gate_proj") and _shares_input(mlp.gate_proj, mlp.up_proj):
            q = mlp.gate_proj.kernel_quantizer
            hidden_states, packed = kernel.add_rmsnorm_quant(hidden_states, attn, norm2.eps, norm2.mean_dim,
                                                             q.clip_ratio, asym=isinstance(q, snn.AsymQuantizer))
            mlp_out = mlp(hidden_states, packed_input=packed)
        else:
            hidden_states = hidden_states + attn
            mlp_out = mlp(norm2(hidden_states))
            if isinstance(mlp_out, tuple):      # sparse block: (output, router logits)
                mlp_out = mlp_out[0]
        return hidden_states, mlp_out


class _Logits:
    __slots__ = ("logits",)

    def __init__(self, logits):
        self.logits = logits


class KernelDecoderModel(torch.nn.Module):
    """Embedding -> decoder layers -> RMSNorm -> fp16 lm_head (the head stays unquantized, as in
    the reference's pipeline).  `forward(input_ids, past_key_values, cache_position)` follows
    the call the graph runner makes."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.config = cfg
        self.embed_tokens = torch.nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=torch.float16)
        self.layers = torch.nn.ModuleList(KernelDecoderLayer(cfg, i) for i in range(cfg.num_hidden_layers))
        self.norm = snn.RMSNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)
        self.lm_head = torch.nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, dtype=torch.float16)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32) / cfg.head_dim))
        self.register_buffer("inv_freq", inv, persistent=False)

    def get_input_embeddings(self):
        return self.embed_tokens

    def rotary(self, positions):
        """cos/sin [1, T, head_dim] in fp16 from int64 positions [T] (fp32 angles, then the cast)."""
        ang = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]
        emb = torch.cat((ang, ang), dim=-1)
        return emb.cos().to(torch.float16)[None], emb.sin().to(torch.float16)[None]

    def forward(self, input_ids, past_key_values=None, use_cache=True, cache_position=None, last_token_only=False):
        t = input_ids.shape[1]
        if cache_position is None:
            start = past_key_values.get_seq_length() if past_key_values is not None else 0
            cache_position = torch.arange(start, start + t, device=input_ids.device)
        elif cache_position.numel() == 1 and t > 1:
            cache_position = cache_position + torch.arange(t, device=input_ids.device)
        pos = self.rotary(cache_position)
        h, delta = self.embed_tokens(input_ids), None
        for layer in self.layers:
            h, delta = layer(h, pos, past_key_values, delta)
        if last_token_only:
            h, delta = h[:, -1:, :], delta[:, -1:, :]
        return _Logits(self.lm_head(self.norm(h + delta)))

    def fuse_projections_(self):
        if self.config.fuse_edges:
            for layer in self.layers:
                fuse_projections_(layer)
        return self

    @torch.no_grad()
    def random_init_(self, seed: int = 0):
        """Random int4 codes, weight scales about 1/K (keeps fp16 activations finite through many
        layers; the trick of benchmarks/decode_sweep.py:65-71), random +-1 adjustment signs,
        N(0, 0.02) embedding and head.  Runs on the module's device."""
        dev = self.embed_tokens.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        cfg = self.config

        def fill(lin: snn.Linear4bit):
            n, k = lin.out_features, lin.in_features
            lin.weight.copy_(torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8, device=dev))
            lin.weight_scales = ((torch.rand((n, 1), generator=g, device=dev) * 0.5 + 0.5) / k).to(torch.float16)

        def sign(n):
            return (torch.randint(0, 2, (n,), generator=g, device=dev) * 2 - 1).to(torch.int8)

        for layer in self.layers:
            at = layer.self_attn
            for lin in (at.q_proj, at.k_proj, at.v_proj, at.o_proj):
                fill(lin.kernel_module)
            if cfg.num_local_experts == 0:
                for lin in (layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
                    fill(lin.kernel_module)
                had = layer.mlp.down_proj.kernel_hadamard
                if had.had_adj_sign is not None:
                    had.had_adj_sign.copy_(sign(cfg.intermediate_size))
            else:
                e, hid, ffn = cfg.num_local_experts, cfg.hidden_size, cfg.intermediate_size

                def stack(n, k):
                    w = torch.randint(0, 256, (e, n, k // 2), generator=g, dtype=torch.uint8, device=dev)
                    s = ((torch.rand((e, n), generator=g, device=dev) * 0.5 + 0.5) / k).to(torch.float16)
                    return w, s
                wg, sg = stack(ffn, hid)
                wu, su = stack(ffn, hid)
                wd, sd = stack(hid, ffn)
                gate = torch.nn.Linear(hid, e, bias=False, dtype=torch.float16, device=dev)
                gate.weight.copy_(torch.randn((e, hid), generator=g, device=dev) * 0.02)
                sd_sign = torch.stack([sign(ffn) for _ in range(e)]).contiguous() if cfg.had_adj else None
                layer.mlp = snn.SignRotMoEBlock(gate, top_k=cfg.num_experts_per_tok, norm_topk_prob=cfg.norm_topk_prob,
                                                w_gate=wg, s_gate=sg, w_up=wu, s_up=su, w_down=wd, s_down=sd,
                                                sign_down=sd_sign, asym=cfg.a_asym, clip_ratio=cfg.a_clip_ratio)
        self.embed_tokens.weight.copy_(torch.randn(self.embed_tokens.weight.shape, generator=g, device=dev) * 0.02)
        self.lm_head.weight.copy_(torch.randn(self.lm_head.weight.shape, generator=g, device=dev) * 0.02)
        return self.fuse_projections_()


def build_paged_cache(model, batch_size, max_length, page_size=None):
    """Paged int4 cache sized for `max_length` tokens per request."""
    from .kv_cache import decode_split
    cfg = model.config
    page = min(page_size or DEFAULT_PAGE_SIZE, max_length)
    device = model.get_input_embeddings().weight.device
    chunks = None
    tp_world = getattr(model, "tp_world", 1)
    if tp_world > 1:   # the split of the unsharded model: same merge order, same bits
        chunks = decode_split(batch_size, cfg.num_key_value_heads * tp_world, -(-max_length // page), device)
    return MultiLayerPagedKVCache4Bit(
        batch_size=batch_size, page_size=page, max_seq_len=max_length, device=device,
        n_layers=cfg.num_hidden_layers, num_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
        hadamard_dtype=torch.float16, group_size=cfg.num_attention_heads // cfg.num_key_value_heads,
        decode_chunks=chunks)


# ----------------------------------------------------------------------------- graph runner

class GraphedDecoder:
    """The decode step as one CUDA graph that needs nothing from the host between replays but the token.

    The graph's first node is the cache's `advance_on_device` launch: it turns the device-resident token
    count into the position of the token being appended (which drives the rotary tables) and into the
    page tables of the sequence that includes it, and increments the count.  The decoder stack follows,
    reading those tensors.  A replay is therefore `token -> buffer, replay`: no index tensor is rewritten
    from the host (the reference's runner refreshes position and cache specs from Python before every
    replay, fake_quant/kernel_utils.py:164-254).  The host keeps its own copy of the length for
    bookkeeping and re-synchronises the device count only when the two were moved apart (an eager step,
    a rewind)."""

    def __init__(self, model, cache, batch_size):
        self.model, self.cache = model, cache
        self.pool = getattr(cache, "inner", cache)
        dev = model.get_input_embeddings().weight.device
        self.token = torch.zeros((batch_size, 1), dtype=torch.long, device=dev)
        self.graph = None
        self.logits = None
        self._device_length = None          # what the device-resident count holds, as far as the host knows

    def _sync(self):
        if self._device_length != self.pool.length:
            self.pool.sync_device_length()
            self._device_length = self.pool.length

    def _body(self):
        """What gets captured.  The Python side effects of the cache's `update` (host length, first-call
        flags) run once at capture time and are undone by the caller."""
        position = self.pool.advance_on_device()
        return self.model(self.token, past_key_values=self.cache, use_cache=True, cache_position=position).logits

    def capture(self, warmup: int = 2):
        pool, at = self.pool, self.pool.length
        if at + 1 > pool.capacity():
            raise RuntimeError(f"the cache holds {pool.capacity()} tokens per request; no room to capture a step at {at}")
        pool.freeze_specs(True)             # `update` must not rewrite the tables the device node owns
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(warmup):     # first-use work (attribute set-up, lazy buffers) outside the capture
                    pool.length, self._device_length = at, None
                    self._sync()
                    self._body()
            torch.cuda.current_stream().wait_stream(side)
            pool.length, self._device_length = at, None
            self._sync()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.logits = self._body()
            self.graph = graph
        finally:
            pool.length = at                # nothing was appended for real: the slot is rewritten by step()
            pool.freeze_specs(False)
        return self

    def step(self, token):
        """Appends `token` [B, 1] and returns the logits buffer (overwritten by the next step)."""
        if self.graph is None:
            raise RuntimeError("capture() must run before step()")
        pool = self.pool
        if pool.length + 1 > pool.capacity():
            raise RuntimeError(f"the cache is full ({pool.capacity()} tokens per request)")
        self._sync()
        self.token.copy_(token)
        self.graph.replay()
        pool.length += 1
        self._device_length = pool.length
        pool._spec_page_cnt = None          # the device node rewrote the page list
        return self.logits


def replay_matches_eager(model, cache, decoder: GraphedDecoder, probes: int = 2, tol: float = 1e-3) -> bool:
    """Runs `probes` unseen tokens through the eager step and through a replay from the same cache state and
    compares the logits.  A capture bakes in every host-side decision taken while it ran (kernel choice,
    chunk counts, buffer addresses); this is the check that those decisions still hold.  Leaves the cache
    where it found it.  Also surfaces a device-side bounded-wait failure, which would otherwise turn every
    later output into garbage without an error."""
    from .. import _lib
    pool, at = decoder.pool, decoder.pool.length
    vocab = model.get_input_embeddings().weight.shape[0]
    gen = torch.Generator().manual_seed(at)
    ok = True
    for _ in range(probes):
        token = torch.randint(0, vocab, decoder.token.shape, generator=gen).to(decoder.token.device)
        pool.length = at
        want = model(token, past_key_values=cache, use_cache=True).logits.float()
        pool.length = at
        got = decoder.step(token).float()
        worst = ((got - want).abs().max() / want.abs().max().clamp_min(1e-6)).item()
        if not worst <= tol:                # also catches NaN
            logging.warning("decode graph replay differs from the eager step by %.3e of the logit range; "
                            "decoding eagerly", worst)
            ok = False
            break
    pool.length = at
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel gave up a bounded device-side wait; outputs since then are undefined")
    return ok


def try_graph_decoder(model, cache, batch_size, warmup=2, validate=True):
    """A captured decoder for `cache`, or None when the step cannot be captured or its replay does not
    reproduce the eager step (the caller then runs the same kernels launch by launch)."""
    if not torch.cuda.is_available():
        return None
    try:
        decoder = GraphedDecoder(model, cache, batch_size).capture(warmup=warmup)
    except Exception as exc:   # capture errors invalidate the stream capture only, not the context
        logging.warning("decode step could not be captured (%s); decoding eagerly", exc)
        torch.cuda.synchronize()
        return None
    if validate and not replay_matches_eager(model, cache, decoder):
        return None
    return decoder


@torch.no_grad()
def generate(model, input_ids, max_new_tokens, page_size=None, use_graph=True):
    """Greedy decoding: prefill, then `max_new_tokens - 1` decode steps (graph-replayed when
    capture succeeds).  Returns int64 tokens [B, max_new_tokens]."""
    bsz, prompt = input_ids.shape
    cache = build_paged_cache(model, bsz, prompt + max_new_tokens, page_size)
    logits = model(input_ids, past_key_values=cache, last_token_only=True).logits
    token = logits[:, -1:].argmax(-1)
    out = [token]
    decoder = try_graph_decoder(model, cache, bsz) if use_graph and max_new_tokens > 1 else None
    for _ in range(max_new_tokens - 1):
        if decoder is not None:
            logits = decoder.step(token)
        else:
            logits = model(token, past_key_values=cache).logits
        token = logits[:, -1:].argmax(-1)
        out.append(token)
    tokens = torch.cat(out, dim=1)
    torch.cuda.synchronize(tokens.device)
    from .. import _lib
    if _lib.device_status() != 0:       # per device: the status word lives on the current device
        raise RuntimeError("a kernel gave up a bounded device-side wait during generation; the tokens are undefined")
    return tokens


# ----------------------------------------------------------------------------- tensor parallelism

class TPRowLinear(torch.nn.Module):
    """o_proj / down_proj of a tensor-parallel layer: this rank holds the input channels of its own
    heads (or of its slice of the MLP width).  The online rotation and the per-token scale span the
    whole input, so the fp16 shards are all-gathered, every rank rotates and quantizes the full row,
    multiplies its K-slice of the codes and the int32 partial sums are all-reduced: integer addition
    is associative, so every TP degree gives the bits of one GPU (`signrot_b200.tp`)."""

    def __init__(self, lin: KernelLinear, group, heads=0, peer=None):
        super().__init__()
        from .. import tp
        had = lin.kernel_hadamard
        full = lin.online_full_had
        self.use_kernel = True
        self.online_full_had, self.online_partial_had = lin.online_full_had, lin.online_partial_had
        self.out_features = lin.out_features
        self.row = tp.RowParallelLinear4bit(
            lin.kernel_module.weight, lin.kernel_module.weight_scales,
            hadK=had.had_rem_dim if full else None, K_had=had.rem_dim if full else 1,
            sign=had.had_adj_sign if full else None, heads=heads, clip_ratio=lin.kernel_quantizer.clip_ratio, group=group,
            peer=peer)

    def forward(self, x_local):
        lead = x_local.shape[:-1]
        out = self.row.forward(x_local.reshape(-1, x_local.shape[-1]).contiguous())
        return out.view(*lead, self.out_features)


def _slice_linear(lin: KernelLinear, begin, end):
    """Output rows [begin, end) of a projection without an online rotation (column parallelism)."""
    has_bias = lin.kernel_module.bias is not None
    new = KernelLinear(lin.in_features, end - begin, bias=has_bias, asym=lin._asym, clip_ratio=lin.kernel_quantizer.clip_ratio)
    new = new.to(lin.kernel_module.weight.device)
    new.kernel_module.weight = lin.kernel_module.weight[begin:end].contiguous()
    new.kernel_module.weight_scales = lin.kernel_module.weight_scales[begin:end].contiguous()
    if has_bias:
        new.kernel_module.bias = lin.kernel_module.bias[begin:end].contiguous()
    return new


def shard_decoder_(model: "KernelDecoderModel", group=None, peer="auto"):
    """Turns a (replicated) `KernelDecoderModel` into this rank's shard, in place: q/k/v column-parallel by heads
    (no collective), o_proj row-parallel (`TPRowLinear`: one gather and one integer reduce), KV cache per rank over
    its own KV heads; a dense MLP is tensor-parallel the same way (gate/up by width, down_proj row-parallel), a
    sparse block expert-parallel (`SignRotMoEBlock.shard_experts_`: every rank routes all tokens and computes its
    own experts, one sum of the partial outputs); residual stream, norms, embedding and head are replicated.
    `peer`: a `signrot_b200.comm.PeerGroup` for the decode-size exchanges ("auto": one is created on CUDA; None:
    the collective library only).  The reference keeps this path on one device
    (fake_quant/kernel_utils.py:365-366)."""
    import torch.distributed as dist
    cfg = model.config
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    hq, hkv, d, ffn = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    sparse = cfg.num_local_experts > 0
    if hq % world or hkv % world:
        raise ValueError(f"{hq} q heads / {hkv} kv heads do not split {world} ways")
    if not sparse and ((ffn // world) % 64 or ffn % world):
        raise ValueError(f"MLP width {ffn} does not split {world} ways")
    if sparse and cfg.num_local_experts % world:
        raise ValueError(f"{cfg.num_local_experts} experts do not split {world} ways")
    if peer == "auto":
        peer = None
        if world > 1 and model.get_input_embeddings().weight.is_cuda:
            from ..comm import PeerGroup
            peer = PeerGroup(group)
    ql, kl, fl = hq // world * d, hkv // world * d, ffn // world
    for layer in model.layers:
        at, mlp = layer.self_attn, layer.mlp
        if "qkv_fused" in at.__dict__:
            object.__delattr__(at, "qkv_fused")
        o_row = TPRowLinear(at.o_proj, group, heads=hq, peer=peer)
        at.q_proj = _slice_linear(at.q_proj, rank * ql, (rank + 1) * ql)
        at.k_proj = _slice_linear(at.k_proj, rank * kl, (rank + 1) * kl)
        at.v_proj = _slice_linear(at.v_proj, rank * kl, (rank + 1) * kl)
        at.o_proj = o_row
        if sparse:
            mlp.shard_experts_(group, peer=peer)
            continue
        if "gate_up_fused" in mlp.__dict__:
            object.__delattr__(mlp, "gate_up_fused")
        down_row = TPRowLinear(mlp.down_proj, group, peer=peer)
        mlp.gate_proj = _slice_linear(mlp.gate_proj, rank * fl, (rank + 1) * fl)
        mlp.up_proj = _slice_linear(mlp.up_proj, rank * fl, (rank + 1) * fl)
        mlp.down_proj = down_row
    # the cache and the attention see this rank's heads only
    from dataclasses import replace
    model.config = replace(cfg, num_attention_heads=hq // world, num_key_value_heads=hkv // world)
    model.tp_world = world
    model.peer_group = peer
    return model.fuse_projections_()


# ----------------------------------------------------------------------------- sparse blocks

def build_moe_block(mlp):
    """A sparse MLP whose experts are per-expert `KernelLinear` triples (`mlp.experts[i].gate_proj / up_proj /
    down_proj`, router `mlp.gate`, `mlp.top_k`, `mlp.norm_topk_prob`) -> one `SignRotMoEBlock` over stacked
    expert weights: routing on the GPU, grouped int4 GEMMs and the per-expert adjustment signs fused into the
    down_proj quantizer (fake_quant/kernel_utils.py:295-349).  Returns None, leaving the module as it is, when
    the experts are not uniformly kernel-enabled."""
    gates = [e.gate_proj for e in mlp.experts]
    ups = [e.up_proj for e in mlp.experts]
    downs = [e.down_proj for e in mlp.experts]
    wrappers = gates + ups + downs
    if not all(getattr(w, "use_kernel", False) and isinstance(w, KernelLinear) for w in wrappers):
        logging.warning("MoE experts are not all kernel-enabled; keeping the per-expert loop")
        return None
    quantizer = gates[0].kernel_quantizer
    assert all(type(w.kernel_quantizer) is type(quantizer) and w.kernel_quantizer.clip_ratio == quantizer.clip_ratio
               for w in wrappers), "MoE stacking expects one activation quantizer config across all experts"
    assert all(w.online_full_had for w in downs), "expert down_proj must run the online Hadamard on the kernel path"
    assert all(w.fp32_had == downs[0].fp32_had for w in downs)
    asym = isinstance(quantizer, snn.AsymQuantizer)
    w_gate, s_gate, _ = snn.SignRotMoEBlock.stack_experts([w.kernel_module for w in gates], need_wsum=False)
    w_up, s_up, _ = snn.SignRotMoEBlock.stack_experts([w.kernel_module for w in ups], need_wsum=False)
    w_down, s_down, _ = snn.SignRotMoEBlock.stack_experts([w.kernel_module for w in downs], need_wsum=False)
    sign_down = None
    if any(w.kernel_hadamard.had_adj_sign is not None for w in downs):
        inter = w_gate.shape[1]
        sign_down = torch.stack([
            w.kernel_hadamard.had_adj_sign.to(w_gate.device) if w.kernel_hadamard.had_adj_sign is not None
            else torch.ones(inter, dtype=torch.int8, device=w_gate.device)      # never-routed experts: identity
            for w in downs]).contiguous()
    return snn.SignRotMoEBlock(mlp.gate, top_k=mlp.top_k, norm_topk_prob=mlp.norm_topk_prob,
                               w_gate=w_gate, s_gate=s_gate, w_up=w_up, s_up=s_up, w_down=w_down, s_down=s_down,
                               sign_down=sign_down, asym=asym, clip_ratio=quantizer.clip_ratio,
                               fp32_had=downs[0].fp32_had)
