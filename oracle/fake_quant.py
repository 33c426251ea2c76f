"""Oracle: the reference's CPU fake-quant path and the seeded inputs of the benchmark
configurations.  Test infrastructure only (also the timed CPU baseline of bench.py).

Fake-quant = quantize-dequantize in floating point followed by an ordinary F.linear: the
non-kernel branch of ActQuantWrapper.forward (fake_quant/quant_utils.py:322-386) with RTN
weights (fake_quant/gptq_utils.py:411-465, quant_utils.py:453-520).  Real-quant = the same
layer through the integer kernels, restated with the other oracle modules.
"""
from __future__ import annotations

import math

import torch

from . import quant as Q
from . import gemm as G
from . import hadamard as H
from . import misc as M

__all__ = ["act_fake_quant", "rtn_weight", "derive_sign", "FakeLinear", "make_linear_case",
           "make_decoder_layer", "decoder_layer_fake_quant", "CONFIG2_SHAPES", "outlier_channels"]

CONFIG2_SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]  # (K, N)


# ----------------------------------------------------------------------------- quantizers

def act_fake_quant(x: torch.Tensor, clip: float = 1.0, sym: bool = True) -> torch.Tensor:
    """Per-token 4-bit quantize-dequantize in x's dtype (ActQuantizer.find_params/forward,
    fake_quant/quant_utils.py:95-144, 41-47; functional/quantization.py:30-40)."""
    shape = x.shape
    r = x.reshape(-1, shape[-1])
    xmin = r.min(1)[0] * clip
    xmax = r.max(1)[0] * clip
    if sym:
        xmax = torch.maximum(xmin.abs(), xmax)
        scale = (xmax / 7).unsqueeze(1)
        scale = torch.where(xmax.unsqueeze(1) == 0, torch.ones_like(scale), scale)
        q = torch.clamp(torch.round(r / scale), -8, 7)
        return (scale * q).reshape(shape).to(x.dtype)
    same = xmin == xmax
    xmin = torch.where(same, xmin - 1, xmin)
    xmax = torch.where(same, xmax + 1, xmax)
    scale = ((xmax - xmin) / 15).unsqueeze(1)
    zero = torch.round(-xmin.unsqueeze(1) / scale)
    q = torch.clamp(torch.round(r / scale) + zero, 0, 15)
    return (scale * (q - zero)).reshape(shape).to(x.dtype)


def rtn_weight(W: torch.Tensor, sign: torch.Tensor | None = None, mse: bool = False):
    """Per-channel symmetric int4 round-to-nearest in W's dtype (WeightQuantizer.find_params,
    quant_utils.py:453-520; rtn_fwrd with sign unfold/refold on the symmetric grid [-7, 7],
    gptq_utils.py:434-457).  Returns (Wq dequantized in W.dtype, scale [N,1] in W.dtype)."""
    minq = -8
    Wu = W
    if sign is not None:
        Wu = W * sign.to(W.dtype)
        minq = -7
    # extend_zero compares against an fp32 zero tensor, which promotes the range (and so the
    # scale and the quantize-dequantize arithmetic) to fp32 (quant_utils.py:468-472)
    xmin = torch.minimum(Wu.min(1)[0], torch.zeros(W.shape[0]))
    xmax = torch.maximum(Wu.max(1)[0], torch.zeros(W.shape[0]))
    xmax = torch.maximum(xmin.abs(), xmax).clamp(min=1e-5)
    scale = xmax / 7
    if mse:
        best = torch.full([W.shape[0]], float("inf"))
        base = scale.clone()
        for i in range(int(0.8 * 100)):
            p = 1 - i / 100
            s1 = (p * xmax) / 7
            q = s1.unsqueeze(1) * torch.clamp(torch.round(Wu / s1.unsqueeze(1)), minq, 7)
            err = (q - Wu).abs_().pow_(2.4).sum(1)
            better = err < best
            best = torch.where(better, err, best)
            base = torch.where(better, s1, base)
        scale = base
    scale = scale.reshape(-1, 1)
    Wq = (scale * torch.clamp(torch.round(Wu / scale), minq, 7)).to(W.dtype)
    if sign is not None:
        Wq = Wq * sign.to(W.dtype)
    return Wq.to(W.dtype), scale


def derive_sign(x_rot: torch.Tensor) -> torch.Tensor:
    """SignRot sign vector from one calibration sample after rotation: the token with the
    largest magnitude, sign of each of its channels as int8 +-1 (quant_utils.py:362-368)."""
    single = x_rot[0] if x_rot.dim() == 3 else x_rot
    t = single.abs().max(dim=-1).values.argmax()
    return ((single[t] >= 0) * 2 - 1).to(torch.int8)


# ----------------------------------------------------------------------------- one linear

class FakeLinear:
    """One quantized linear with its online rotation, in both statements.

    rot: None | ("full", hadK, K) | ("heads", n_heads).  `sign` (int8 [K]) is folded into the
    weight columns and applied to the rotated activation (SignRot).  Weights are stored
    dequantized (`Wq`, model dtype) for the fake path and packed (`w_packed`, `w_scale` fp16)
    for the integer path, as ActQuantWrapper.enable_kernel builds them
    (quant_utils.py:214-276, nn/linear.py:52-73)."""

    def __init__(self, W: torch.Tensor, rot=None, sign: torch.Tensor | None = None, clip: float = 1.0,
                 mse: bool = False):
        self.rot, self.sign, self.clip = rot, sign, clip
        if sign is not None:
            W = W * sign.to(W.dtype)  # fold: quant_utils.py:367
        self.Wq, scale = rtn_weight(W, sign, mse)
        w16 = self.Wq.to(torch.float16)
        self.w_scale = scale.to(torch.float16)
        codes = (w16 / self.w_scale).round().to(torch.int32)
        self.w_codes = codes
        self.w_packed = Q.pack_i4(codes)

    def _rotate(self, x, dtype_mode):
        if self.rot is None:
            y = x
        elif self.rot[0] == "full":
            y = H.rotate(x, self.rot[1], self.rot[2], None)
        else:
            y = H.rotate_heads(x, self.rot[1])
        if self.sign is not None:
            y = y * self.sign.to(y.dtype)
        return y

    def fake(self, x: torch.Tensor) -> torch.Tensor:
        """quant_utils.py:322-386: rotate in x.dtype, sign, fake-quant, F.linear."""
        y = self._rotate(x, None)
        y = act_fake_quant(y, self.clip, True).to(x.dtype)
        return torch.nn.functional.linear(y, self.Wq.to(x.dtype)).to(x.dtype)

    def real(self, x: torch.Tensor) -> torch.Tensor:
        """quant_utils.py:278-296 through the integer path: x.to(fp16), rotation with fp16
        rounding points, Quantizer, int4 GEMM, dequant; result cast back to x.dtype."""
        x16 = x.to(torch.float16)
        y = self._rotate(x16, None)
        codes, s = Q.sym_quant_dynamic(y.reshape(-1, y.shape[-1]), self.clip)
        out = G.w4a4_linear(Q.pack_codes(codes), s, self.w_packed, self.w_scale)
        return out.reshape(*x.shape[:-1], -1).to(x.dtype)

    def real_parts(self, x: torch.Tensor):
        """(codes, scale, int32 accumulators, fp16 output) of the integer path."""
        x16 = x.to(torch.float16)
        y = self._rotate(x16, None)
        codes, s = Q.sym_quant_dynamic(y.reshape(-1, y.shape[-1]), self.clip)
        acc = G.matmul_i4(Q.pack_codes(codes), self.w_packed)
        return codes, s, acc, Q.sym_dequant(acc, s, self.w_scale)


def outlier_channels(K: int) -> torch.Tensor:
    """The fixed 0.1 % of channels that carry x100 outliers in the op-sweep inputs."""
    n = max(1, math.ceil(K / 1000))
    g = torch.Generator().manual_seed(1234 + K)
    return torch.randperm(K, generator=g)[:n].sort().values


def make_linear_case(M: int, K: int, N: int, seed: int = 0, dtype=torch.bfloat16):
    """Seeded inputs of the fused-op sweep: activations ~N(0,1) in bf16 with 0.1 % of the
    channels x100, int4 weight codes uniform in [-8, 7], fp16 weight scales ~U(0.001, 0.01),
    random +-1 sign vector (as scripts/reproduce/analysis/efficiency/speedup_single_linear.py:27-29
    draws it).  Returns dict(x, w_packed, w_scale, sign)."""
    g = torch.Generator().manual_seed(seed * 1000003 + K * 31 + N)
    x = torch.randn((M, K), generator=g, dtype=torch.float32)
    ch = outlier_channels(K)
    x[:, ch] *= 100.0
    codes = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int32)
    w_scale = (torch.rand((N, 1), generator=g) * 0.009 + 0.001).to(torch.float16)
    sign = (torch.randint(0, 2, (K,), generator=g) * 2 - 1).to(torch.int8)
    return {"x": x.to(dtype), "w_packed": Q.pack_i4(codes), "w_scale": w_scale, "sign": sign}


# ----------------------------------------------------------------------------- decoder layer (config 1)

def _random_hadamard(n: int, g: torch.Generator) -> torch.Tensor:
    """H diag(+-1) in float64 (signrot/functional/hadamard.py:70-75)."""
    d = torch.randint(0, 2, (n,), generator=g).to(torch.float64) * 2 - 1
    return H.fwht(torch.diag(d)) / math.sqrt(n)


def make_decoder_layer(seed: int = 0, hidden=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336,
                       tokens=2048, dtype=torch.bfloat16, hadK_ffn=None, K_ffn=1, outlier=(1415, 2533)):
    """One Llama-3-8B-shaped decoder layer after the offline pipeline, from a seed:
    weights ~N(0, 0.02) in `dtype`; randomized-Hadamard Q folded into every linear
    (rotation_utils.py:281-350: input side of q/k/v/gate/up, output side of o/down), exact
    Hadamard on down_proj's input side (:208-210) and per-head Hadamard on v_proj's output /
    o_proj's input (:225-235); input x ~N(0,1) with two fixed channels set to +-800 on every
    token; SignRot sign for down_proj derived from this x by the reference procedure; RTN int4
    weights.  Returns dict with the FakeLinear objects and x (already in the rotated basis)."""
    g = torch.Generator().manual_seed(seed)
    def w(n, k):
        return (torch.randn((n, k), generator=g) * 0.02).to(torch.float64)
    Wq, Wk, Wv = w(heads * head_dim, hidden), w(kv_heads * head_dim, hidden), w(kv_heads * head_dim, hidden)
    Wo, Wg, Wu, Wd = w(hidden, heads * head_dim), w(ffn, hidden), w(ffn, hidden), w(hidden, ffn)
    x = torch.randn((1, tokens, hidden), generator=g, dtype=torch.float64)
    if outlier and hidden > max(outlier):
        x[..., outlier[0]] = 800.0
        x[..., outlier[1]] = -800.0
    Qm = _random_hadamard(hidden, g)
    # y = W x  ->  (W Q)(Q^T x): inputs live in the rotated basis
    Wq, Wk, Wv, Wg, Wu = Wq @ Qm, Wk @ Qm, Wv @ Qm, Wg @ Qm, Wu @ Qm
    Wo, Wd = Qm.T @ Wo, Qm.T @ Wd
    xr = (x @ Qm).to(dtype)
    # down_proj input: exact Hadamard folded on the weight's input side
    Wd = H.rotate(Wd.float(), hadK_ffn, K_ffn, None).double()
    # v_proj output / o_proj input: per-head Hadamard (head_dim) and across-heads Hadamard
    Wv = (H.fwht(Wv.T.reshape(hidden, kv_heads, head_dim).float()) / math.sqrt(head_dim)).reshape(hidden, -1).T.double()
    Wo = (H.fwht(Wo.reshape(hidden, heads, head_dim).float()) / math.sqrt(head_dim)).reshape(hidden, -1).double()
    Wo = H.rotate_heads(Wo.float(), heads).double()
    layer = {
        "hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim, "ffn": ffn, "x": xr,
        "q": FakeLinear(Wq.to(dtype)), "k": FakeLinear(Wk.to(dtype)), "v": FakeLinear(Wv.to(dtype)),
        "o": FakeLinear(Wo.to(dtype), rot=("heads", heads)),
        "gate": FakeLinear(Wg.to(dtype)), "up": FakeLinear(Wu.to(dtype)),
        "down_W": Wd.to(dtype), "down_rot": ("full", hadK_ffn, K_ffn),
    }
    return layer


def _rope_tables(tokens, head_dim, dtype, theta=500000.0):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(tokens, dtype=torch.float32), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype)[None], emb.sin().to(dtype)[None]


def _rope(x, cos, sin):
    d = x.shape[-1] // 2
    rot = torch.cat((-x[..., d:], x[..., :d]), dim=-1)
    return x * cos.unsqueeze(2) + rot * sin.unsqueeze(2)


def decoder_layer_fake_quant(layer: dict, mode: str = "fake", attn_fp32: bool = False,
                             trace: dict | None = None) -> torch.Tensor:
    """Forward of the layer on layer['x'] with every linear fake-quantized (mode 'fake') or run
    through the integer path (mode 'real').  Derives the down_proj sign on first use
    (quant_utils.py:358-368).  Returns the layer output [1, T, hidden] in the model dtype."""
    x = layer["x"]
    dt = x.dtype
    Hh, Hk, D = layer["heads"], layer["kv_heads"], layer["head_dim"]
    T = x.shape[1]
    def run(lin_name, t):
        lin = layer[lin_name]
        out = lin.fake(t) if mode == "fake" else lin.real(t)
        if trace is not None:
            trace[lin_name] = (t, out)
        return out
    def norm(t):
        tf = t.float()
        return (tf * torch.rsqrt(tf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dt)
    h = norm(x)
    q = run("q", h).view(1, T, Hh, D)
    k = run("k", h).view(1, T, Hk, D)
    v = run("v", h).view(1, T, Hk, D)
    cos, sin = _rope_tables(T, D, dt)
    q, k = _rope(q, cos, sin), _rope(k, cos, sin)
    adt = torch.float32 if attn_fp32 else dt  # prefill attention is dense and outside the path
    attn = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2).to(adt), k.transpose(1, 2).repeat_interleave(Hh // Hk, dim=1).to(adt),
        v.transpose(1, 2).repeat_interleave(Hh // Hk, dim=1).to(adt), is_causal=True)
    attn = attn.transpose(1, 2).reshape(1, T, Hh * D).to(dt)
    x1 = x + run("o", attn)
    if trace is not None:
        trace["x1"] = x1
    h2 = norm(x1)
    g, u = run("gate", h2), run("up", h2)
    m = (torch.nn.functional.silu(g) * u).to(dt)
    if "down" not in layer:
        rot = layer["down_rot"]
        m_rot = H.rotate(m if mode == "fake" else m.to(torch.float16), rot[1], rot[2], None)
        sign = derive_sign(m_rot)
        layer["down_sign"] = sign
        layer["down"] = FakeLinear(layer["down_W"], rot=rot, sign=sign)
    return x1 + run("down", m)
