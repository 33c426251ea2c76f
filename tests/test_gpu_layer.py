"""One decoder layer through the package's modules (real int4 kernels) against the oracle's
integer statement and its fake-quant statement of the same layer (Llama-3-8B layer shapes with the
two massive-outlier channels, shortened in tokens so the CPU side stays within seconds).
fp16 outputs: rel-L2 <= 1e-3."""
import pytest
import torch

import oracle
from oracle import fake_quant as fq
from conftest import rel_l2
from signrot_b200 import nn as snn
from signrot_b200.functional import kernel
from signrot_b200.functional.hadamard import get_hadK

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lin(fl):
    m = snn.Linear4bit(fl.w_packed.shape[1] * 2, fl.w_packed.shape[0]).to(DEV)
    m.weight.copy_(fl.w_packed)
    m.weight_scales = fl.w_scale.to(DEV)
    return m


def gpu_layer(layer):
    x = layer["x"].to(DEV)
    dt = x.dtype
    Hh, Hk, D, hidden = layer["heads"], layer["kv_heads"], layer["head_dim"], layer["hidden"]
    T = x.shape[1]
    lin = {k: _lin(layer[k]) for k in ("q", "k", "v", "o", "gate", "up", "down")}
    quant = snn.Quantizer()
    norm = snn.RMSNorm(hidden, eps=1e-5)
    h = norm(x.to(torch.float16))
    pk = quant(h)                                   # q/k/v share one quantization
    q = lin["q"](pk).view(1, T, Hh, D)
    k = lin["k"](pk).view(1, T, Hk, D)
    v = lin["v"](pk).view(1, T, Hk, D)
    cos, sin = fq._rope_tables(T, D, torch.float16)
    kernel.rope_qk(q, k, cos.to(DEV), sin.to(DEV))
    attn = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2).float(), k.transpose(1, 2).repeat_interleave(Hh // Hk, dim=1).float(),
        v.transpose(1, 2).repeat_interleave(Hh // Hk, dim=1).float(), is_causal=True)
    attn = attn.transpose(1, 2).reshape(1, T, Hh * D).to(torch.float16)
    o = lin["o"](kernel.rotate_quant(attn, heads=Hh))
    x1 = (x.to(torch.float16) + o).to(dt)
    h2 = norm(x1.to(torch.float16))
    pk2 = quant(h2)                                 # gate/up share one quantization
    m = kernel.swiglu(lin["gate"](pk2), lin["up"](pk2))
    rot = layer["down_rot"]
    d = lin["down"](kernel.rotate_quant(m, rot[1], rot[2], sign=layer["down_sign"].to(DEV)))
    return (x1.to(torch.float16) + d).to(dt)


@pytest.mark.parametrize("shape", ["small", "llama3-8b"])
def test_decoder_layer_fp16(shape):
    if shape == "small":
        hadK, K = get_hadK(768)
        cfg = dict(hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=768, tokens=96, outlier=(15, 33))
    else:
        hadK, K = get_hadK(14336)
        cfg = dict(hidden=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336, tokens=64, outlier=(1415, 2533))
    layer = fq.make_decoder_layer(seed=0, dtype=torch.float16, hadK_ffn=hadK, K_ffn=K, **cfg)
    trace = {}
    want_real = fq.decoder_layer_fake_quant(layer, "real", attn_fp32=True, trace=trace)  # also derives the sign
    want_fake = fq.decoder_layer_fake_quant(layer, "fake", attn_fp32=True)

    # every quantized linear on the oracle's own input: rel-L2 <= 1e-3 against the integer
    # statement (codes can only differ at exact rounding ties)
    quant = snn.Quantizer()
    for name in ("q", "k", "v", "gate", "up"):
        xin, want = trace[name]
        got = _lin(layer[name])(quant(xin.to(DEV).view(-1, xin.shape[-1]))).cpu().view(want.shape)
        assert rel_l2(got, want) <= 1e-3, name
    xin, want = trace["o"]
    got = _lin(layer["o"])(kernel.rotate_quant(xin.to(DEV).view(-1, xin.shape[-1]), heads=cfg["heads"])).cpu()
    assert rel_l2(got.view(want.shape), want) <= 1e-3
    xin, want = trace["down"]
    rot = layer["down_rot"]
    got = _lin(layer["down"])(kernel.rotate_quant(xin.to(DEV).view(-1, xin.shape[-1]), rot[1], rot[2],
                                                  sign=layer["down_sign"].to(DEV))).cpu()
    assert rel_l2(got.view(want.shape), want) <= 1e-3

    # teacher-forced layer: every quantizer of the GPU layer is fed the oracle's tensor at that point, so
    # the layer output is the oracle's residual stream plus the GPU's down_proj of the oracle's SwiGLU output
    forced = (trace["x1"].to(torch.float16) + got.view(want.shape)).to(layer["x"].dtype)
    err_forced = rel_l2(forced, want_real)
    assert err_forced <= 1e-3, err_forced

    # free-running layer: a one-ulp difference upstream of a quantizer (RMSNorm's summation order, the
    # attention product) can move codes downstream, so the end-to-end distance is a quantization-noise
    # figure, not a rounding figure; the oracle's own fake-vs-integer gap on this layer is ~8e-3
    got = gpu_layer(layer).cpu()
    assert torch.isfinite(got).all()
    err_real, err_fake = rel_l2(got, want_real), rel_l2(got, want_fake)
    print(f"free-running layer rel-L2: {err_real:.3e} vs integer statement, {err_fake:.3e} vs fake-quant "
          f"(teacher-forced {err_forced:.3e})")
    assert err_real <= 1e-2, err_real
    assert err_fake <= 2e-2, err_fake
