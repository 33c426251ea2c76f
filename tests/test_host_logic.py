"""Host-side pieces of the package that need no GPU: packing, Hadamard tables and butterfly,
module construction, state-dict names, offline weight preparation."""
import numpy as np
import pytest
import scipy.linalg
import torch

import oracle
import signrot_b200
from signrot_b200 import functional as F
from signrot_b200.functional import hadamard as sh
from signrot_b200.functional import quantization as qz


def test_pack_unpack_roundtrip_and_oracle_agreement():
    q = torch.randint(-8, 8, (7, 96), dtype=torch.int8)
    p = qz.pack_i4(q)
    assert p.dtype == torch.uint8 and p.shape == (7, 48)
    assert torch.equal(p, oracle.pack_i4(q.to(torch.int32)))
    assert torch.equal(qz.unpack_i4(p).to(torch.int8), q)
    assert torch.equal(qz.unpack_ui4(p), oracle.unpack_ui4(p))
    with pytest.raises(AssertionError):
        qz.pack_i4(torch.tensor([[9, 0]], dtype=torch.int8))


@pytest.mark.parametrize("n,K", [(4096, 1), (128, 1), (32, 1), (14336, 28), (768, 12), (11008, 172), (5120, 40)])
def test_get_hadK(n, K):
    h, k = sh.get_hadK(n)
    assert k == K
    assert (h is None) == (K == 1)


def test_get_hadK_rejects_unknown():
    with pytest.raises(AssertionError):
        sh.get_hadK(3 * 50)


@pytest.mark.parametrize("n", [64, 96, 224])
def test_matmul_hadU_is_kronecker_product(n):
    x = torch.randn(3, n, dtype=torch.float64)
    hadK, K = sh.get_hadK(n)
    Hs = torch.from_numpy(scipy.linalg.hadamard(n // K).astype(np.float64))
    full = torch.kron(hadK.double(), Hs) if K > 1 else Hs
    want = x @ full.T / np.sqrt(n)
    assert torch.allclose(sh.matmul_hadU(x), want, atol=1e-12)


def test_module_buffers_and_names():
    lin = signrot_b200.nn.Linear4bit(64, 32, bias=True)
    sd = lin.state_dict()
    assert set(sd) == {"weight_scales", "weight", "bias"}
    assert sd["weight"].shape == (32, 32) and sd["weight"].dtype == torch.uint8
    had = signrot_b200.nn.OnlineHadamard(768, had_adj=True)
    assert had.rem_dim == 12 and had.had_rem_dim.dtype == torch.float16
    assert set(had.state_dict()) == {"had_rem_dim", "had_adj_sign"}
    assert had.had_adj_sign.dtype == torch.int8
    had2 = signrot_b200.nn.OnlineHadamard(4096, force_fp32=True)
    assert had2.rem_dim == 1 and had2.had_rem_dim is None
    q = signrot_b200.nn.Quantizer(clip_ratio=0.9)
    assert q.clip_ratio == 0.9
    assert int(signrot_b200.nn.AsymQuantizer().maxq) == 15


def test_from_float_packs_rounded_weights_and_float_path():
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 16, bias=False).half()
    scales = (lin.weight.data.abs().amax(dim=1, keepdim=True).float() / 7).half()
    wq = (scales * torch.clamp(torch.round(lin.weight.data / scales), -8, 7)).half()
    lin.weight.data = wq
    q4 = signrot_b200.nn.Linear4bit.from_float(lin, weight_scales=scales)
    codes = qz.unpack_i4(q4.weight)
    assert torch.equal(codes, torch.round(wq / scales).to(torch.int32))
    # float input: dense fallback on the dequantized weight (signrot/nn/linear.py:31-34)
    x = torch.randn(3, 64)
    y = q4.float()(x)
    assert torch.allclose(y, torch.nn.functional.linear(x, codes.float() * scales.float()), atol=1e-5)


def test_apply_exact_had_to_linear():
    lin = torch.nn.Linear(96, 8, bias=False)
    w0 = lin.weight.data.clone().double()
    sh.apply_exact_had_to_linear(lin, had_dim=-1, output=False)
    hadK, K = sh.get_hadK(96)
    Hs = torch.from_numpy(scipy.linalg.hadamard(8).astype(np.float64))
    full = torch.kron(hadK.double(), Hs) / np.sqrt(96)
    assert torch.allclose(lin.weight.data.double(), w0 @ full.T, atol=1e-5)
    lin2 = torch.nn.Linear(8, 64, bias=False)
    w1 = lin2.weight.data.clone().double()
    sh.apply_exact_had_to_linear(lin2, had_dim=16, output=True)
    H16 = torch.from_numpy(scipy.linalg.hadamard(16).astype(np.float64)) / 4
    want = (w1.T.reshape(8, 4, 16) @ H16.T).reshape(8, 64).T
    assert torch.allclose(lin2.weight.data.double(), want, atol=1e-5)


def test_install_as_signrot_aliases():
    import sys
    saved = {k: v for k, v in sys.modules.items() if k == "signrot" or k.startswith("signrot.")}
    try:
        signrot_b200.install_as_signrot()
        import signrot.nn
        import signrot.functional.kernel as k
        assert signrot.nn.Linear4bit is signrot_b200.nn.Linear4bit
        assert k.PackedQuantizedTensor is F.kernel.PackedQuantizedTensor
    finally:
        for k_ in [k for k in sys.modules if k == "signrot" or k.startswith("signrot.")]:
            del sys.modules[k_]
        sys.modules.update(saved)


def test_shared_quantization_rules():
    """Sibling projections share one quantized activation only when neither rotates its input and
    both quantize the same way (fake_quant/quant_utils.py:298-308)."""
    from signrot_b200.transformers import kernel_utils as ku
    cfg = ku.DecoderConfig(hidden_size=512, intermediate_size=1536, num_hidden_layers=1, num_attention_heads=4,
                           num_key_value_heads=2, vocab_size=64)
    layer = ku.KernelDecoderLayer(cfg, 0)
    at, mlp = layer.self_attn, layer.mlp
    assert at.q_proj.shares_kernel_input_with(at.k_proj) and at.q_proj.shares_kernel_input_with(at.v_proj)
    assert mlp.gate_proj.shares_kernel_input_with(mlp.up_proj)
    assert not at.o_proj.shares_kernel_input_with(at.q_proj)        # rotated input
    assert not mlp.down_proj.shares_kernel_input_with(mlp.gate_proj)
    assert not at.q_proj.shares_kernel_input_with(ku.KernelLinear(512, 64, clip_ratio=0.9))
    assert not at.q_proj.shares_kernel_input_with(ku.KernelLinear(512, 64, asym=True))
    assert mlp.down_proj.kernel_hadamard.rem_dim == 12 and mlp.down_proj.kernel_hadamard.had_adj_sign is not None


def test_oracle_decoder_prefill_then_decode_is_consistent():
    """The oracle's stack: decoding token T over a cache of T prompt tokens lands near a prefill of
    T+1 tokens (they differ by the int4 rounding of the cached K/V and by the dense prefill
    attention), and the cache advances by one."""
    import math
    from oracle.decoder import DecoderRef
    from oracle import quant as Q
    from signrot_b200.functional.hadamard import get_hadK
    g = torch.Generator().manual_seed(0)
    hid, ffn, heads, kvh, D, V = 256, 768, 2, 1, 128, 64
    def lin(n, k):
        return (Q.pack_codes(torch.randint(0, 16, (n, k), generator=g).to(torch.int32)),
                ((torch.rand((n, 1), generator=g) * 0.5 + 0.5) / math.sqrt(k) / 4).half())
    L = {}
    for tag, (n, k) in dict(q=(heads * D, hid), k=(kvh * D, hid), v=(kvh * D, hid), o=(hid, heads * D),
                            g=(ffn, hid), u=(ffn, hid), d=(hid, ffn)).items():
        L["w" + tag], L["s" + tag] = lin(n, k)
    L["sign_d"] = (torch.randint(0, 2, (ffn,), generator=g) * 2 - 1).to(torch.int8)
    hadK, K = get_hadK(ffn)
    cfg = dict(hidden=hid, heads=heads, kv_heads=kvh, head_dim=D, ffn=ffn, eps=1e-5, theta=10000.0,
               hadK=hadK.half(), K=K)
    state = {"embed": (torch.randn((V, hid), generator=g)).half(), "lm_head": (torch.randn((V, hid), generator=g) * 0.05).half(),
             "layers": [L]}
    ids = torch.randint(0, V, (1, 9), generator=g)
    a = DecoderRef(state, cfg, 1, 4, 16)
    a.forward(ids[:, :8])
    step = a.forward(ids[:, 8:9])
    b = DecoderRef(state, cfg, 1, 4, 16)
    full = b.forward(ids)
    assert a.length == b.length == 9
    num = (step[:, 0].float() - full[:, 8].float()).norm()
    assert torch.isfinite(step).all() and num / full[:, 8].float().norm() < 0.35
