"""The oracle against golden vectors produced by the reference's own Python
(tests/golden/make_golden.py).  CPU only."""
import math

import numpy as np
import pytest
import torch

import oracle
from oracle import fake_quant as fq
from conftest import load_golden, t
from signrot_b200.functional import hadamard as sh
from signrot_b200.functional import hadamard_matrices as hm


def test_pack_unpack_golden():
    g = load_golden("pack.npz")
    q = t(g["q"])
    assert torch.equal(oracle.pack_i4(q.to(torch.int32)), t(g["packed"]))
    assert torch.equal(oracle.unpack_i4(t(g["packed"])), t(g["unpack_i4"]))
    assert torch.equal(oracle.unpack_ui4(t(g["packed"])), t(g["unpack_ui4"]))


@pytest.mark.parametrize("n", [128, 768, 2048, 4096, 14336])
def test_hadamard_butterfly_golden(n):
    """fp32 transform: the oracle's rotation (scale before the had-K factor) and the
    reference butterfly (scale at the end) agree to fp32 rounding."""
    g = load_golden("hadamard.npz")
    x, y = t(g[f"x_{n}"]), t(g[f"y_{n}"])
    hadK, K = sh.get_hadK(n)
    assert K == int(g[f"K_{n}"])
    got = oracle.rotate(x, hadK, K, None, fp32_mode=True)
    assert (got - y).abs().max().item() <= 4e-6 * max(1.0, y.abs().max().item())
    # the product's host-side butterfly is the same function as the reference's
    assert torch.allclose(sh.matmul_hadU(x), y, rtol=0, atol=4e-6 * max(1.0, y.abs().max().item()))


def test_random_hadamard_golden():
    g = load_golden("hadamard.npz")
    torch.manual_seed(7)
    got = sh.random_hadamard_matrix(64, "cpu")
    assert torch.allclose(got, t(g["randhad_64_seed7"]), atol=1e-12)


def test_kv_quant_golden():
    g = load_golden("kv_quant.npz")
    x = t(g["x"])
    q, p = oracle.kv_quant_pack(x)
    assert torch.equal(q, t(g["q"]))
    assert torch.equal(p[..., 0:1], t(g["scale"]))
    assert torch.equal(p[..., 1:2], t(g["zero"]))
    deq = oracle.kv_dequant(q, p)
    # the torch twin dequantizes in fp16, the kernels in fp32: equal to fp16 rounding
    assert torch.allclose(deq, t(g["deq"]).float(), atol=3e-2, rtol=2e-3)


def test_rmsnorm_golden():
    g = load_golden("rmsnorm.npz")
    assert torch.equal(oracle.rmsnorm(t(g["x"]), 1e-5, 256), t(g["y"]))


@pytest.mark.parametrize("tag,sym,clip", [("sym", True, 1.0), ("asym", False, 1.0), ("asym_clip", False, 0.9)])
def test_act_fake_quant_golden(tag, sym, clip):
    g = load_golden("act_fake_quant.npz")
    got = fq.act_fake_quant(t(g["x"]), clip, sym)
    assert torch.equal(got, t(g[tag]))


@pytest.mark.parametrize("tag,mse,sign", [("rtn", False, False), ("rtn_mse", True, False), ("rtn_symgrid", False, True)])
def test_rtn_golden(tag, mse, sign):
    g = load_golden("rtn.npz")
    W = t(g["W"])
    s = torch.ones(W.shape[1], dtype=torch.int8) if sign else None  # all-ones sign: only the grid changes
    Wq, scale = fq.rtn_weight(W, s, mse)
    assert torch.equal(scale, t(g[f"{tag}_scale"]))
    assert torch.equal(Wq, t(g[f"{tag}_wq"]))


CASES = [("plain512_f16", False, None, 0, False), ("plain512_bf16", True, None, 0, False),
         ("full768_adj_f16", False, 768, 0, True), ("full1024_adj_bf16", True, 1024, 0, True),
         ("heads256_f16", False, None, 4, False)]


@pytest.mark.parametrize("tag,bf16,full,heads,adj", CASES)
def test_fake_quant_wrapper_golden(tag, bf16, full, heads, adj):
    """ActQuantWrapper.forward (fake path) incl. the sign derivation and the weight fold."""
    g = load_golden("fake_quant_wrapper.npz")
    x, w0, y = t(g[f"{tag}_x"], bf16), t(g[f"{tag}_w0"], bf16), t(g[f"{tag}_y"], bf16)
    rot = None
    if full:
        hadK, K = sh.get_hadK(full)
        rot = ("full", hadK, K)
    if heads:
        rot = ("heads", heads)
    xr = x
    sign = None
    if adj:
        xr = oracle.rotate(x, rot[1], rot[2], None)
        sign = fq.derive_sign(xr)
        assert torch.equal(sign, t(g[f"{tag}_sign"]))
        assert torch.equal(w0 * sign.to(w0.dtype), t(g[f"{tag}_w1"], bf16))
    # the golden case keeps the fp weight (no RTN): emulate with a FakeLinear whose Wq is the folded weight
    lin = fq.FakeLinear.__new__(fq.FakeLinear)
    lin.rot, lin.sign, lin.clip = rot, sign, 1.0
    lin.Wq = w0 * sign.to(w0.dtype) if sign is not None else w0
    got = lin.fake(x)
    # F.linear accumulates in a different order inside BLAS: compare to fp rounding
    tol = 2e-2 if bf16 else 3e-3
    assert torch.allclose(got.float(), y.float(), atol=tol, rtol=tol)


def test_asym_wrapper_golden():
    g = load_golden("fake_quant_wrapper.npz")
    x, w0, y = t(g["asym512_clip_f16_x"]), t(g["asym512_clip_f16_w0"]), t(g["asym512_clip_f16_y"])
    got = torch.nn.functional.linear(fq.act_fake_quant(x, 0.9, False), w0)
    assert torch.allclose(got.float(), y.float(), atol=3e-3, rtol=3e-3)


def test_tables_are_hadamard():
    for k in hm.ORDERS:
        h = hm.get_had(k).double()
        assert torch.equal(h @ h.T, torch.eye(k, dtype=torch.float64) * k)


def test_real_vs_fake_small_layer():
    """Integer path vs fake-quant path of a small decoder layer in fp16: rel-L2 <= 1e-3."""
    hadK, K = sh.get_hadK(768)
    layer = fq.make_decoder_layer(seed=1, hidden=256, heads=4, kv_heads=2, head_dim=64, ffn=768, tokens=48,
                                  dtype=torch.float16, hadK_ffn=hadK, K_ffn=K, outlier=(15, 33))
    yf = fq.decoder_layer_fake_quant(layer, "fake")
    yr = fq.decoder_layer_fake_quant(layer, "real")
    rel = ((yf.float() - yr.float()).norm() / yr.float().norm()).item()
    assert rel <= 1e-3, rel


@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_quantizer_scale_order_golden(clip):
    """Scales written by the torch statements of the three quantizer modules
    (signrot/nn/quantization.py:23-28, 44-48, 67-76)."""
    g = load_golden("quantizer_scales.npz")
    x = t(g["x"])
    tag = f"clip{int(clip * 100)}"
    # Quantizer: rn_h(amax / 7) first, then * clip -- the order of the fused kernel (fused.cu:83-98)
    _, scale = oracle.sym_quant_dynamic(x, clip)
    assert torch.equal(scale, t(g[f"quantizer_{tag}"]))
    # SymQuantizer applies the clip BEFORE the division
    amax = x.abs().amax(dim=-1).unsqueeze(1) * clip
    assert torch.equal((amax / 7).to(torch.float16), t(g[f"symquantizer_{tag}"]))
    if clip == 1.0:
        assert torch.equal(t(g[f"symquantizer_{tag}"]), scale)
    # AsymQuantizer's torch statement keeps every step in fp16; the kernel order (fused.cu:156-198) is the same
    _, a_scale, a_zero = oracle.asym_quant_dynamic(x, clip)
    assert torch.equal(a_scale, t(g[f"asym_scale_{tag}"]))
    assert torch.equal(a_zero, t(g[f"asym_zero_{tag}"]))


@pytest.mark.parametrize("tag", ["b4t3", "b2t5_shared"])
def test_rope_golden(tag):
    """oracle.rope_qk == HF apply_rotary_pos_emb in fp16, bit for bit
    (benchmarks/test_fused_equivalence.py:102-115)."""
    g = load_golden("rope.npz")
    q, k = oracle.rope_qk(t(g[f"{tag}_q"]), t(g[f"{tag}_k"]), t(g[f"{tag}_cos"]), t(g[f"{tag}_sin"]))
    assert torch.equal(q, t(g[f"{tag}_q_out"]))
    assert torch.equal(k, t(g[f"{tag}_k_out"]))


def test_decode_attention_golden():
    """PagedCacheRef + decode_attention_ref against the reference's fp32 attention over its own dequantized
    paged cache (benchmarks/test_split_decode.py:22-46; signrot/transformers/kv_cache.py:12-73)."""
    g = load_golden("attention.npz")
    k, v, q = t(g["k"]), t(g["v"]), t(g["q"])
    B, T, Hh, _ = k.shape
    ref = oracle.PagedCacheRef(B, 2, Hh, int(g["page"]), 4)
    ref.append(1, k, v)
    kf, vf = ref.dense(1)
    got = oracle.decode_attention_ref(q, kf, vf, hadamard_q=True)
    want = t(g["out"])
    # the reference dequantizes in fp16 (q * scale - zero rounded twice), the oracle and the kernels in fp32
    assert (got - want).abs().max().item() <= 2e-3
    _, indices, last = ref.specs(1)
    assert int(last[0]) == T % int(g["page"]) and indices.numel() == B * ((T + int(g["page"]) - 1) // int(g["page"]))


def test_moe_block_golden():
    """oracle.moe_block against the reference's SignRotMoEBlock.forward run on the CPU (router, stable sort,
    gathers, un-permute and weighted sum are the reference's lines; signrot/nn/moe.py:160-236)."""
    g = load_golden("moe_block.npz")
    x = t(g["x"])
    hidden = x.shape[-1]
    xf = x.view(-1, hidden)
    logits = torch.nn.functional.linear(xf, t(g["gate_w"]))
    assert torch.equal(logits, t(g["logits"]))
    inter = t(g["w_gate"]).shape[1]
    hadK, K = sh.get_hadK(inter)
    got = oracle.moe_block(xf, logits, int(g["top_k"]), True, t(g["w_gate"]), t(g["s_gate"]), t(g["w_up"]), t(g["s_up"]),
                           t(g["w_down"]), t(g["s_down"]), t(g["sign_down"]), hadK, K)
    assert torch.equal(got.view(x.shape), t(g["y"]))
