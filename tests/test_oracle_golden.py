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
