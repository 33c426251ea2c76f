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
