"""Offline weight preparation on the GPU (RTN + SignRot sign refold + packing in one kernel, exact
Hadamard fold through the library's fp32 transform) against the oracle's statement of
rtn_fwrd / WeightQuantizer / Linear4bit.from_float."""
import pytest
import torch

import oracle
from oracle import fake_quant as fq
from signrot_b200 import nn as snn
from signrot_b200.functional import hadamard as sh
from signrot_b200.functional import kernel
from signrot_b200.functional import quantization as qz
from signrot_b200.nn.linear import linear4bit_from_float_rtn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(n, k, dtype, seed, with_sign):
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn((n, k), generator=g) * 0.02).to(dtype)
    W[0] = 0                                   # an all-zero channel: scale clamps at 1e-5 / 7
    if n > 2:
        W[1, :] = W[1, :].abs()                # one-sided channel
    sign = (torch.randint(0, 2, (k,), generator=g) * 2 - 1).to(torch.int8) if with_sign else None
    return W, sign


def _oracle_codes(W, sign, mse):
    Wq, scale = fq.rtn_weight(W, sign, mse)
    s16 = scale.to(torch.float16)
    codes = (Wq.to(torch.float16) / s16).round().to(torch.int32)
    return codes, s16


@pytest.mark.parametrize("n,k", [(64, 256), (48, 14336), (333, 768), (5, 4096)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("with_sign", [False, True])
def test_rtn_pack_matches_oracle(n, k, dtype, with_sign):
    W, sign = _case(n, k, dtype, n + k, with_sign)
    want_codes, want_scale = _oracle_codes(W, sign, False)
    packed, scale = kernel.rtn_pack(W.to(DEV), sign.to(DEV) if with_sign else None)
    assert torch.equal(scale.cpu(), want_scale)
    assert torch.equal(packed.cpu(), oracle.pack_i4(want_codes))
    if with_sign:
        assert int(qz.unpack_i4(packed).min()) >= -7     # the refolded grid is symmetric


@pytest.mark.parametrize("with_sign", [False, True])
def test_rtn_pack_mse_search(with_sign):
    W, sign = _case(256, 1024, torch.bfloat16, 3, with_sign)
    want_codes, want_scale = _oracle_codes(W, sign, True)
    packed, scale = kernel.rtn_pack(W.to(DEV), sign.to(DEV) if with_sign else None, mse=True)
    same = (scale.cpu() == want_scale).view(-1)
    # candidates whose fp32 error sums tie within summation noise may swap: rare
    assert same.float().mean() >= 0.98
    got_codes = qz.unpack_i4(packed).cpu().to(torch.int32)
    assert torch.equal(got_codes[same], want_codes[same])
    plain_scale = kernel.rtn_pack(W.to(DEV), sign.to(DEV) if with_sign else None)[1]
    assert (scale <= plain_scale).all() and (scale < plain_scale).any()   # the search only shrinks


def test_linear_from_float_rtn_runs_the_same_gemm():
    k, n = 768, 512
    W, sign = _case(n, k, torch.float16, 9, True)
    lin = torch.nn.Linear(k, n, bias=False, dtype=torch.float16)
    lin.weight.data = W * sign.to(W.dtype)         # the sign is already folded into the stored weight
    q4 = linear4bit_from_float_rtn(lin.to(DEV), sign=sign.to(DEV))
    ref = fq.FakeLinear(W, sign=sign)              # folds the sign itself
    assert torch.equal(q4.weight.cpu(), ref.w_packed) and torch.equal(q4.weight_scales.cpu(), ref.w_scale)
    x = torch.randn((9, k), generator=torch.Generator().manual_seed(1)).half()
    got = q4(snn.Quantizer()(x.to(DEV))).cpu()
    codes, s = oracle.sym_quant_dynamic(x, 1.0)
    want = oracle.w4a4_linear(oracle.pack_codes(codes), s, ref.w_packed, ref.w_scale)
    assert torch.equal(got, want)


@pytest.mark.parametrize("features,output,had_dim", [((512, 768), False, -1), ((768, 512), True, -1), ((512, 512), True, 128)])
def test_exact_hadamard_fold_on_gpu_matches_cpu(features, output, had_dim):
    in_f, out_f = features
    g = torch.Generator().manual_seed(in_f + out_f)
    W = torch.randn((out_f, in_f), generator=g) * 0.02
    a = torch.nn.Linear(in_f, out_f, bias=False)
    b = torch.nn.Linear(in_f, out_f, bias=False)
    a.weight.data = W.clone()
    b.weight.data = W.clone().to(DEV)
    sh.apply_exact_had_to_linear(a, had_dim=had_dim, output=output)
    sh.apply_exact_had_to_linear(b, had_dim=had_dim, output=output)
    assert torch.allclose(a.weight.data, b.weight.data.cpu(), rtol=0, atol=2e-6)
