"""Quantizer / dequant / adjacent-op kernels against the CPU oracle, through the C ABI.
Shapes and edge cases follow the reference's own equivalence script
(benchmarks/test_fused_equivalence.py:33-122, benchmarks/test_moe_kernels.py:36-89)."""
import pytest
import torch

import oracle
from conftest import assert_codes_close
from signrot_b200.functional import kernel
from signrot_b200 import nn as snn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _x(rows, cols, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn((rows, cols), generator=g) * scale).half()


def _edge_rows(cols):
    x = _x(8, cols, 3)
    x[0] = 0                      # all-zero row: scale 0, codes 0
    x[1] = 0
    x[1, cols // 2] = 37.5        # single spike
    x[2] *= 1e3
    x[3] *= 1e-4
    x[4] = -x[4].abs()            # all-negative
    x[5] = 1.25                   # constant
    return x


@pytest.mark.parametrize("rows", [1, 8, 16, 2048])
@pytest.mark.parametrize("cols", [4096, 11008, 128, 14336, 72, 1000])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_sym_quant_dynamic(rows, cols, clip):
    if rows == 2048 and cols > 11008:
        rows = 256
    x = _x(rows, cols, rows + cols)
    q, s = kernel.sym_quant_dynamic(x.to(DEV), clip)
    codes, scale = oracle.sym_quant_dynamic(x, clip)
    assert torch.equal(s.cpu(), scale)                      # scales are bit-exact
    assert q.shape == (rows, (cols + 1) // 2) and s.shape == (rows, 1)
    assert_codes_close(oracle.unpack_i4(q.cpu())[:, :cols], codes)


@pytest.mark.parametrize("cols", [4096, 128, 1000])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_asym_quant_dynamic(cols, clip):
    x = _x(64, cols, 5)
    q, s, z = kernel.asym_quant_dynamic(x.to(DEV), clip)
    codes, scale, zero = oracle.asym_quant_dynamic(x, clip)
    assert torch.equal(s.cpu(), scale) and torch.equal(z.cpu(), zero)
    assert_codes_close(oracle.unpack_ui4(q.cpu())[:, :cols], codes)


@pytest.mark.parametrize("cols", [128, 4096])
def test_dynamic_quant_edge_rows(cols):
    x = _edge_rows(cols)
    q, s = kernel.sym_quant_dynamic(x.to(DEV))
    codes, scale = oracle.sym_quant_dynamic(x)
    assert torch.equal(s.cpu(), scale)
    assert_codes_close(oracle.unpack_i4(q.cpu()), codes, frac=1e-3)
    assert int(oracle.unpack_i4(q.cpu())[0].abs().max()) == 0
    xa = x[2:]  # the asymmetric reference divides by zero on all-zero/constant rows
    xa = xa[[0, 1, 2, 4, 5]]
    q, s, z = kernel.asym_quant_dynamic(xa.to(DEV))
    codes, scale, zero = oracle.asym_quant_dynamic(xa)
    assert torch.equal(s.cpu(), scale) and torch.equal(z.cpu(), zero)
    assert_codes_close(oracle.unpack_ui4(q.cpu()), codes, frac=1e-3)


def test_quantizer_modules_fused_vs_unfused():
    """nn.Quantizer / AsymQuantizer: the fused kernel against the unfused chain (range from the tensor
    library, then the given-scale quantizer kernels), bit-exact: the criterion and the chain of
    benchmarks/test_fused_equivalence.py:65-74 and signrot/nn/quantization.py:23-28, 67-76."""
    for rows, cols in [(1, 4096), (8, 11008), (16, 128), (2048, 4096)]:
        x = _x(rows, cols, 11).to(DEV)
        for clip in (1.0, 0.9):
            a = snn.Quantizer(clip_ratio=clip)(x)
            scales = (x.abs().amax(dim=-1).unsqueeze(1) / 7).to(torch.float16) * clip
            assert torch.equal(a.scales_x, scales) and torch.equal(a.quantized_x, kernel.sym_quant(x, scales))
        a = snn.AsymQuantizer()(x)
        lo, hi = x.amin(dim=-1, keepdim=True), x.amax(dim=-1, keepdim=True)
        scales = (hi - lo) / 15
        zeros = (-lo / scales).round()
        assert torch.equal(a.scales_x, scales) and torch.equal(a.zeros_x, zeros.to(torch.int8))
        assert torch.equal(a.quantized_x, kernel.asym_quant_f16_ui4(x, scales, zeros))
    # SymQuantizer applies the clip before the division
    x = _x(9, 512, 3).to(DEV)
    b = snn.SymQuantizer(clip_ratio=0.9)(x)
    want = (x.abs().amax(dim=-1, keepdim=True) * 0.9 / 7).to(torch.float16)
    assert torch.equal(b.scales_x, want) and torch.equal(b.quantized_x, kernel.sym_quant(x, want))
    c = snn.SymQuantizer()(x)
    d = snn.Quantizer()(x)
    assert torch.equal(c.quantized_x, d.quantized_x) and torch.equal(c.scales_x, d.scales_x)


def test_given_scale_quantizers():
    x = _x(33, 250, 2)
    scale = (x.abs().amax(dim=-1, keepdim=True).float() / 7).half()
    q = kernel.sym_quant(x.to(DEV), scale.to(DEV))
    assert_codes_close(oracle.unpack_i4(q.cpu()), oracle.sym_quant_codes(x, scale))
    zero = torch.full_like(scale, 3.0)
    qs = kernel.asym_quant_f16_si4(x.to(DEV), scale.to(DEV), zero.to(DEV))
    qu = kernel.asym_quant_f16_ui4(x.to(DEV), scale.to(DEV), zero.to(DEV))
    assert_codes_close(oracle.unpack_i4(qs.cpu()), oracle.asym_quant_codes(x, scale, zero, -8, 7))
    assert_codes_close(oracle.unpack_ui4(qu.cpu()), oracle.asym_quant_codes(x, scale, zero, 0, 15))


@pytest.mark.parametrize("rows,cols", [(1, 4096), (37, 14336), (16, 40), (2048, 1024)])
def test_sym_dequant(rows, cols):
    g = torch.Generator().manual_seed(rows)
    acc = torch.randint(-900000, 900000, (rows, cols), generator=g, dtype=torch.int32)
    sr = (torch.rand((rows, 1), generator=g) * 0.5 + 0.01).half()
    sc = (torch.rand((cols, 1), generator=g) * 0.009 + 0.001).half()
    out = kernel.sym_dequant(acc.to(DEV), sr.to(DEV), sc.to(DEV))
    assert torch.equal(out.cpu(), oracle.sym_dequant(acc, sr, sc))


def test_moe_quant_and_dequant():
    g = torch.Generator().manual_seed(9)
    E, rows, cols = 5, 70, 768
    x = _x(rows, cols, 4)
    sign = (torch.randint(0, 2, (E, cols), generator=g) * 2 - 1).to(torch.int8)
    eid = torch.randint(0, E, (rows,), generator=g).sort().values.to(torch.int32)
    q, s = kernel.sym_quant_dynamic_moe(x.to(DEV), sign.to(DEV), eid.to(DEV))
    codes, scale = oracle.sym_quant_dynamic(x, 1.0, sign, eid)
    assert torch.equal(s.cpu(), scale)
    assert_codes_close(oracle.unpack_i4(q.cpu()), codes)
    # == sign multiply followed by the plain kernel (benchmarks/test_moe_kernels.py:36-49)
    q2, s2 = kernel.sym_quant_dynamic((x * sign[eid.long()]).to(DEV))
    assert torch.equal(q, q2) and torch.equal(s, s2)
    q, s, z = kernel.asym_quant_dynamic_moe(x.to(DEV), sign.to(DEV), eid.to(DEV), 0.9)
    codes, scale, zero = oracle.asym_quant_dynamic(x, 0.9, sign, eid)
    assert torch.equal(s.cpu(), scale) and torch.equal(z.cpu(), zero)
    assert_codes_close(oracle.unpack_ui4(q.cpu()), codes)
    q0, s0 = kernel.sym_quant_dynamic_moe(x.to(DEV), None, eid.to(DEV))
    q1, s1 = kernel.sym_quant_dynamic(x.to(DEV))
    assert torch.equal(q0, q1) and torch.equal(s0, s1)

    acc = torch.randint(-50000, 50000, (rows, 96), generator=g, dtype=torch.int32)
    ws = (torch.rand((E, 96), generator=g) * 0.01).half()
    wsum = torch.randint(-300, 300, (E, 96), generator=g, dtype=torch.int32)
    zr = torch.randint(0, 16, (rows,), generator=g).to(torch.int8)
    sr = (torch.rand((rows, 1), generator=g) + 0.1).half()
    out = kernel.sym_dequant_moe(acc.to(DEV), sr.to(DEV), ws.to(DEV), eid.to(DEV), zr.to(DEV), wsum.to(DEV))
    assert torch.equal(out.cpu(), oracle.sym_dequant_moe(acc, sr, ws, eid, zr, wsum))
    out = kernel.sym_dequant_moe(acc.to(DEV), sr.to(DEV), ws.to(DEV), eid.to(DEV))
    assert torch.equal(out.cpu(), oracle.sym_dequant_moe(acc, sr, ws, eid))


def test_sum_i4_and_colrow():
    g = torch.Generator().manual_seed(1)
    p = torch.randint(0, 256, (19, 333), generator=g, dtype=torch.uint8)
    assert torch.equal(kernel.sum_i4(p.to(DEV)).cpu(), oracle.sum_i4(p, True))
    assert torch.equal(kernel.sum_i4(p.to(DEV), is_signed=False).cpu(), oracle.sum_i4(p, False))
    a = torch.randint(-128, 128, (11, 1), generator=g).to(torch.int8)
    b = torch.randint(-10000, 10000, (1, 77), generator=g, dtype=torch.int32)
    assert torch.equal(kernel.matmul_colrow_i8_i32(a.to(DEV), b.to(DEV)).cpu(), oracle.matmul_colrow(a, b))


def test_kv_quant_pack():
    x = _x(2 * 5 * 8, 128, 6).view(2, 5, 8, 128)
    x[0, 0, 0] = 0.5  # constant vector
    q, p = kernel.kv_quant_pack(x.to(DEV))
    oq, op = oracle.kv_quant_pack(x)
    assert torch.equal(q.cpu(), oq) and torch.equal(p.cpu(), op)
    x = _x(6, 96, 7)
    q, p = kernel.kv_quant_pack(x.to(DEV))
    oq, op = oracle.kv_quant_pack(x)
    assert torch.equal(q.cpu(), oq) and torch.equal(p.cpu(), op)


@pytest.mark.parametrize("rows,cols", [(1, 4096), (5, 11008), (64, 128), (3, 100)])
def test_rmsnorm(rows, cols):
    x = _x(rows, cols, 8)
    y = kernel.rmsnorm(x.to(DEV), 1e-5, cols).cpu()
    want = oracle.rmsnorm(x, 1e-5, cols)
    # the row sum is reduced in a different order: within one fp16 ulp (test_fused_equivalence.py:92-100)
    ulp = (want.float().abs() * 2 ** -10).clamp_min(2 ** -24)
    assert bool(((y.float() - want.float()).abs() <= ulp).all())
    assert torch.equal(snn.RMSNorm(cols)(x.to(DEV)).cpu(), y)


@pytest.mark.parametrize("B,T,Hq,Hk,D,cb", [(2, 5, 4, 2, 128, 1), (1, 1, 32, 8, 128, 1), (3, 2, 2, 2, 64, 3), (1, 3, 1, 1, 6, 1)])
def test_rope_qk(B, T, Hq, Hk, D, cb):
    g = torch.Generator().manual_seed(B * T)
    q = torch.randn((B, T, Hq, D), generator=g).half()
    k = torch.randn((B, T, Hk, D), generator=g).half()
    ang = torch.rand((cb, T, D), generator=g) * 6.28
    cos, sin = ang.cos().half(), ang.sin().half()
    wq, wk = oracle.rope_qk(q, k, cos.expand(B, T, D) if cb == 1 else cos, sin.expand(B, T, D) if cb == 1 else sin)
    gq, gk = q.clone().to(DEV), k.clone().to(DEV)
    kernel.rope_qk(gq, gk, cos.to(DEV), sin.to(DEV))
    assert torch.equal(gq.cpu(), wq) and torch.equal(gk.cpu(), wk)


def test_swiglu():
    g = torch.Generator().manual_seed(3)
    a = (torch.randn((7, 1001), generator=g) * 3).half()
    b = torch.randn((7, 1001), generator=g).half()
    y = kernel.swiglu(a.to(DEV), b.to(DEV)).cpu()
    want = oracle.swiglu(a, b)
    # expf on the GPU and exp on the CPU may differ in the last bit before the fp16 rounding
    d = (y.float() - want.float()).abs()
    assert bool((d <= want.float().abs() * 2 ** -10 + 1e-7).all())
    assert (y != want).float().mean().item() < 1e-3


@pytest.mark.parametrize("rows,cols", [(1, 4096), (16, 4096), (37, 512), (300, 2048), (5, 14336), (3, 8192)])
@pytest.mark.parametrize("with_delta", [True, False])
@pytest.mark.parametrize("asym", [False, True])
def test_add_rmsnorm_quant_equals_the_three_launches(rows, cols, with_delta, asym):
    """The fused residual add + RMSNorm + quantizer gives the bits of `x + delta`, `rmsnorm`,
    `sym/asym_quant_dynamic` run one after the other."""
    x = _x(rows, cols, seed=rows + cols).to(DEV)
    delta = _x(rows, cols, seed=7, scale=0.5).to(DEV) if with_delta else None
    total, packed, normed = kernel.add_rmsnorm_quant(x, delta, 1e-5, cols, clip_ratio=0.9 if asym else 1.0,
                                                      asym=asym, return_normed=True)
    want_total = x + delta if with_delta else x
    want_normed = kernel.rmsnorm(want_total, 1e-5, cols)
    assert torch.equal(total, want_total) and torch.equal(normed, want_normed)
    if asym:
        q, s, z = kernel.asym_quant_dynamic(want_normed, 0.9)
        assert torch.equal(packed.zeros_x, z.to(torch.int8))
    else:
        q, s = kernel.sym_quant_dynamic(want_normed, 1.0)
        assert packed.zeros_x is None
    assert torch.equal(packed.quantized_x, q) and torch.equal(packed.scales_x, s)
    # and the oracle's statement of the normalisation (row sum reduced in another order: one fp16 ulp)
    want_h = oracle.rmsnorm(want_total.cpu(), 1e-5, cols)
    ulp = (want_h.float().abs() * 2 ** -10).clamp_min(2 ** -24)
    assert bool(((normed.cpu().float() - want_h.float()).abs() <= ulp).all())


def test_add_rmsnorm_quant_rejects_odd_widths():
    x = _x(2, 100).to(DEV)
    with pytest.raises(RuntimeError):
        kernel.add_rmsnorm_quant(x, None, 1e-5, 100)
