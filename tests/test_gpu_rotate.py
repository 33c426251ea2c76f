"""Online rotation (+ sign + quantizer) against the oracle.  The rotated fp16 row may differ
from the oracle by one fp16 ulp where two fp32 summation orders round differently; codes may
differ only by +-1 in at most 1e-4 of the elements."""
import pytest
import torch

import oracle
from conftest import assert_act_quant_matches
from signrot_b200.functional import kernel
from signrot_b200.functional.hadamard import get_hadK, matmul_hadU_cuda
from signrot_b200 import nn as snn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _x(rows, n, seed, dtype=torch.float16, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((rows, n), generator=g)
    if outliers:
        x[:, 3] *= 100.0
        x[rows // 2, :] *= 30.0
    return x.to(dtype)


def _ulp_close(got, want, ulps=1.0):
    """One fp16 ulp of the value, or (for outputs that are tiny next to the row's largest ones)
    the fp32 rounding noise of a different summation order: 2^-17 of the row maximum."""
    g, w = got.float(), want.float()
    tol = (w.abs() * 2 ** -10).clamp_min(2 ** -24) * ulps + w.abs().amax(dim=-1, keepdim=True) * 2 ** -17
    bad = (g - w).abs() > tol
    # Kronecker shapes round twice (after the Walsh-Hadamard stage and after the had-K stage): a
    # one-ulp difference in one intermediate value moves the K outputs that sum it by one ulp of
    # the INTERMEDIATE (up to 2^-10 of the row maximum), however small those outputs are.  Such
    # events are a few per hundred thousand values (tensor-core sums round differently from the
    # reference's butterflies; the bound is the one the code comparison uses, 1e-4).
    assert bad.float().mean().item() <= 1e-4, f"{int(bad.sum())} values differ by more than {ulps} ulp"
    worst = ((g - w).abs() - tol).clamp_min(0) / w.abs().amax(dim=-1, keepdim=True).clamp_min(1e-30)
    assert worst.max().item() <= 2 ** -9, "a value is off by more than one ulp of an intermediate"
    return (g != w).float().mean().item()


@pytest.mark.parametrize("n", [32, 128, 512, 768, 1024, 4096, 8192, 14336, 2560])
@pytest.mark.parametrize("rows", [1, 19])
def test_hadamard_f16(n, rows):
    x = _x(rows, n, n + rows)
    hadK, K = get_hadK(n)
    got = matmul_hadU_cuda(x.to(DEV), hadK, K).cpu()
    want = oracle.rotate(x, hadK, K)
    frac = _ulp_close(got, want)
    assert frac < 2e-2


@pytest.mark.parametrize("n,dtype", [(4096, torch.bfloat16), (768, torch.float32), (14336, torch.float32), (128, torch.bfloat16)])
def test_hadamard_other_dtypes(n, dtype):
    x = _x(5, n, n, dtype)
    hadK, K = get_hadK(n)
    got = matmul_hadU_cuda(x.to(DEV), hadK, K).cpu()
    want = oracle.rotate(x, hadK, K)
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=1e-5 * want.abs().max().item(), rtol=1e-5)
    else:
        g, w = got.float(), want.float()
        assert bool(((g - w).abs() <= w.abs() * 2 ** -7 + 1e-30).all())


@pytest.mark.parametrize("n", [768, 4096, 14336])
@pytest.mark.parametrize("fp32", [False, True])
def test_online_hadamard_module_with_sign(n, fp32):
    g = torch.Generator().manual_seed(n)
    x = _x(9, n, 1)
    sign = (torch.randint(0, 2, (n,), generator=g) * 2 - 1).to(torch.int8)
    mod = snn.OnlineHadamard(n, force_fp32=fp32, had_adj=True).to(DEV)
    mod.had_adj_sign = sign.to(DEV)
    got = mod(x.to(DEV)).cpu()
    hadK, K = get_hadK(n)
    want = oracle.rotate(x, hadK, K, sign, fp32_mode=fp32)
    assert got.dtype == torch.float16
    _ulp_close(got, want)


def test_online_hadamard_rejects_unset_sign():
    mod = snn.OnlineHadamard(128, had_adj=True).to(DEV)
    mod.had_adj_sign.zero_()
    with pytest.raises(RuntimeError, match="not implemented"):
        mod(torch.zeros(2, 128, dtype=torch.float16, device=DEV))


@pytest.mark.parametrize("heads,dim", [(32, 128), (4, 64), (8, 16)])
def test_hadamard_heads(heads, dim):
    x = _x(7, heads * dim, heads)
    got = kernel.hadamard_heads(x.to(DEV), heads).cpu()
    _ulp_close(got, oracle.rotate_heads(x, heads))


@pytest.mark.parametrize("M,n", [(1, 4096), (16, 4096), (256, 4096), (1, 14336), (16, 14336), (200, 14336),
                                 (33, 768), (64, 128), (5, 2048)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rotate_quant(M, n, dtype):
    """The fused kernel on the op-sweep input distribution (bf16 ~N(0,1), 0.1 % channels x100)."""
    from oracle import fake_quant as fq
    case = fq.make_linear_case(M, n, 8, seed=M)
    x, sign = case["x"].to(dtype), case["sign"]
    hadK, K = get_hadK(n)
    pk, rot = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV), return_rotated=True)
    want_rot = oracle.rotate(x, hadK, K, sign, cast_in_to_f16=True, out_dtype=torch.float16)
    _ulp_close(rot.cpu(), want_rot)
    # every row: scale equal or adjacent to the oracle's, codes within the tie rule for the scale written
    assert_act_quant_matches(pk.quantized_x, pk.scales_x, want_rot)
    # self-consistency: codes are exactly the quantizer applied to the kernel's own rotated rows
    q2, s2 = kernel.sym_quant_dynamic(rot)
    assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
    # the launch that does not return the rotated rows takes a different code path (sign applied to the codes)
    pk3 = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV))
    assert torch.equal(pk3.quantized_x, pk.quantized_x) and torch.equal(pk3.scales_x, pk.scales_x)


@pytest.mark.parametrize("n", [4096, 14336])
def test_rotate_quant_benchmark_size_against_oracle(n):
    """The benchmarked launch (4096 token rows, bf16 activations of the op-sweep distribution): rotated
    rows, scales and codes of EVERY row against the oracle."""
    from oracle import fake_quant as fq
    case = fq.make_linear_case(4096, n, 8, seed=4096)
    x, sign = case["x"].to(torch.bfloat16), case["sign"]
    hadK, K = get_hadK(n)
    pk, rot = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV), return_rotated=True)
    pk3 = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV))     # the benchmarked launch itself
    assert torch.equal(pk3.quantized_x, pk.quantized_x) and torch.equal(pk3.scales_x, pk.scales_x)
    want_rot = oracle.rotate(x, hadK, K, sign, cast_in_to_f16=True, out_dtype=torch.float16)
    _ulp_close(rot.cpu(), want_rot)
    assert_act_quant_matches(pk.quantized_x, pk.scales_x, want_rot)


def test_rotate_quant_tiny_rows_take_the_clamped_path():
    """Rows whose scale is a subnormal fp16 number (quotients can exceed the code range) and all-zero rows."""
    for n in (4096, 14336):
        x = _x(9, n, 21, torch.float16, outliers=False) * 1e-5
        x[4] = 0
        sign = (torch.randint(0, 2, (n,), generator=torch.Generator().manual_seed(8)) * 2 - 1).to(torch.int8)
        hadK, K = get_hadK(n)
        pk, rot = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV), return_rotated=True)
        q2, s2 = kernel.sym_quant_dynamic(rot)
        assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
        pk3 = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV))
        assert torch.equal(pk3.quantized_x, pk.quantized_x) and torch.equal(pk3.scales_x, pk.scales_x)


def test_rotate_quant_asym_heads_and_clip():
    x = _x(12, 4096, 5, torch.bfloat16)
    pk, rot = kernel.rotate_quant(x.to(DEV), heads=32, asym=True, clip_ratio=0.9, return_rotated=True)
    want_rot = oracle.rotate_heads(x, 32, cast_in_to_f16=True)
    _ulp_close(rot.cpu(), want_rot)
    q2, s2, z2 = kernel.asym_quant_dynamic(rot, 0.9)
    assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
    assert torch.equal(z2.to(torch.int8), pk.zeros_x)


@pytest.mark.parametrize("n,rows,sorted_rows", [(768, 21, False), (14336, 300, True), (14336, 37, False), (4096, 50, True)])
def test_rotate_quant_expert_signs(n, rows, sorted_rows):
    """Per-row sign tables (MoE down_proj): the fused kernel against rotation followed by the expert-indexed
    quantizer, with and without the rotated rows as a second output (the two take different code paths for
    n = 14336: sign on the packed codes, sign on the values)."""
    g = torch.Generator().manual_seed(2)
    E = 4
    x = _x(rows, n, 9)
    sign = (torch.randint(0, 2, (E, n), generator=g) * 2 - 1).to(torch.int8)
    eid = torch.randint(0, E, (rows,), generator=g).to(torch.int32)
    if sorted_rows:
        eid = eid.sort()[0]
    hadK, K = get_hadK(n)
    pk = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV), expert_ids=eid.to(DEV))
    pk2, rot = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV), expert_ids=eid.to(DEV), return_rotated=True)
    assert torch.equal(pk.quantized_x, pk2.quantized_x) and torch.equal(pk.scales_x, pk2.scales_x)
    q2, s2 = kernel.sym_quant_dynamic(rot)
    assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
    if n == 768:   # generic kernel: same rounding points as the separate rotation
        h = kernel.hadamard(x.to(DEV), hadK, K)
        q3, s3 = kernel.sym_quant_dynamic_moe(h, sign.to(DEV), eid.to(DEV))
        assert torch.equal(q3, pk.quantized_x) and torch.equal(s3, pk.scales_x)
    want = oracle.rotate(x, hadK, K, None, cast_in_to_f16=True, out_dtype=torch.float16) * sign[eid.long()].to(torch.float16)
    _ulp_close(rot.cpu(), want)


@pytest.mark.parametrize("n,with_ids", [(14336, True), (14336, False), (4096, True), (4096, False)])
def test_rows_of_arbitrary_bits_do_not_touch_their_neighbours(n, with_ids):
    """An expert-parallel MoE block hands the rotation a buffer in which the rows of other ranks' experts were never
    written: whatever they hold (NaN, infinities), the rows in between must come out as if those rows were zeros.
    (Calls with per-row sign tables are the ones that see such buffers; the same holds without them: one request's
    overflow must not reach another request's tokens.)"""
    g = torch.Generator().manual_seed(31)
    rows, E = 96, 4
    x = _x(rows, n, 13)
    bad = torch.zeros(rows, dtype=torch.bool)
    bad[5:9] = True
    bad[40] = True
    bad[70:96:3] = True
    clean = x.clone()
    clean[bad] = 0
    dirty = x.clone()
    dirty[bad] = float("nan")
    dirty[6, ::2] = float("inf")
    sign = (torch.randint(0, 2, (E, n), generator=g) * 2 - 1).to(torch.int8)
    eid = torch.sort(torch.randint(0, E, (rows,), generator=g)).values.to(torch.int32)
    hadK, K = get_hadK(n)
    kw = dict(sign=sign.to(DEV), expert_ids=eid.to(DEV)) if with_ids else dict(sign=sign[0].to(DEV))
    a = kernel.rotate_quant(clean.to(DEV), hadK, K, **kw)
    b = kernel.rotate_quant(dirty.to(DEV), hadK, K, **kw)
    good = ~bad
    assert torch.equal(a.quantized_x.cpu()[good], b.quantized_x.cpu()[good])
    assert torch.equal(a.scales_x.cpu()[good], b.scales_x.cpu()[good])


def test_rotation_is_orthogonal_at_full_size():
    """Size-independent property at the benchmark size: ||H x|| = ||x|| and H(H x) = x
    (had28 is symmetric, so the Kronecker transform is an involution as well)."""
    for n in (4096, 14336):
        x = _x(4096, n, 3, outliers=False).to(DEV)
        hadK, K = get_hadK(n)
        y = kernel.hadamard(x.float(), hadK, K)
        assert torch.allclose(y.norm(dim=-1), x.float().norm(dim=-1), rtol=1e-4)
        z = kernel.hadamard(y, hadK, K)
        assert torch.allclose(z, x.float(), atol=2e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_rotate_quant_4096_asym_full_width(dtype, clip):
    """Full-width rotation with asymmetric codes (the tensor-core kernel's second code path)."""
    x = _x(37, 4096, 11, dtype)
    sign = (torch.randint(0, 2, (4096,), generator=torch.Generator().manual_seed(5)) * 2 - 1).to(torch.int8)
    pk, rot = kernel.rotate_quant(x.to(DEV), None, 1, sign=sign.to(DEV), asym=True, clip_ratio=clip,
                                  return_rotated=True)
    want_rot = oracle.rotate(x, None, 1, sign, cast_in_to_f16=True, out_dtype=torch.float16)
    _ulp_close(rot.cpu(), want_rot)
    q2, s2, z2 = kernel.asym_quant_dynamic(rot, clip)
    assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
    assert torch.equal(z2.to(torch.int8), pk.zeros_x)


@pytest.mark.parametrize("rows", [300, 4096])
def test_rotate_quant_4096_many_rows_self_consistent(rows):
    """Every row of a launch that keeps all SMs busy for several rounds: the packed codes are
    exactly the stand-alone quantizer applied to the rotated rows the same launch wrote, and
    those rows equal the stand-alone rotation."""
    x = _x(rows, 4096, 13, torch.bfloat16).to(DEV)
    sign = (torch.randint(0, 2, (4096,), generator=torch.Generator().manual_seed(6)) * 2 - 1).to(torch.int8).to(DEV)
    pk, rot = kernel.rotate_quant(x, None, 1, sign=sign, return_rotated=True)
    q2, s2 = kernel.sym_quant_dynamic(rot)
    assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
    pk2 = kernel.rotate_quant(x, None, 1, sign=sign)
    assert torch.equal(pk2.quantized_x, pk.quantized_x) and torch.equal(pk2.scales_x, pk.scales_x)
    ref = kernel.hadamard(x.half(), None, 1) * sign.to(torch.float16)
    diff = (rot.float() - ref.float()).abs()
    tol = rot.float().abs() * 2.0 ** -10 + rot.float().abs().amax(dim=-1, keepdim=True) * 2.0 ** -17
    assert (diff > tol).float().mean().item() <= 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows", [1, 37, 600])
def test_rotate_quant_heads32_symmetric(dtype, rows):
    """Head-wise rotation of a 32-head, head_dim-128 row (the o_proj input) with symmetric codes:
    the tensor-core kernel against the oracle and against the stand-alone quantizer."""
    x = _x(rows, 4096, 17 + rows, dtype)
    pk, rot = kernel.rotate_quant(x.to(DEV), heads=32, return_rotated=True)
    want_rot = oracle.rotate_heads(x, 32, cast_in_to_f16=True)
    _ulp_close(rot.cpu(), want_rot)
    q2, s2 = kernel.sym_quant_dynamic(rot)
    assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
    pk3 = kernel.rotate_quant(x.to(DEV), heads=32)
    assert torch.equal(pk3.quantized_x, pk.quantized_x) and torch.equal(pk3.scales_x, pk.scales_x)
    assert_act_quant_matches(pk.quantized_x, pk.scales_x, want_rot)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_rotate_quant_had28_asym(dtype, clip):
    """had28 x 512 rotation with asymmetric codes (zero padding rows of the 28 -> 32 product must not enter the range)."""
    n = 14336
    x = _x(21, n, 31, dtype)
    x = (x.float() + 0.75).to(dtype)          # a range that is not symmetric around zero
    sign = (torch.randint(0, 2, (n,), generator=torch.Generator().manual_seed(9)) * 2 - 1).to(torch.int8)
    hadK, K = get_hadK(n)
    pk, rot = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV), asym=True, clip_ratio=clip, return_rotated=True)
    want_rot = oracle.rotate(x, hadK, K, sign, cast_in_to_f16=True, out_dtype=torch.float16)
    _ulp_close(rot.cpu(), want_rot)
    q2, s2, z2 = kernel.asym_quant_dynamic(rot, clip)
    assert torch.equal(q2, pk.quantized_x) and torch.equal(s2, pk.scales_x)
    assert torch.equal(z2.to(torch.int8), pk.zeros_x)
    pk3 = kernel.rotate_quant(x.to(DEV), hadK, K, sign=sign.to(DEV), asym=True, clip_ratio=clip)
    assert torch.equal(pk3.quantized_x, pk.quantized_x) and torch.equal(pk3.zeros_x, pk.zeros_x)
