"""This library's kernels beside the reference's own CUDA kernels, on the same device buffers.

oracle/build_ref.py compiles the reference's extension module (signrot/kernels/*.cu + bindings.cpp, the module
the reference imports as signrot._CUDA) for sm_100a into the git-ignored oracle/_ref/native/; where that file
exists, every export of it that lies on the path is called here with the inputs the reference's own tests and
benchmarks use (benchmarks/test_fused_equivalence.py, test_grouped_gemm.py, test_split_decode.py) and compared
with the entry point that replaces it.  Integer and byte results, and every fp16 result whose rounding points the
reference fixes (quantizer scales and zero points, dequantized outputs, RoPE, SwiGLU, KV parameters), must be equal
bit for bit.  Two results depend on an fp32 summation order that the reference does not fix: RMSNorm (one fp16 ulp
on at most 1e-3 of the values) and decode attention (the reference's own criterion for a split against an unsplit
run, 2e-3).

The module is a checker: nothing in the package imports it.  Without the file (no reference checkout and no
flashinfer wheel at build time) the tests are skipped, and the CPU oracle remains the only checker.
"""
import pytest
import torch

from oracle import build_ref
from signrot_b200.functional import kernel
from signrot_b200.transformers import kv_cache as kvc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load_native()
    if mod is None:
        pytest.skip("oracle/_ref/native/_CUDA.so was not built")
    return mod


def _same(a, b):
    """Equal bit for bit; fp16 NaNs (the zero point of a row without range: 0 / 0) count as equal to each other."""
    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.dtype.is_floating_point:
        return bool(((a == b) | (a.isnan() & b.isnan())).all())
    return torch.equal(a, b)


def _acts(rows, cols, seed, outliers=True):
    """Activation rows as config 2 of the benchmark draws them: N(0, 1) with 0.1 % of the channels x 100."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((rows, cols), generator=g)
    if outliers:
        x[:, torch.randperm(cols, generator=g)[: max(1, cols // 1000)]] *= 100.0
    return x.half().to(DEV)


def _packed(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8).to(DEV)


@pytest.mark.parametrize("rows,cols", [(1, 4096), (33, 4096), (256, 14336), (7, 128), (64, 768)])
@pytest.mark.parametrize("clip", [1.0, 0.9])
def test_sym_and_asym_quant_dynamic(ref, rows, cols, clip):
    x = _acts(rows, cols, rows + cols)
    x[0, :] = 0                                     # the all-zero row of test_fused_equivalence.py:52
    if rows > 2:
        x[1, :] = 3.0                               # a constant row (asym range 0)
        x[2, 0] = 65504.0                           # the largest fp16 value
    q, s = kernel.sym_quant_dynamic(x, clip)
    rq, rs = ref.sym_quant_dynamic(x, clip)
    assert _same(s, rs) and _same(q, rq)
    q, s, z = kernel.asym_quant_dynamic(x, clip)
    rq, rs, rz = ref.asym_quant_dynamic(x, clip)
    assert _same(s, rs) and _same(z, rz) and _same(q, rq)


def test_quant_with_given_scales(ref):
    x = _acts(40, 4096, 3)
    _, s = kernel.sym_quant_dynamic(x)
    assert torch.equal(kernel.sym_quant(x, s), ref.sym_quant(x, s))
    _, s, z = kernel.asym_quant_dynamic(x)
    assert torch.equal(kernel.asym_quant_f16_ui4(x, s, z), ref.asym_quant_f16_ui4(x, s, z))
    zs = torch.randint(-8, 8, (40, 1), generator=torch.Generator().manual_seed(0)).half().to(DEV)
    assert torch.equal(kernel.asym_quant_f16_si4(x, s, zs), ref.asym_quant_f16_si4(x, s, zs))


@pytest.mark.parametrize("asym", [False, True])
def test_moe_quantizers_and_dequant(ref, asym):
    E, rows, cols, n = 8, 70, 14336, 512
    g = torch.Generator().manual_seed(5)
    x = _acts(rows, cols, 6)
    eid = torch.sort(torch.randint(0, E, (rows,), generator=g)).values.to(torch.int32).to(DEV)
    sign = (torch.randint(0, 2, (E, cols), generator=g) * 2 - 1).to(torch.int8).to(DEV)
    for sg in (sign, None):
        if asym:
            got, want = kernel.asym_quant_dynamic_moe(x, sg, eid, 1.0), ref.asym_quant_dynamic_moe(x, sg, eid, 1.0)
        else:
            got, want = kernel.sym_quant_dynamic_moe(x, sg, eid, 1.0), ref.sym_quant_dynamic_moe(x, sg, eid, 1.0)
        for a, b in zip(got, want):
            assert _same(a, b)
    acc = torch.randint(-200000, 200000, (rows, n), generator=g, dtype=torch.int32).to(DEV)
    sr_ = (torch.rand((rows, 1), generator=g) * 0.1).half().to(DEV)
    ws = (torch.rand((E, n), generator=g) * 0.01).half().to(DEV)
    zero = torch.randint(0, 16, (rows, 1), generator=g).to(torch.int8).to(DEV) if asym else None
    wsum = torch.randint(-3000, 3000, (E, n), generator=g, dtype=torch.int32).to(DEV) if asym else None
    assert torch.equal(kernel.sym_dequant_moe(acc, sr_, ws, eid, zero, wsum), ref.sym_dequant_moe(acc, sr_, ws, eid, zero, wsum))


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (16, 14336, 4096), (256, 4096, 14336), (300, 520, 512), (4096, 512, 4096)])
def test_matmul_and_dequant(ref, M, N, K):
    """Every kernel behind the GEMM entry (weight streaming, tcgen05 CTA pairs) against the reference's CUTLASS
    kernel: the int32 sums, then the dequantized fp16 matrix through both dequant routes."""
    A, B = _packed(M, K, 1), _packed(N, K, 2)
    c = kernel.matmul_si4_si4(A, B)
    assert torch.equal(c, ref.matmul(A, B))
    assert torch.equal(kernel.matmul_ui4_si4(A, B), ref.matmul_ui4_si4(A, B))
    g = torch.Generator().manual_seed(3)
    sa = (torch.rand((M, 1), generator=g) * 0.1).half().to(DEV)
    sw = (torch.rand((N, 1), generator=g) * 0.01).half().to(DEV)
    want = ref.sym_dequant(c, sa, sw, 32)
    assert torch.equal(kernel.sym_dequant(c, sa, sw, 32), want)
    fused = kernel.w4a4_linear(kernel.PackedQuantizedTensor(A, sa), B, sw)
    assert torch.equal(fused, want)


def test_sum_and_colrow(ref):
    W = _packed(520, 4096, 4)
    for signed in (True, False):
        assert torch.equal(kernel.sum_i4(W, signed), ref.sum_i4(W, signed))
    g = torch.Generator().manual_seed(1)
    a = torch.randint(-128, 128, (77, 1), generator=g).to(torch.int8).to(DEV)
    b = torch.randint(-30000, 30000, (1, 520), generator=g, dtype=torch.int32).to(DEV)
    assert torch.equal(kernel.matmul_colrow_i8_i32(a, b), ref.matmul_colrow_i8_i32(a, b))


@pytest.mark.parametrize("ms", [[700, 0, 129, 256, 1, 333, 64, 517], [3, 0, 2, 1, 0, 0, 5, 1]])
@pytest.mark.parametrize("signed", [True, False])
def test_matmul_grouped(ref, ms, signed):
    """Prefill-sized (tensor-core kernel here) and decode-sized (CUDA-core kernel here) problem lists in the MoE
    block's layout (signrot/nn/moe.py:96-111), against the reference's CUTLASS grouped kernel."""
    P, n, k = len(ms), 512, 4096
    rows = sum(ms)
    A, B = _packed(rows, k, 7), _packed(P * n, k, 8).view(P, n, k // 2)
    off = torch.tensor([sum(ms[:i]) for i in range(P)], dtype=torch.int64)
    ps = torch.tensor([[m, n, k] for m in ms], dtype=torch.int32, device=DEV)
    ptr_a = (A.data_ptr() + off * (k // 2)).to(DEV)
    ptr_b = (B.data_ptr() + torch.arange(P, dtype=torch.int64) * B.stride(0)).to(DEV)
    ld_ab = torch.full((P,), k, dtype=torch.int64, device=DEV)
    ld_c = torch.full((P,), n, dtype=torch.int64, device=DEV)
    out = []
    for fn in (kernel.matmul_grouped, ref.matmul_grouped):
        C = torch.full((rows, n), -777, dtype=torch.int32, device=DEV)
        ptr_c = (C.data_ptr() + off * (n * 4)).to(DEV)
        fn(ps, ptr_a, ptr_b, ptr_c, ld_ab, ld_ab, ld_c, signed)
        torch.cuda.synchronize()
        out.append(C)
    assert torch.equal(out[0], out[1])


def test_kv_quant_pack_rope_swiglu_rmsnorm(ref):
    g = torch.Generator().manual_seed(9)
    kv = torch.randn((4, 33, 8, 128), generator=g).half().to(DEV)
    kv[0, 0, 0] = 0.5                                # a constant vector: the range floor of fused.cu:236-261
    q, p = kernel.kv_quant_pack(kv)
    rq, rp = ref.kv_quant_pack(kv)
    assert torch.equal(p, rp) and torch.equal(q, rq)

    B, T, Hq, Hk, D = 2, 37, 32, 8, 128
    qh, kh = torch.randn((B, T, Hq, D), generator=g).half().to(DEV), torch.randn((B, T, Hk, D), generator=g).half().to(DEV)
    ang = torch.rand((1, T, D), generator=g) * 6.28
    cos, sin = ang.cos().half().to(DEV), ang.sin().half().to(DEV)
    q1, k1, q2, k2 = qh.clone(), kh.clone(), qh.clone(), kh.clone()
    kernel.rope_qk(q1, k1, cos, sin)
    ref.rope_qk(q2, k2, cos, sin)
    assert torch.equal(q1, q2) and torch.equal(k1, k2)

    gate, up = (torch.randn((40, 14336), generator=g) * 3).half().to(DEV), torch.randn((40, 14336), generator=g).half().to(DEV)
    assert torch.equal(kernel.swiglu(gate, up), ref.swiglu(gate, up))

    # RMSNorm: the fp32 sum of squares is taken in another order (128-bit loads here, a strided scalar loop in
    # fused.cu:278-302), so the factor can differ in its last bit and a few outputs land on the neighbouring fp16
    # value; both are equally close to the fp64 result.  Bound: one fp16 ulp, at most 1e-3 of the values.
    for outliers in (True, False):
        x = _acts(40, 4096, 11, outliers)
        a, b = kernel.rmsnorm(x, 1e-5, 4096), ref.rmsnorm(x, 1e-5, 4096)
        ulp = (a.view(torch.int16).int() - b.view(torch.int16).int()).abs()
        assert ulp.max().item() <= 1 and (ulp > 0).float().mean().item() <= 1e-3


@pytest.mark.parametrize("chunks", [1, 3])
def test_paged_cache_and_decode_attention(ref, chunks):
    """init_kv_i4 / append_kv_i4 fill the same bytes; batch_decode_i4 over that cache agrees within the reference's
    split-vs-unsplit bound (benchmarks/test_split_decode.py).  One KV head per query head, the only geometry in which
    the reference's repeated-head cache and this library's are the same array."""
    B, H, D, page, L, T = 4, 8, 128, 16, 2, 100
    pages = (T + 1 + page - 1) // page
    g = torch.Generator().manual_seed(21)
    k, v = torch.randn((B, T, H, D), generator=g).half().to(DEV), torch.randn((B, T, H, D), generator=g).half().to(DEV)
    kq, kp = ref.kv_quant_pack(k)
    vq, vp = ref.kv_quant_pack(v)
    indptr = (torch.arange(B + 1, dtype=torch.int32) * pages).to(DEV)
    indices = (torch.arange(pages, dtype=torch.int32).view(1, -1) * B + torch.arange(B, dtype=torch.int32).view(-1, 1)).reshape(-1).to(DEV)
    seq = (torch.arange(B + 1, dtype=torch.int32) * T).to(DEV)
    k1, v1 = torch.randn((B, 1, H, D), generator=g).half().to(DEV), torch.randn((B, 1, H, D), generator=g).half().to(DEV)
    k1q, k1p = ref.kv_quant_pack(k1)
    v1q, v1p = ref.kv_quant_pack(v1)
    caches = []
    for mod in (kvc, ref):
        data = torch.zeros((pages * B, L, 2, H, page, D // 2), dtype=torch.uint8, device=DEV)
        param = torch.zeros((pages * B, L, 2, H, page, 2), dtype=torch.float16, device=DEV)
        last = torch.full((B,), T % page or page, dtype=torch.int32, device=DEV)
        mod.init_kv_i4(data, param, indptr, indices, last, kq.view(-1, H, D // 2), vq.view(-1, H, D // 2),
                       kp.view(-1, H, 2), vp.view(-1, H, 2), seq, 1)
        last.fill_((T + 1) % page or page)
        mod.append_kv_i4(data, param, indptr, indices, last, k1q.view(B, H, D // 2), v1q.view(B, H, D // 2),
                         k1p.view(B, H, 2), v1p.view(B, H, 2), 1)
        torch.cuda.synchronize()
        caches.append((data, param, last))
    assert torch.equal(caches[0][0], caches[1][0]) and torch.equal(caches[0][1], caches[1][1])
    q = torch.randn((B, H, D), generator=g).half().to(DEV)
    outs = []
    for mod, (data, param, last) in zip((kvc, ref), caches):
        o = torch.empty_like(q)
        tmp = torch.empty((B, H, chunks, D + 4), dtype=torch.float32, device=DEV) if chunks > 1 else None
        mod.batch_decode_i4(o, q, data, param, indptr, indices, last, 1, tmp, chunks)
        torch.cuda.synchronize()
        outs.append(o.float())
    assert (outs[0] - outs[1]).abs().max().item() <= 2e-3


def test_gqa_decode_against_the_repeated_head_cache(ref):
    """32 q heads on 8 KV heads: this library keeps every KV head once, the reference's cache repeats it for each q head
    of its group (signrot/transformers/kv_cache.py:346-353).  Fill this library's cache, repeat its heads into the
    reference's layout, decode with both kernels: the reference's own split-vs-unsplit bound (2e-3)."""
    B, Hq, Hkv, D, page, T = 4, 32, 8, 128, 16, 333
    G = Hq // Hkv
    g = torch.Generator().manual_seed(5)
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 8, DEV, 1, Hkv, D, group_size=G)
    cache.pages.zero_()
    cache.scales.zero_()
    k, v = torch.randn((B, T, Hkv, D), generator=g).half().to(DEV), torch.randn((B, T, Hkv, D), generator=g).half().to(DEV)
    cache.update(k, v, 0)
    specs = cache.refresh_specs()
    q = torch.randn((B, Hq, D), generator=g).half().to(DEV)
    mine = torch.empty_like(q)
    kvc.batch_decode_i4(mine, q, **specs, layer_idx=0, hadamard_q=False)
    ref_data = specs["kv_data"].repeat_interleave(G, dim=3).contiguous()
    ref_param = specs["kv_param"].repeat_interleave(G, dim=3).contiguous()
    theirs = torch.empty_like(q)
    ref.batch_decode_i4(theirs, q, ref_data, ref_param, specs["kv_indptr"], specs["kv_indices"], specs["last_page_offset"], 0)
    torch.cuda.synchronize()
    assert (mine.float() - theirs.float()).abs().max().item() <= 2e-3


@pytest.mark.parametrize("n,heads", [(14336, 0), (4096, 32), (768, 0)])
def test_fused_rotation_feeds_the_reference_quantizer(ref, n, heads):
    """The reference has no GPU rotation of its own (fast_hadamard_transform is not in the checkout), but its quantizer
    can be run on the rotated rows this library returns beside the codes: the codes and scales of the fused kernel must
    be what signrot._CUDA.sym_quant_dynamic makes of those rows, bit for bit."""
    from signrot_b200.functional.hadamard import get_hadK
    x = _acts(64, n, 3)
    g = torch.Generator().manual_seed(4)
    if heads:
        pk, rot = kernel.rotate_quant(x, heads=heads, return_rotated=True)
    else:
        hadK, K = get_hadK(n)
        sign = (torch.randint(0, 2, (n,), generator=g) * 2 - 1).to(torch.int8).to(DEV)
        pk, rot = kernel.rotate_quant(x, hadK, K, sign=sign, return_rotated=True)
    rq, rs = ref.sym_quant_dynamic(rot.contiguous(), 1.0)
    assert _same(pk.scales_x.view(-1), rs.view(-1)) and _same(pk.quantized_x, rq)
