"""int4 GEMM kernels (weight-streaming mma.sync kernel of the decode regime: M <= 32, or M <= 64 with N <= 32 x the SM count;
CTA-pair tcgen05 kernel above it) against the integer oracle: int32 accumulators bit-exact, fused dequant
epilogue bit-exact.  The shapes below reach both kernels."""
import pytest
import torch

import oracle
from signrot_b200 import _lib
from signrot_b200.functional import kernel
from signrot_b200 import nn as snn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _codes(rows, K, seed, lo=-8, hi=8):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi, (rows, K), generator=g, dtype=torch.int32)


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert _lib.device_status() == 0


SHAPES = [(1, 4096, 4096), (16, 4096, 4096), (3, 64, 40), (33, 256, 96), (128, 4096, 512), (256, 4096, 4096),
          (200, 1024, 300), (129, 14336, 264), (512, 2048, 14336), (64, 14336, 256), (16, 14336, 4096),
          (32, 4096, 14336), (33, 4096, 14336), (64, 4096, 8192), (65, 512, 8192), (40, 1024, 9000), (1, 64, 8), (257, 64, 257)]


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_matmul_si4_bit_exact(M, K, N):
    a, b = _codes(M, K, M + K), _codes(N, K, N + 7)
    A, B = oracle.pack_i4(a), oracle.pack_i4(b)
    C = kernel.matmul_si4_si4(A.to(DEV), B.to(DEV)).cpu()
    assert _lib.device_status() == 0
    assert torch.equal(C, oracle.matmul_i4(A, B))


@pytest.mark.parametrize("M", [130, 24])
def test_matmul_ui4_and_extremes(M):
    K, N = 1024, 257 + 7
    a, b = _codes(M, K, 1, 0, 16), _codes(N, K, 2)
    A, B = oracle.pack_codes(a), oracle.pack_i4(b)
    C = kernel.matmul_ui4_si4(A.to(DEV), B.to(DEV)).cpu()
    assert torch.equal(C, oracle.matmul_i4(A, B, a_unsigned=True))
    # worst-case magnitudes: every product 64 (signed) / -120 (unsigned x -8)
    A = oracle.pack_i4(torch.full((M, 4096), -8, dtype=torch.int32))
    B = oracle.pack_i4(torch.full((40, 4096), -8, dtype=torch.int32))
    C = kernel.matmul_si4_si4(A.to(DEV), B.to(DEV)).cpu()
    assert int(C.min()) == int(C.max()) == 64 * 4096
    A = oracle.pack_codes(torch.full((M, 4096), 15, dtype=torch.int32))
    C = kernel.matmul_ui4_si4(A.to(DEV), B.to(DEV)).cpu()
    assert int(C.min()) == int(C.max()) == -120 * 4096


@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 14336), (14336, 4096)])
def test_w4a4_linear_benchmark_shapes(K, N):
    """The benchmarked launches (M = 4096 token rows, the library's own kernel choice): int32 accumulators and
    the fused fp16 output against the oracle on a random 256-row subset, and EVERY row through a
    checksum the integer product must satisfy exactly: sum_m C[m, :] = (sum_m A[m, :]) B^T."""
    M = 4096
    g = torch.Generator().manual_seed(K + N)
    A = torch.randint(0, 256, (M, K // 2), generator=g, dtype=torch.uint8)
    W = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    sa = (torch.rand((M, 1), generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand((N, 1), generator=g) * 0.009 + 0.001).half()
    acc = kernel.matmul_si4_si4(A.to(DEV), W.to(DEV))
    out = kernel.w4a4_linear(kernel.PackedQuantizedTensor(A.to(DEV), sa.to(DEV)), W.to(DEV), sw.to(DEV))
    assert _lib.device_status() == 0
    rows = torch.randperm(M, generator=g)[:256].sort().values
    want_acc = oracle.matmul_i4(A[rows], W)
    assert torch.equal(acc[rows.to(DEV)].cpu(), want_acc)
    assert torch.equal(out[rows.to(DEV)].cpu(), oracle.sym_dequant(want_acc, sa[rows], sw))
    col_sum = oracle.unpack_i4(A).sum(0, dtype=torch.int64).double()            # |.| <= 8 * 4096
    want_sum = (col_sum[None, :] @ oracle.unpack_i4(W).double().T).to(torch.int64).view(-1)
    assert torch.equal(acc.sum(0, dtype=torch.int64).cpu(), want_sum)
    # the fp16 output of every row is the dequant of the accumulator the same launch family produced
    assert torch.equal(out, kernel.sym_dequant(acc, sa.to(DEV), sw.to(DEV)))


def test_k_limit_of_the_int32_accumulator():
    """Products are carried times 256 by the tensor-core kernel: K is refused where the worst case leaves int32."""
    A = torch.zeros((1, 131072 // 2), dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="accumulator range"):
        kernel.matmul_si4_si4(A, A)
    with pytest.raises(RuntimeError, match="accumulator range"):
        kernel.matmul_ui4_si4(A[:, : 65600 // 2].contiguous(), A[:, : 65600 // 2].contiguous())


def test_matmul_leading_dims_and_empty():
    a, b = _codes(6, 128, 1), _codes(10, 128, 2)
    A, B = oracle.pack_i4(a).view(2, 3, 64), oracle.pack_i4(b)
    C = kernel.matmul_si4_si4(A.to(DEV), B.to(DEV))
    assert C.shape == (2, 3, 10)
    assert torch.equal(C.cpu().view(6, 10), oracle.matmul_i4(A.view(6, 64), B))
    E = kernel.matmul_si4_si4(torch.empty((0, 64), dtype=torch.uint8, device=DEV), B.to(DEV))
    assert E.shape == (0, 10)


@pytest.mark.parametrize("M,K,N,asym,bias", [(16, 4096, 4096, False, False), (200, 1024, 264, False, True),
                                             (130, 2048, 512, True, False), (7, 256, 40, True, True),
                                             (70, 256, 40, True, True), (16, 1024, 264, False, True), (300, 4096, 4096, True, False)])
def test_w4a4_linear_fused_epilogue(M, K, N, asym, bias):
    g = torch.Generator().manual_seed(M)
    a = _codes(M, K, 3, 0 if asym else -8, 16 if asym else 8)
    w = _codes(N, K, 4)
    A, W = oracle.pack_codes(a), oracle.pack_i4(w)
    sa = (torch.rand((M, 1), generator=g) * 0.5 + 0.05).half()
    sw = (torch.rand((N, 1), generator=g) * 0.009 + 0.001).half()
    za = torch.randint(0, 16, (M, 1), generator=g).to(torch.int8) if asym else None
    bs = torch.randn((N,), generator=g).half() if bias else None
    wsum = oracle.sum_i4(W)
    want = oracle.w4a4_linear(A, sa, W, sw, za, wsum if asym else None, bs)
    lin = snn.Linear4bit(K, N, bias=bias).to(DEV)
    lin.weight.copy_(W)
    lin.weight_scales = sw.to(DEV)
    if bias:
        lin.bias.copy_(bs)
    pk = kernel.PackedQuantizedTensor(A.to(DEV), sa.to(DEV), za.to(DEV) if asym else None)
    got = lin(pk)
    assert torch.equal(got.cpu(), want)
    # the reference's operator chain (matmul -> colrow -> dequant -> bias) gives the same bits
    assert torch.equal(lin.forward_unfused(pk).cpu(), want)


@pytest.mark.parametrize("M,K,N,asym,bias", [(256, 14336, 4096, False, False), (130, 8192, 512, True, True),
                                             (512, 14336, 4096, False, False), (300, 14336, 2048, True, False),
                                             (200, 8192, 264, True, True), (65, 16384, 1032, False, True)])
def test_w4a4_linear_split_k_same_bits(M, K, N, asym, bias):
    """Long-K shapes with few output tiles split K over CTA pairs and meet in a workspace (`sr_w4a4_linear_ws`): the
    bits of the unsplit launch and of the oracle's row subset, call after call (the counters only grow) and from a
    replayed graph."""
    import ctypes
    from signrot_b200._lib import call_nostream, ptr, run
    g = torch.Generator().manual_seed(M + N)
    a = _codes(M, K, 3, 0 if asym else -8, 16 if asym else 8)
    w = _codes(N, K, 4)
    A, W = oracle.pack_codes(a).to(DEV), oracle.pack_i4(w).to(DEV)
    sa = (torch.rand((M,), generator=g) * 0.5 + 0.05).half().to(DEV)
    sw = (torch.rand((N,), generator=g) * 0.009 + 0.001).half().to(DEV)
    za = torch.randint(0, 16, (M,), generator=g).to(torch.int8).to(DEV) if asym else None
    bs = torch.randn((N,), generator=g).half().to(DEV) if bias else None
    wsum = kernel.sum_i4(W).reshape(-1) if asym else None
    need = ctypes.c_int64(0)
    call_nostream("sr_w4a4_linear_ws_bytes", M, N, K, ctypes.byref(need))
    assert need.value > 0, "this shape is expected to split K"
    plain = torch.empty((M, N), dtype=torch.float16, device=DEV)
    run(torch.device(DEV, 0), "sr_w4a4_linear", ptr(A), ptr(sa), ptr(za), ptr(W), ptr(sw), ptr(wsum), ptr(bs), M, N, K, ptr(plain))
    rows = torch.randperm(M, generator=g)[:24]
    want = oracle.w4a4_linear(A[rows].cpu(), sa[rows].cpu().view(-1, 1), W.cpu(), sw.cpu().view(-1, 1),
                              za[rows].cpu().view(-1, 1) if asym else None, wsum.cpu().view(-1, 1) if asym else None,
                              bs.cpu() if bias else None)
    assert torch.equal(plain[rows.to(DEV)].cpu(), want)
    pk = kernel.PackedQuantizedTensor(A, sa, za)
    for _ in range(3):                                   # the wrapper takes the split route by itself
        got = kernel.w4a4_linear(pk, W, sw, wsum, bs)
        assert torch.equal(got, plain)
    key = (0, torch.cuda.current_stream().cuda_stream)
    assert int(kernel._SPLIT_COUNTERS[key].sum()) > 0, "the split-K entry was not used"
    # captured on a stream that has its counters already (a first call inside a capture runs unsplit: nothing may be
    # zero-filled there), replayed twice
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        assert torch.equal(kernel.w4a4_linear(pk, W, sw, wsum, bs), plain)
    side.synchronize()
    skey = (0, side.cuda_stream)
    before = int(kernel._SPLIT_COUNTERS[skey].sum())
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr, stream=side):
        out = kernel.w4a4_linear(pk, W, sw, wsum, bs)
    for _ in range(2):
        out.zero_()
        torch.cuda.synchronize()
        gr.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, plain)
    assert int(kernel._SPLIT_COUNTERS[skey].sum()) > before, "the captured launch did not split K"


def test_asym_symm_linear():
    M, K, N = 9, 256, 48
    g = torch.Generator().manual_seed(0)
    a, w = _codes(M, K, 5), _codes(N, K, 6)
    A, W = oracle.pack_i4(a), oracle.pack_i4(w)
    sa = torch.rand((M, 1), generator=g).half() + 0.1
    sw = (torch.rand((N, 1), generator=g) * 0.01).half()
    za = torch.randint(-8, 8, (M, 1), generator=g).to(torch.int8)
    lin = snn.AsymSymmLinear4bit(K, N).to(DEV)
    lin.weight.copy_(W)
    lin.weight_scales = sw.to(DEV)
    lin.weight_sum = oracle.sum_i4(W).to(DEV)
    got = lin(kernel.PackedQuantizedTensor(A.to(DEV), sa.to(DEV), za.to(DEV))).cpu()
    acc = oracle.matmul_i4(A, W) - oracle.matmul_colrow(za, oracle.sum_i4(W).view(1, -1))
    assert torch.equal(got, oracle.sym_dequant(acc, sa, sw))


def test_determinism():
    a, b = _codes(300, 4096, 1), _codes(520, 4096, 2)
    A, B = oracle.pack_i4(a).to(DEV), oracle.pack_i4(b).to(DEV)
    c1 = kernel.matmul_si4_si4(A, B)
    c2 = kernel.matmul_si4_si4(A, B)
    assert torch.equal(c1, c2)


def test_grouped_matches_dense():
    """Grouped GEMM == per-problem dense GEMM, incl. empty problems, skew, M=1, M=513
    (benchmarks/test_grouped_gemm.py:76-91)."""
    for ms, n, k, signed in [([5, 0, 17, 1], 96, 256, True), ([4096, 3, 0, 1], 64, 128, True), ([1], 40, 64, True),
                             ([513, 7], 72, 512, False), ([0, 0], 32, 64, True)]:
        P = len(ms)
        a_all = _codes(sum(ms), k, 1, -8 if signed else 0, 8 if signed else 16)
        A = oracle.pack_codes(a_all).to(DEV)
        Bs = [oracle.pack_i4(_codes(n, k, 10 + i)) for i in range(P)]
        B = torch.stack(Bs).to(DEV)
        C = torch.full((sum(ms), n), -777, dtype=torch.int32, device=DEV)
        off = torch.tensor([sum(ms[:i]) for i in range(P)], dtype=torch.int64)
        ps = torch.tensor([[m, n, k] for m in ms], dtype=torch.int32, device=DEV)
        ptr_a = (A.data_ptr() + off * (k // 2)).to(DEV)
        ptr_b = (B.data_ptr() + torch.arange(P, dtype=torch.int64) * B.stride(0)).to(DEV)
        ptr_c = (C.data_ptr() + off * (n * 4)).to(DEV)
        ld_ab = torch.full((P,), k, dtype=torch.int64, device=DEV)
        ld_c = torch.full((P,), n, dtype=torch.int64, device=DEV)
        for max_k in (0, k):
            C.fill_(-777)
            kernel.matmul_grouped(ps, ptr_a, ptr_b, ptr_c, ld_ab, ld_ab, ld_c, signed_a=signed, max_k=max_k)
            got = C.cpu()
            row = 0
            for i, m in enumerate(ms):
                want = oracle.matmul_i4(oracle.pack_codes(a_all[row:row + m]), Bs[i], a_unsigned=not signed)
                assert torch.equal(got[row:row + m], want)
                row += m
        assert _lib.device_status() == 0


def _grouped_case(ms, n, k, signed, seed=0, ldc=None, order=None):
    """Device arrays of one matmul_grouped call in the layout signrot/nn/moe.py:96-111 builds (rows sorted by
    problem, stacked weights, one output matrix); `order` permutes the problem list, which keeps every problem
    valid but is no longer that layout."""
    P = len(ms)
    ldc = ldc or n
    a_all = _codes(sum(ms), k, 1 + seed, -8 if signed else 0, 8 if signed else 16)
    A = oracle.pack_codes(a_all).to(DEV)
    Bs = [oracle.pack_i4(_codes(n, k, 10 + seed + i)) for i in range(P)]
    B = torch.stack(Bs).to(DEV)
    C = torch.full((sum(ms), ldc), -777, dtype=torch.int32, device=DEV)
    off = torch.tensor([sum(ms[:i]) for i in range(P)], dtype=torch.int64)
    idx = torch.tensor(order if order is not None else list(range(P)))
    ps = torch.tensor([[m, n, k] for m in ms], dtype=torch.int32)[idx].to(DEV)
    ptr_a = (A.data_ptr() + off * (k // 2))[idx].to(DEV)
    ptr_b = (B.data_ptr() + torch.arange(P, dtype=torch.int64) * B.stride(0))[idx].to(DEV)
    ptr_c = (C.data_ptr() + off * (ldc * 4))[idx].to(DEV)
    ld_ab = torch.full((P,), k, dtype=torch.int64, device=DEV)
    ld_c = torch.full((P,), ldc, dtype=torch.int64, device=DEV)
    return dict(a_all=a_all, A=A, Bs=Bs, B=B, C=C, ps=ps, ptr_a=ptr_a, ptr_b=ptr_b, ptr_c=ptr_c, ld_ab=ld_ab,
                ld_c=ld_c, ms=ms, n=n, signed=signed)


def _check_grouped(c):
    got = c["C"].cpu()
    row = 0
    for i, m in enumerate(c["ms"]):
        want = oracle.matmul_i4(oracle.pack_codes(c["a_all"][row:row + m]), c["Bs"][i], a_unsigned=not c["signed"])
        assert torch.equal(got[row:row + m, :c["n"]], want), f"problem {i}"
        row += m
    assert bool((got[:, c["n"]:] == -777).all())          # padding columns of a wide output stay untouched


@pytest.mark.parametrize("signed", [True, False])
def test_grouped_prefill_size_on_both_kernels(signed):
    """The pointer-array entry at prefill size.  The expert-sorted layout goes to the tensor cores, the same problems
    listed in another order (a layout the planning kernel does not recognise) go to the CUDA-core kernel, and so does a
    decode-sized call; all give the oracle's integers.  Sizes: 8 experts, uneven rows incl. an empty expert, n not a
    multiple of the tile, an output matrix wider than n."""
    ms = [700, 0, 129, 256, 1, 333, 64, 517]
    for kwargs in (dict(), dict(order=[3, 0, 7, 1, 2, 6, 5, 4]), dict(ldc=328)):
        c = _grouped_case(ms, 320, 1024, signed, seed=3, **kwargs)
        kernel.matmul_grouped(c["ps"], c["ptr_a"], c["ptr_b"], c["ptr_c"], c["ld_ab"], c["ld_ab"], c["ld_c"],
                              signed_a=signed)
        _check_grouped(c)
    c = _grouped_case([3, 0, 2, 1], 320, 1024, signed, seed=4)
    kernel.matmul_grouped(c["ps"], c["ptr_a"], c["ptr_b"], c["ptr_c"], c["ld_ab"], c["ld_ab"], c["ld_c"], signed_a=signed)
    _check_grouped(c)
    assert _lib.device_status() == 0


def test_grouped_graph_replay_switches_kernels_with_the_sizes():
    """Nothing of a matmul_grouped call is read on the host (signrot/kernels/bindings.cpp:49-91), so a captured call
    follows the device arrays: replayed with prefill-sized row counts it runs on the tensor cores, with a few rows per
    expert on the CUDA cores, and back, from one capture."""
    big = _grouped_case([300, 40, 0, 260], 256, 512, True, seed=5)
    small_ms = [2, 1, 0, 3]
    ps, ptr_a, ptr_c = big["ps"].clone(), big["ptr_a"].clone(), big["ptr_c"].clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        kernel.matmul_grouped(ps, ptr_a, big["ptr_b"], ptr_c, big["ld_ab"], big["ld_ab"], big["ld_c"])  # warm-up
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            kernel.matmul_grouped(ps, ptr_a, big["ptr_b"], ptr_c, big["ld_ab"], big["ld_ab"], big["ld_c"])
    off_small = torch.tensor([sum(small_ms[:i]) for i in range(4)], dtype=torch.int64)
    for ms in (big["ms"], small_ms, big["ms"]):
        if ms is small_ms:
            ps.copy_(torch.tensor([[m, 256, 512] for m in ms], dtype=torch.int32))
            ptr_a.copy_(big["A"].data_ptr() + off_small * 256)
            ptr_c.copy_(big["C"].data_ptr() + off_small * 256 * 4)
        else:
            ps.copy_(big["ps"]); ptr_a.copy_(big["ptr_a"]); ptr_c.copy_(big["ptr_c"])
        big["C"].fill_(-777)
        graph.replay()
        torch.cuda.synchronize()
        got = big["C"].cpu()
        row = 0
        for i, m in enumerate(ms):
            want = oracle.matmul_i4(oracle.pack_codes(big["a_all"][row:row + m]), big["Bs"][i])
            assert torch.equal(got[row:row + m], want)
            row += m
        assert bool((got[row:] == -777).all())
    assert _lib.device_status() == 0


@pytest.mark.parametrize("M", [1, 8, 13, 16, 32, 40])
@pytest.mark.parametrize("F,K", [(1536, 512), (14336, 4096), (104, 256)])
@pytest.mark.parametrize("asym", [False, True])
def test_w4a4_swiglu_equals_two_linears_and_swiglu(M, F, K, asym):
    """gate_proj + up_proj + SwiGLU in one launch: the bits of the three separate launches (rows
    beyond 32 take the separate route inside the wrapper)."""
    g = torch.Generator().manual_seed(M * 131 + F)
    w = torch.randint(0, 256, (2 * F, K // 2), generator=g, dtype=torch.uint8).to(DEV)
    ws = ((torch.rand((2 * F, 1), generator=g) * 0.5 + 0.5) / K).half().to(DEV)
    x = torch.randn((M, K), generator=g).half().to(DEV)
    if asym:
        q, s, z = kernel.asym_quant_dynamic(x)
        packed = kernel.PackedQuantizedTensor(q, s, z.to(torch.int8))
        wsum = kernel.sum_i4(w)
    else:
        q, s = kernel.sym_quant_dynamic(x)
        packed = kernel.PackedQuantizedTensor(q, s)
        wsum = None
    got = kernel.w4a4_swiglu(packed, w, ws, wsum)
    gate = kernel.w4a4_linear(packed, w[:F], ws[:F], wsum[:F] if asym else None)
    up = kernel.w4a4_linear(packed, w[F:], ws[F:], wsum[F:] if asym else None)
    want = kernel.swiglu(gate, up)
    assert got.shape == (M, F) and torch.equal(got, want)


def test_bounded_wait_gives_up_and_the_next_launch_is_clean():
    """The give-up path of the device-side waits, without provoking anything: a one-thread wait with a budget of
    1e5 cycles on a barrier nobody arrives on returns, the status word reports its code until it is read and
    cleared, a GEMM launched while the word is set does no work, and the launch after the clear is correct."""
    a, b = _codes(300, 512, 1), _codes(264, 512, 2)
    A, B = oracle.pack_i4(a).to(DEV), oracle.pack_i4(b).to(DEV)
    want = oracle.matmul_i4(A.cpu(), B.cpu())
    assert torch.equal(kernel.matmul_si4_si4(A, B).cpu(), want)
    _lib.call("sr_selftest_bounded_wait", 100000)
    torch.cuda.synchronize()                       # returns: the kernel ended by itself
    assert _lib.device_status(clear=False) == 99
    skipped = kernel.matmul_si4_si4(A, B)          # sticky word: the tensor-core kernel drains without computing
    torch.cuda.synchronize()
    del skipped
    assert _lib.device_status() == 99              # read and clear
    assert _lib.device_status() == 0
    assert torch.equal(kernel.matmul_si4_si4(A, B).cpu(), want)
    with pytest.raises(RuntimeError, match="budget"):
        _lib.call("sr_selftest_bounded_wait", 10 ** 9)


@pytest.mark.parametrize("M,N", [(8, 4096), (40, 512), (300, 264)])
def test_matmul_on_a_column_range_of_the_codes(M, N):
    """The K-slice product of a row-parallel linear: columns [begin, end) of a wider code matrix, read in place
    (weight-streaming kernel for few rows, tensor-core kernel otherwise) == the product on a copy of the slice."""
    K_full, begin, end = 4096, 1024, 3072           # values; packed bytes are half of these
    a, b = _codes(M, K_full, M), _codes(N, end - begin, N + 1)
    A, B = oracle.pack_i4(a).to(DEV), oracle.pack_i4(b).to(DEV)
    got = kernel.matmul_si4_cols(A, begin // 2, end // 2, B)
    assert _lib.device_status() == 0
    assert torch.equal(got.cpu(), oracle.matmul_i4(A[:, begin // 2:end // 2].cpu(), B.cpu()))
    with pytest.raises(RuntimeError, match="column range"):
        kernel.matmul_si4_cols(A, 8, 8 + (end - begin) // 2, B)
