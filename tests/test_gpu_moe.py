"""SignRotMoEBlock: grouped path == per-expert loop bit-exact, both == integer oracle, and
CUDA-graph replay on unseen inputs (benchmarks/test_moe_equivalence.py:103-157)."""
import pytest
import torch

import oracle
from conftest import rel_l2
from signrot_b200 import nn as snn
from signrot_b200.functional import kernel
from signrot_b200.functional.hadamard import get_hadK

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _block(E, hidden, inter, top_k, seed, asym=False, sign=True):
    g = torch.Generator().manual_seed(seed)
    def w(n, k):
        return oracle.pack_i4(torch.randint(-8, 8, (E, n, k), generator=g, dtype=torch.int32).view(E * n, k)).view(E, n, k // 2)
    def s(n, k):
        return (torch.rand((E, n), generator=g) * 0.5 / k + 0.5 / k).half()
    gate = torch.nn.Linear(hidden, E, bias=False).half()
    gate.weight.data = torch.randn((E, hidden), generator=g).half()
    sg = (torch.randint(0, 2, (E, inter), generator=g) * 2 - 1).to(torch.int8) if sign else None
    blk = snn.SignRotMoEBlock(gate.to(DEV), top_k=top_k, norm_topk_prob=True,
                              w_gate=w(inter, hidden).to(DEV), s_gate=s(inter, hidden).to(DEV),
                              w_up=w(inter, hidden).to(DEV), s_up=s(inter, hidden).to(DEV),
                              w_down=w(hidden, inter).to(DEV), s_down=s(hidden, inter).to(DEV),
                              sign_down=sg.to(DEV) if sign else None, asym=asym)
    return blk


def _per_expert_loop(blk, x):
    """The block's forward as a host loop over experts through the DENSE kernels (the reference keeps the same
    loop as its equivalence check, signrot/nn/moe.py:138-157): identical inputs must give identical bits."""
    hid = x.shape[-1]
    xf = x.reshape(-1, hid)
    logits = blk.gate(xf)
    weights, _, tok, eid, inv, row_off = kernel.moe_route(logits, blk.top_k, blk.norm_topk_prob)
    if blk.asym:
        q, s, z = kernel.asym_quant_dynamic(xf, blk.clip_ratio)
        z = z.to(torch.int8)
    else:
        (q, s), z = kernel.sym_quant_dynamic(xf, blk.clip_ratio), None
    t = tok.long()
    q, s, z = q[t], s[t], (z[t] if z is not None else None)
    offs = row_off.tolist()

    def dense(q_, s_, z_, w, s_w, wsum):
        out = torch.empty((q_.shape[0], w.shape[1]), dtype=torch.float16, device=q_.device)
        for e in range(blk.num_experts):
            sl = slice(offs[e], offs[e + 1])
            if sl.start == sl.stop:
                continue
            if z_ is not None:
                acc = kernel.matmul_ui4_si4(q_[sl], w[e]) - kernel.matmul_colrow_i8_i32(z_[sl], wsum[e].view(1, -1))
            else:
                acc = kernel.matmul_si4_si4(q_[sl], w[e])
            out[sl] = kernel.sym_dequant(acc, s_[sl], s_w[e].view(-1, 1))
        return out
    inter = kernel.swiglu(dense(q, s, z, blk.w_gate, blk.s_gate, blk.wsum_gate), dense(q, s, z, blk.w_up, blk.s_up, blk.wsum_up))
    h = kernel.hadamard(inter, blk.had_K, blk.K)
    if blk.sign_down is not None:
        h = h * blk.sign_down[eid.long()]
    if blk.asym:
        q2, s2, z2 = kernel.asym_quant_dynamic(h, blk.clip_ratio)
        z2 = z2.to(torch.int8)
    else:
        (q2, s2), z2 = kernel.sym_quant_dynamic(h, blk.clip_ratio), None
    y = dense(q2, s2, z2, blk.w_down, blk.s_down, blk.wsum_down)
    out = (y[inv.long()].view(-1, blk.top_k, hid) * weights.unsqueeze(-1)).sum(dim=1)
    return out.view(x.shape), logits


@pytest.mark.parametrize("E,hidden,inter,top_k,tokens", [(16, 256, 192, 4, 40), (8, 512, 768, 2, 64), (4, 128, 64, 1, 5)])
@pytest.mark.parametrize("asym", [False, True])
def test_grouped_equals_loop(E, hidden, inter, top_k, tokens, asym):
    blk = _block(E, hidden, inter, top_k, 1, asym=asym)
    x = (torch.randn((2, tokens // 2, hidden), generator=torch.Generator().manual_seed(3))).half().to(DEV)
    y1, logits1 = blk(x)
    y2, logits2 = _per_expert_loop(blk, x)
    assert torch.equal(logits1, logits2)
    if top_k <= 2:
        assert torch.equal(y1, y2)
    else:   # more than two addends: the combine kernel sums in fp32 and rounds once, the tensor chain per pair
        assert rel_l2(y1.cpu(), y2.cpu()) <= 1e-3
    assert y1.shape == x.shape and torch.isfinite(y1).all()


def test_block_accepts_other_dtypes_and_fp32_rotation():
    """bf16 hidden states are cast around the fp16 kernels; `fp32_had` takes the unfused rotation."""
    blk = _block(8, 256, 768, 2, 9)
    x = torch.randn((1, 12, 256), generator=torch.Generator().manual_seed(1)).half().to(DEV)
    y16, _ = blk(x)
    blk.gate = blk.gate.to(torch.bfloat16)          # the router follows the model dtype
    yb, _ = blk(x.to(torch.bfloat16))
    blk.gate = blk.gate.to(torch.float16)
    # bf16 inputs and router: a different rounding of x and of the logits, possibly a different expert for a token
    assert yb.dtype == torch.bfloat16 and torch.isfinite(yb).all() and rel_l2(yb.float().cpu(), y16.float().cpu()) <= 0.5
    blk.fp32_had = True
    blk.had_K = blk.had_K.float()
    y32, _ = blk(x)
    assert rel_l2(y32.cpu(), y16.cpu()) <= 5e-2


def _packed_block(E, hidden, inter, top_k, seed):
    """Like _block, for big geometries: packed weight bytes drawn directly."""
    g = torch.Generator().manual_seed(seed)
    def w(n, k):
        return torch.randint(0, 256, (E, n, k // 2), generator=g, dtype=torch.uint8)
    def s(n, k):
        return (torch.rand((E, n), generator=g) * 0.5 / k + 0.5 / k).half()
    gate = torch.nn.Linear(hidden, E, bias=False).half()
    gate.weight.data = torch.randn((E, hidden), generator=g).half()
    sg = (torch.randint(0, 2, (E, inter), generator=g) * 2 - 1).to(torch.int8)
    return snn.SignRotMoEBlock(gate.to(DEV), top_k=top_k, norm_topk_prob=True,
                               w_gate=w(inter, hidden).to(DEV), s_gate=s(inter, hidden).to(DEV),
                               w_up=w(inter, hidden).to(DEV), s_up=s(inter, hidden).to(DEV),
                               w_down=w(hidden, inter).to(DEV), s_down=s(hidden, inter).to(DEV), sign_down=sg.to(DEV))


@pytest.mark.parametrize("E,hidden,inter,top_k,tokens", [(8, 256, 768, 2, 24), (8, 4096, 14336, 2, 64)],
                         ids=["small", "mixtral-8x7b-shape"])
def test_block_against_integer_oracle(E, hidden, inter, top_k, tokens):
    """The sparse block against the oracle's integer statement of it, expert by expert: quantizer, gate/up
    GEMMs, SwiGLU, sign-adjusted rotation, quantizer, down GEMM, routing-weighted sum
    (signrot/nn/moe.py:167-235).  Routing decisions are taken from the block's own logits."""
    blk = _block(E, hidden, inter, top_k, 2) if hidden <= 512 else _packed_block(E, hidden, inter, top_k, 2)
    g = torch.Generator().manual_seed(4)
    x = torch.randn((1, tokens, hidden), generator=g).half()
    y, logits = blk(x.to(DEV))
    hadK, K = get_hadK(inter)
    cpu = lambda a: a.cpu()
    want = oracle.moe_block(x.view(-1, hidden), logits.cpu(), top_k, True, cpu(blk.w_gate), cpu(blk.s_gate),
                            cpu(blk.w_up), cpu(blk.s_up), cpu(blk.w_down), cpu(blk.s_down), cpu(blk.sign_down), hadK, K)
    err = rel_l2(y.cpu().view(-1, hidden), want)
    assert err <= 1e-3, err


def test_cuda_graph_replay():
    blk = _block(8, 256, 192, 2, 5)
    static_x = torch.zeros((1, 16, 256), dtype=torch.float16, device=DEV)
    for _ in range(2):
        blk(static_x)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_y, _ = blk(static_x)
    for seed in (1, 2):
        x = torch.randn((1, 16, 256), generator=torch.Generator().manual_seed(seed)).half().to(DEV)
        static_x.copy_(x)
        graph.replay()
        torch.cuda.synchronize()
        eager, _ = blk(x)
        assert torch.equal(static_y, eager)


@pytest.mark.parametrize("counts,N,K", [
    ([5, 0, 300, 1, 0, 257, 64, 0], 320, 256),      # empty experts, several m-tiles, ragged N
    ([0, 0, 700], 256, 4096),                       # leading empty experts
    ([130] * 16, 768, 512),
    ([1, 2, 3, 4], 40, 64),
    ([40, 0, 3, 1, 0, 0, 20, 0], 4096, 512),        # an expert with more rows than one pass of the decode kernel
])
@pytest.mark.parametrize("asym", [False, True])
def test_grouped_linear_bit_exact(counts, N, K, asym):
    """One launch for all experts == per-expert integer GEMM + expert-indexed dequant; the cases reach both grouped
    kernels (weight streaming for at most 16 rows per expert on average, CTA-pair tcgen05 above)."""
    from signrot_b200 import _lib
    E, rows = len(counts), sum(counts)
    g = torch.Generator().manual_seed(rows + N)
    lo, hi = (0, 16) if asym else (-8, 8)
    a = torch.randint(lo, hi, (rows, K), generator=g, dtype=torch.int32)
    w = torch.randint(-8, 8, (E, N, K), generator=g, dtype=torch.int32)
    A = oracle.pack_codes(a) if asym else oracle.pack_i4(a)
    W = oracle.pack_i4(w.view(E * N, K)).view(E, N, K // 2)
    sa = (torch.rand((rows,), generator=g) * 0.1 + 0.01).half()
    sw = (torch.rand((E, N), generator=g) * 0.1 + 0.01).half()
    eid = torch.repeat_interleave(torch.arange(E, dtype=torch.int32), torch.tensor(counts))
    off = torch.zeros(E + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(torch.tensor(counts), 0)
    zero = torch.randint(0, 16, (rows,), generator=g, dtype=torch.int32).to(torch.int8) if asym else None
    wsum = w.sum(-1).to(torch.int32) if asym else None
    acc = torch.empty((rows, N), dtype=torch.int32)
    for e in range(E):
        sl = slice(int(off[e]), int(off[e + 1]))
        acc[sl] = a[sl] @ w[e].T
    want = oracle.sym_dequant_moe(acc, sa.view(-1, 1), sw, eid, zero, wsum)
    pk = kernel.PackedQuantizedTensor(A.to(DEV), sa.to(DEV), zero.to(DEV) if asym else None)
    got = kernel.grouped_linear(pk, eid.to(DEV), off.to(DEV), W.to(DEV), sw.to(DEV), wsum.to(DEV) if asym else None)
    assert _lib.device_status() == 0
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("T,E,k,renorm", [(64, 8, 2, True), (5, 4, 1, True), (300, 128, 8, True), (33, 16, 4, False),
                                          (1, 8, 2, True), (2000, 8, 2, True)])
def test_moe_route_matches_the_tensor_chain(T, E, k, renorm):
    """One-launch routing against softmax / topk / stable argsort (signrot/nn/moe.py:159-190)."""
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn((T, E), generator=g).half().to(DEV)
    w, chosen, tok, eid, inv, row_off = kernel.moe_route(logits, k, renorm)
    probs = torch.softmax(logits, dim=1, dtype=torch.float)
    pw, sel = torch.topk(probs, k, dim=-1)
    if renorm:
        pw = pw / pw.sum(dim=-1, keepdim=True)
    # equal fp16 logits are common among 128 experts: the chosen experts may differ there, their
    # probabilities may not
    picked = probs.gather(1, chosen.long())
    assert torch.equal(picked, torch.topk(probs, k, dim=-1)[0])
    assert bool((chosen.long().sort(dim=1)[0].diff(dim=1) != 0).all()) or k == 1     # k distinct experts
    ulp = pw.abs() * 2 ** -10 + 2 ** -24
    assert bool(((w.float() - pw.half().float()).abs() <= ulp).all())
    flat = chosen.long().reshape(-1)
    perm = torch.argsort(flat, stable=True)
    assert torch.equal(tok.long(), perm // k)
    assert torch.equal(eid.long(), flat[perm])
    assert torch.equal(inv.long(), torch.argsort(perm))
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(row_off.long(), torch.cat([counts.new_zeros(1), counts.cumsum(0)]))


def test_moe_route_survives_non_finite_logits():
    """An overflowed router (inf, NaN in the fp16 logits) still routes every token to k DISTINCT valid experts, places
    every routed row, and the gather / combine that follow stay inside their buffers."""
    T, E, k, hid = 40, 8, 2, 256
    g = torch.Generator().manual_seed(3)
    logits = torch.randn((T, E), generator=g).half()
    logits[3, 2] = float("inf")
    logits[5, :] = float("nan")
    logits[7, 1] = float("nan")
    logits[9, 6] = float("-inf")
    logits[11, :] = float("inf")
    logits[13, :] = float("-inf")
    w, chosen, tok, eid, inv, row_off = kernel.moe_route(logits.to(DEV), k, True)
    torch.cuda.synchronize()
    c = chosen.cpu().long()
    assert bool(((c >= 0) & (c < E)).all()) and bool((c[:, 0] != c[:, 1]).all())
    assert c[3, 0] == 2 and c[7, 0] == 1 and 6 not in c[9].tolist()
    assert torch.isfinite(w.float()).all()
    assert int(row_off[-1]) == T * k and bool((row_off.cpu().diff() >= 0).all())
    assert sorted(tok.cpu().tolist()) == sorted(list(range(T)) * k)
    assert sorted(inv.cpu().tolist()) == list(range(T * k))
    assert bool(((eid.cpu() >= 0) & (eid.cpu() < E)).all())
    x = torch.randn((T, hid), generator=g).half().to(DEV)
    routed = kernel.moe_gather(kernel.PackedQuantizedTensor(*kernel.sym_quant_dynamic(x)), tok)
    y = torch.randn((T * k, hid), generator=g).half().to(DEV)
    out = kernel.moe_combine(y, w, inv)
    torch.cuda.synchronize()
    assert routed.quantized_x.shape[0] == T * k and torch.isfinite(out).all()


def test_moe_route_breaks_ties_by_index():
    logits = torch.zeros((3, 8), dtype=torch.float16, device=DEV)
    logits[1, 5] = 1.0
    w, chosen, tok, eid, inv, row_off = kernel.moe_route(logits, 2, True)
    assert chosen.tolist() == [[0, 1], [5, 0], [0, 1]]
    assert row_off.tolist() == [0, 3, 5, 5, 5, 5, 6, 6, 6]


@pytest.mark.parametrize("asym", [False, True])
def test_moe_gather_and_combine(asym):
    T, k, hid = 37, 2, 512
    g = torch.Generator().manual_seed(5)
    x = torch.randn((T, hid), generator=g).half().to(DEV)
    if asym:
        q, s, z = kernel.asym_quant_dynamic(x)
        packed = kernel.PackedQuantizedTensor(q, s, z.to(torch.int8))
    else:
        q, s = kernel.sym_quant_dynamic(x)
        packed = kernel.PackedQuantizedTensor(q, s)
    logits = torch.randn((T, 8), generator=g).half().to(DEV)
    w, chosen, tok, eid, inv, row_off = kernel.moe_route(logits, k, True)
    routed = kernel.moe_gather(packed, tok)
    assert torch.equal(routed.quantized_x, packed.quantized_x[tok.long()])
    assert torch.equal(routed.scales_x, packed.scales_x[tok.long()])
    assert (routed.zeros_x is None) == (not asym)
    if asym:
        assert torch.equal(routed.zeros_x, packed.zeros_x[tok.long()])
    y = torch.randn((T * k, hid), generator=g).half().to(DEV)
    got = kernel.moe_combine(y, w, inv)
    want = (y[inv.long()].view(T, k, hid) * w.unsqueeze(-1)).sum(dim=1)
    assert torch.equal(got, want)                          # two addends: one rounding either way


@torch.no_grad()
def test_build_moe_block_from_per_expert_linears():
    """Per-expert KernelLinear triples behind a host loop -> stacked SignRotMoEBlock: same output as running
    each routed token through its experts one by one."""
    from types import SimpleNamespace
    from signrot_b200.transformers import kernel_utils as ku
    E, hid, ffn, k, T = 4, 256, 768, 2, 19
    g = torch.Generator().manual_seed(21)

    def lin(i, o, **kw):
        m = ku.KernelLinear(i, o, **kw).to(DEV)
        m.kernel_module.weight.copy_(torch.randint(0, 256, (o, i // 2), generator=g, dtype=torch.uint8))
        m.kernel_module.weight_scales = ((torch.rand((o, 1), generator=g) * 0.5 + 0.5) / i).half().to(DEV)
        return m
    experts = []
    for _ in range(E):
        down = lin(ffn, hid, online_full_had=True, had_adj=True)
        down.kernel_hadamard.had_adj_sign.copy_((torch.randint(0, 2, (ffn,), generator=g) * 2 - 1).to(torch.int8))
        experts.append(SimpleNamespace(gate_proj=lin(hid, ffn), up_proj=lin(hid, ffn), down_proj=down))
    gate = torch.nn.Linear(hid, E, bias=False).half().to(DEV)
    gate.weight.data = torch.randn((E, hid), generator=g).half().to(DEV)
    mlp = SimpleNamespace(experts=experts, gate=gate, top_k=k, norm_topk_prob=True)
    blk = ku.build_moe_block(mlp)
    assert blk is not None and blk.num_experts == E and blk.sign_down.shape == (E, ffn)
    x = torch.randn((1, T, hid), generator=g).half().to(DEV)
    y, logits = blk(x)
    probs = torch.softmax(logits.float(), dim=1)
    pw, sel = torch.topk(probs, k, dim=-1)
    pw = (pw / pw.sum(-1, keepdim=True)).half()
    want = torch.zeros((T, k, hid), dtype=torch.float16, device=DEV)
    for t in range(T):
        for j in range(k):
            e = experts[int(sel[t, j])]
            xt = x[0, t:t + 1]
            inter = kernel.swiglu(e.gate_proj(xt), e.up_proj(xt))
            want[t, j] = e.down_proj(inter)[0]
    want = (want * pw.unsqueeze(-1)).sum(dim=1)
    assert rel_l2(y.view(T, hid).cpu(), want.cpu()) <= 1e-3
    experts[0].gate_proj.use_kernel = False
    assert ku.build_moe_block(mlp) is None
