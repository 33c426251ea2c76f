"""int4 paged KV cache and decode attention against the oracle; cases follow
benchmarks/test_split_decode.py:57-92 (T in {1024, 1000, 513, 256, 2048}, page 128/256)."""
import math

import pytest
import torch

import oracle
from signrot_b200 import _lib
from signrot_b200.functional import kernel
from signrot_b200.transformers import kv_cache as kvc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _fill(B, L, Hkv, page, T, seed, hadamard=True):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn((B, T, Hkv, 128), generator=g).half()
    v = torch.randn((B, T, Hkv, 128), generator=g).half()
    pages = (T + 1 + page - 1) // page + 1
    ref = oracle.PagedCacheRef(B, L, Hkv, page, pages, hadamard=hadamard)
    return k, v, ref, pages


@pytest.mark.parametrize("T,page,Hq,Hkv", [(1024, 128, 8, 8), (1000, 256, 8, 2), (513, 128, 32, 8), (256, 256, 4, 4),
                                           (2048, 256, 32, 8), (1, 16, 8, 8), (17, 16, 16, 2)])
def test_fused_append_and_decode(T, page, Hq, Hkv):
    B, L, layer = 3, 2, 1
    k, v, ref, pages = _fill(B, L, Hkv, page, T, T)
    ref.append(layer, k, v)
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 8, DEV, L, Hkv, 128, group_size=Hq // Hkv)
    # prefill through the cache object (layer 0 first: it advances the length)
    cache.update(k.to(DEV), v.to(DEV), 0)
    out = cache.update(k.to(DEV), v.to(DEV), layer)
    assert isinstance(out, tuple)
    indptr, indices, last = ref.specs(layer)
    P = indptr[1].item()
    got_data = cache.pages[: P * B, layer].cpu()
    got_param = cache.scales[: P * B, layer].cpu()
    # compare only written slots
    for b in range(B):
        for pos in (0, T // 2, T - 1):
            pg, e = (pos // page) * B + b, pos % page
            assert torch.equal(got_data[pg, :, :, e], ref.data[pg, layer, :, :, e])
            assert torch.equal(got_param[pg, :, :, e], ref.param[pg, layer, :, :, e])
    # decode one token
    g = torch.Generator().manual_seed(5)
    k1 = torch.randn((B, 1, Hkv, 128), generator=g).half()
    v1 = torch.randn((B, 1, Hkv, 128), generator=g).half()
    q = torch.randn((B, 1, Hq, 128), generator=g).half()
    ref.append(layer, k1, v1)
    cache.update(k1.to(DEV), v1.to(DEV), 0)
    attend = cache.update(k1.to(DEV), v1.to(DEV), layer)
    o = attend(q.to(DEV)).cpu().view(B, Hq, 128)
    kf, vf = ref.dense(layer)
    want = oracle.decode_attention_ref(q.view(B, Hq, 128), kf, vf, hadamard_q=True)
    assert (o.float() - want).abs().max().item() <= 3e-2
    # split-KV vs unsplit (2e-3), through the module-level entry point
    specs = cache.refresh_specs()
    qd = q.view(B, Hq, 128).to(DEV).contiguous()
    o1 = torch.empty_like(qd)
    kvc.batch_decode_i4(o1, qd, **specs, layer_idx=layer, hadamard_q=True)
    for chunks in (2, 3, 7, 12):     # up to 8: merged inside a cluster; more: the separate merge launch
        tmp = torch.empty((B, Hq, chunks, 132), dtype=torch.float32, device=DEV)
        o2 = torch.empty_like(qd)
        kvc.batch_decode_i4(o2, qd, **specs, layer_idx=layer, tmp=tmp, num_chunks=chunks, hadamard_q=True)
        assert (o1.float() - o2.float()).abs().max().item() <= 2e-3


def test_decode_attention_benchmark_geometry():
    """Batch 16, 4096 cached tokens + 1 new, page 256 (17 pages per request), 32 q / 8 kv heads: cache bytes
    of every slot and the decode output against the oracle (3e-2 vs fp32 attention over the dequantized
    cache; 2e-3 between the cache object's split-KV schedule and one unsplit pass)."""
    B, L, Hq, Hkv, page, T = 16, 1, 32, 8, 256, 4096
    g = torch.Generator().manual_seed(11)
    k = torch.randn((B, T + 1, Hkv, 128), generator=g).half()
    v = torch.randn((B, T + 1, Hkv, 128), generator=g).half()
    q = torch.randn((B, 1, Hq, 128), generator=g).half()
    ref = oracle.PagedCacheRef(B, L, Hkv, page, 18)
    ref.append(0, k[:, :T], v[:, :T])
    ref.append(0, k[:, T:], v[:, T:])
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 64, DEV, L, Hkv, 128, group_size=Hq // Hkv)
    cache.update(k[:, :T].contiguous().to(DEV), v[:, :T].contiguous().to(DEV), 0)
    attend = cache.update(k[:, T:].contiguous().to(DEV), v[:, T:].contiguous().to(DEV), 0)
    o = attend(q.to(DEV)).cpu().view(B, Hq, 128)
    used = 17 * B
    assert torch.equal(cache.pages[:used, 0].cpu()[:16 * B], ref.data[:16 * B, 0])          # full pages
    assert torch.equal(cache.pages[16 * B:used, 0, :, :, :1].cpu(), ref.data[16 * B:used, 0, :, :, :1])
    assert torch.equal(cache.scales[:used, 0].cpu()[:16 * B], ref.param[:16 * B, 0])
    kf, vf = ref.dense(0)
    want = oracle.decode_attention_ref(q.view(B, Hq, 128), kf, vf, hadamard_q=True)
    err = (o.float() - want).abs().max().item()
    assert err <= 3e-2, err
    specs = cache.refresh_specs()
    qd = q.view(B, Hq, 128).to(DEV).contiguous()
    o1 = torch.empty_like(qd)
    kvc.batch_decode_i4(o1, qd, **specs, layer_idx=0, hadamard_q=True)
    assert (o1.float().cpu() - o.float()).abs().max().item() <= 2e-3
    assert (o1.float().cpu() - want).abs().max().item() <= 3e-2


def test_prequantized_init_append_roundtrip():
    """init_kv_i4 / append_kv_i4 with codes from kv_quant_pack (the reference's unfused chain)."""
    B, L, H, page, T = 2, 1, 4, 16, 37
    g = torch.Generator().manual_seed(0)
    k = torch.randn((B, T, H, 128), generator=g).half().to(DEV)
    v = torch.randn((B, T, H, 128), generator=g).half().to(DEV)
    kq, kp = kernel.kv_quant_pack(k)
    vq, vp = kernel.kv_quant_pack(v)
    pages = (T + 1 + page - 1) // page
    data = torch.zeros((pages * B, L, 2, H, page, 64), dtype=torch.uint8, device=DEV)
    param = torch.zeros((pages * B, L, 2, H, page, 2), dtype=torch.float16, device=DEV)
    def specs(n):
        pc = (n + page - 1) // page
        last = n % page or page
        idx = (torch.arange(pc, dtype=torch.int32) * B).unsqueeze(0) + torch.arange(B, dtype=torch.int32).unsqueeze(1)
        return dict(kv_indptr=(torch.arange(B + 1, dtype=torch.int32) * pc).to(DEV), kv_indices=idx.reshape(-1).to(DEV),
                    last_page_offset=torch.full((B,), last, dtype=torch.int32, device=DEV))
    seq = (torch.arange(B + 1, dtype=torch.int32) * T).to(DEV)
    kvc.init_kv_i4(data, param, **specs(T), k=kq.view(-1, H, 64), v=vq.view(-1, H, 64), k_param=kp.view(-1, H, 2),
                   v_param=vp.view(-1, H, 2), seqlen_indptr=seq, layer_idx=0)
    k1 = torch.randn((B, 1, H, 128), generator=g).half().to(DEV)
    k1q, k1p = kernel.kv_quant_pack(k1)
    kvc.append_kv_i4(data, param, **specs(T + 1), k=k1q.view(B, H, 64), v=k1q.view(B, H, 64), k_param=k1p.view(B, H, 2),
                     v_param=k1p.view(B, H, 2), layer_idx=0)
    for b in range(B):
        for pos in (0, 15, 16, T - 1):
            pg, e = (pos // page) * B + b, pos % page
            assert torch.equal(data[pg, 0, 0, :, e], kq[b, pos]) and torch.equal(data[pg, 0, 1, :, e], vq[b, pos])
            assert torch.equal(param[pg, 0, 0, :, e], kp[b, pos]) and torch.equal(param[pg, 0, 1, :, e], vp[b, pos])
        pg, e = (T // page) * B + b, T % page
        assert torch.equal(data[pg, 0, 0, :, e], k1q[b, 0]) and torch.equal(param[pg, 0, 1, :, e], k1p[b, 0])
    # the fused path writes the same bytes
    data2, param2 = torch.zeros_like(data), torch.zeros_like(param)
    kvc.kv_append_quant(data2, param2, **specs(T), k=k, v=v, layer_idx=0, hadamard_k=False)
    kvc.kv_append_quant(data2, param2, **specs(T + 1), k=k1, v=k1, layer_idx=0, hadamard_k=False)
    assert torch.equal(data2, data) and torch.equal(param2, param)


def test_cache_reset_and_graph_friendly_specs():
    B, page, H = 2, 16, 2
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, 64, DEV, 1, H, 128)
    ptrs = {k: v.data_ptr() for k, v in cache.refresh_specs().items()}
    k = torch.randn((B, 20, H, 128), device=DEV).half()
    cache.update(k, k, 0)
    assert cache.get_seq_length() == 20 and cache.seen_tokens == 20
    cache.update(k[:, :1], k[:, :1], 0)
    assert cache.get_seq_length() == 21
    assert {k_: v.data_ptr() for k_, v in cache.refresh_specs().items()} == ptrs
    cache.reset()
    assert cache.get_seq_length() == 0
    assert isinstance(cache.update(k, k, 0), tuple)


@pytest.mark.parametrize("T,start,fused_input", [(1, 37, True), (1, 0, False), (20, 0, True), (33, 0, False)])
def test_rope_kv_append_equals_rope_then_append(T, start, fused_input):
    """One launch for rotary embedding + K rotation + K/V quantizers + page scatter: same cache
    bytes and same rotated q as `rope_qk` followed by `update`; q/k/v may be column ranges of one
    fused projection output."""
    B, Hq, Hkv, D, page, L = 3, 8, 2, 128, 16, 2
    g = torch.Generator().manual_seed(T * 7 + start)
    total = (Hq + 2 * Hkv) * D
    qkv = torch.randn((B, T, total), generator=g).half().to(DEV)
    q = qkv[..., :Hq * D].unflatten(-1, (Hq, D))
    k = qkv[..., Hq * D:(Hq + Hkv) * D].unflatten(-1, (Hkv, D))
    v = qkv[..., (Hq + Hkv) * D:].unflatten(-1, (Hkv, D))
    if not fused_input:
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    ang = torch.rand((1, T, D), generator=g) * 6.0
    cos, sin = ang.cos().half().to(DEV), ang.sin().half().to(DEV)

    def fresh():
        c = kvc.MultiLayerPagedKVCache4Bit(B, page, start + T + 4, DEV, L, Hkv, D, group_size=Hq // Hkv)
        if start:
            pk = torch.randn((B, start, Hkv, D), generator=torch.Generator().manual_seed(1)).half().to(DEV)
            for layer in range(L):
                c.update(pk, pk, layer)
        return c
    a, b = fresh(), fresh()
    layer = 1
    # reference route: rope in place on copies, then the fused append
    q2, k2 = q.contiguous().clone(), k.contiguous().clone()
    kernel.rope_qk(q2, k2, cos, sin)
    a.update(k2, v.contiguous(), 0)
    out_a = a.update(k2, v.contiguous(), layer)
    q_rot, _ = b.update_with_rope(q, k, v, cos, sin, 0)
    q_rot, out_b = b.update_with_rope(q, k, v, cos, sin, layer)
    assert torch.equal(q_rot, q2)
    if start == 0:
        assert isinstance(out_a, tuple) and isinstance(out_b, tuple)
        assert torch.equal(out_b[0], k2) and torch.equal(out_b[1], v)
    else:
        assert callable(out_b)
        assert torch.equal(out_b(q_rot), out_a(q2))
    pages = a.page_cnt_from_length(start + T) * B
    # slots past the sequence end are never written: compare through a decode-independent mask
    pa, pb = a.pages[:pages, layer], b.pages[:pages, layer]
    sa, sb = a.scales[:pages, layer], b.scales[:pages, layer]
    n = start + T
    for pos in range(start, n):
        for bb in range(B):
            pg, e = (pos // page) * B + bb, pos % page
            assert torch.equal(pa[pg, :, :, e], pb[pg, :, :, e]) and torch.equal(sa[pg, :, :, e], sb[pg, :, :, e])


@pytest.mark.parametrize("T,page,Hq,Hkv,chunks", [(513, 128, 32, 8, 3), (1000, 16, 8, 2, 7), (300, 32, 4, 4, 2),
                                                  (1000, 16, 8, 2, 12), (2100, 256, 32, 8, 5)])
def test_in_kernel_merge_equals_merge_pass(T, page, Hq, Hkv, chunks):
    """Three ways to merge the split-KV states give the same bits: inside the cluster that the chunks of a
    (request, KV head) form (the default up to 8 chunks), the separate merge launch (more chunks), and the last CTA
    behind arrival counters, which are back at zero after every call."""
    B, L = 3, 1
    k, v, ref, pages = _fill(B, L, Hkv, page, T, T + 1)
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 8, DEV, L, Hkv, 128, group_size=Hq // Hkv)
    cache.update(k.to(DEV), v.to(DEV), 0)
    specs = cache.refresh_specs()
    g = torch.Generator().manual_seed(3)
    tmp = torch.empty((B, Hq, chunks, 132), dtype=torch.float32, device=DEV)
    counters = torch.zeros(B * Hkv, dtype=torch.int32, device=DEV)
    for _ in range(3):
        q = torch.randn((B, Hq, 128), generator=g).half().to(DEV)
        a, b = torch.empty_like(q), torch.empty_like(q)
        kvc.batch_decode_i4(a, q, **specs, layer_idx=0, tmp=tmp, num_chunks=chunks, hadamard_q=True)
        kvc.batch_decode_i4(b, q, **specs, layer_idx=0, tmp=tmp, num_chunks=chunks, hadamard_q=True, counters=counters)
        assert torch.equal(a, b)
        assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("chunks", [1, 2, 4, 3])
def test_large_batch_takes_the_four_warp_form(chunks):
    """More CTAs than fit the GPU at two per SM (batch 40 x 8 KV heads x chunks): the kernel runs with four warps per
    CTA.  Against fp32 attention over the dequantized cache, split against unsplit, cluster merge against the counter
    merge, and the one-launch decode step against its two launches."""
    B, L, Hq, Hkv, page, T = 40, 1, 32, 8, 64, 200
    k, v, ref, pages = _fill(B, L, Hkv, page, T, T + 1)
    ref.append(0, k, v)
    caches = []
    for fuse in (False, True):
        c = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 8, DEV, L, Hkv, 128, group_size=Hq // Hkv, decode_chunks=chunks)
        c.fuse_decode = fuse
        c.pages.zero_()
        c.scales.zero_()
        c.update(k.to(DEV), v.to(DEV), 0)
        caches.append(c)
    specs = caches[0].refresh_specs()
    g = torch.Generator().manual_seed(11)
    q = torch.randn((B, Hq, 128), generator=g).half().to(DEV)
    kf, vf = ref.dense(0)
    want = oracle.decode_attention_ref(q.cpu(), kf, vf, hadamard_q=True)
    one = torch.empty_like(q)
    kvc.batch_decode_i4(one, q, **specs, layer_idx=0, hadamard_q=True)
    assert (one.float().cpu() - want).abs().max().item() <= 3e-2
    if chunks > 1:
        tmp = torch.empty((B, Hq, chunks, 132), dtype=torch.float32, device=DEV)
        counters = torch.zeros(B * Hkv, dtype=torch.int32, device=DEV)
        a, b = torch.empty_like(q), torch.empty_like(q)
        kvc.batch_decode_i4(a, q, **specs, layer_idx=0, tmp=tmp, num_chunks=chunks, hadamard_q=True)
        kvc.batch_decode_i4(b, q, **specs, layer_idx=0, tmp=tmp, num_chunks=chunks, hadamard_q=True, counters=counters)
        assert torch.equal(a, b) and int(counters.abs().sum()) == 0
        assert (a.float() - one.float()).abs().max().item() <= 2e-3
    qkv = torch.randn((B, 1, (Hq + 2 * Hkv) * 128), generator=g).half().to(DEV)
    q1 = qkv[..., :Hq * 128].unflatten(-1, (Hq, 128))
    k1 = qkv[..., Hq * 128:(Hq + Hkv) * 128].unflatten(-1, (Hkv, 128))
    v1 = qkv[..., (Hq + Hkv) * 128:].unflatten(-1, (Hkv, 128))
    ang = torch.rand((1, 1, 128), generator=g) * 6.28
    cos, sin = ang.cos().half().to(DEV), ang.sin().half().to(DEV)
    outs = []
    for c in caches:
        q_in, attend = c.update_with_rope(q1, k1, v1, cos, sin, 0, defer_append=True)
        outs.append(attend(q_in))
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(caches[0].pages, caches[1].pages) and torch.equal(caches[0].scales, caches[1].scales)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("T,page,Hq,Hkv,chunks,per_request_cos", [(2100, 256, 32, 8, None, False), (513, 128, 32, 8, 3, True),
                                                                  (1000, 16, 8, 2, 12, False), (300, 32, 4, 4, 1, True),
                                                                  (255, 256, 16, 2, None, False), (256, 256, 8, 8, 2, True),
                                                                  (40, 16, 8, 2, 4, False), (70, 64, 8, 8, 4, True)])
def test_decode_step_in_one_launch_equals_two(T, page, Hq, Hkv, chunks, per_request_cos):
    """Rotary embedding + K/V append + attention as one launch (`rope_decode_i4`) against `rope_kv_append` followed
    by `batch_decode_i4`: same attention output, same cache bytes, for three decode steps in a row (the second and
    third read what the first appended; T = 255 / 256 put the new token at the end of a page / on a new page; T = 40 and
    70 with 4 chunks leave the last chunk of the cluster without a block, so the new token belongs to the third), with
    q / k / v as column ranges of one fused projection output."""
    B, L = 3, 2
    k, v, ref, pages = _fill(B, L, Hkv, page, T, T + 4)
    caches = []
    for fuse in (False, True):
        c = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 8, DEV, L, Hkv, 128, group_size=Hq // Hkv, decode_chunks=chunks)
        c.fuse_decode = fuse
        c.pages.zero_()          # the pools come from torch.empty: make the never-written slots comparable
        c.scales.zero_()
        for layer in range(L):
            c.update(k.to(DEV), v.to(DEV), layer)
        caches.append(c)
    g = torch.Generator().manual_seed(17)
    for step in range(3):
        qkv = torch.randn((B, 1, (Hq + 2 * Hkv) * 128), generator=g).half().to(DEV)
        q = qkv[..., :Hq * 128].unflatten(-1, (Hq, 128))
        kk = qkv[..., Hq * 128:(Hq + Hkv) * 128].unflatten(-1, (Hkv, 128))
        vv = qkv[..., (Hq + Hkv) * 128:].unflatten(-1, (Hkv, 128))
        ang = torch.rand((B if per_request_cos else 1, 1, 128), generator=g) * 6.28
        cos, sin = ang.cos().half().to(DEV), ang.sin().half().to(DEV)
        outs = []
        for c in caches:
            for layer in range(L):
                q_in, attend = c.update_with_rope(q, kk, vv, cos, sin, layer, defer_append=True)
                out = attend(q_in)
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), f"step {step}"
        assert torch.equal(caches[0].pages, caches[1].pages) and torch.equal(caches[0].scales, caches[1].scales)
    assert _lib.device_status() == 0
