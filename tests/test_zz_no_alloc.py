"""The workspace-free decode entry point, called through the C ABI.

`sr_batch_decode_i4_static` serves hosts that cannot allocate device memory themselves (a
serving process with a fixed memory plan and no allocator for plug-ins, a loop that cannot
afford the synchronisation an allocation implies, a thin foreign-language binding): its
split-KV partials live in a buffer inside the library.  The test calls it twice in
a row (the second call finds the first call's leftovers in that buffer) and checks both results
against the ordinary entry point fed with a caller-allocated workspace.  The file name keeps it
last in collection order, so a failure here cannot hide another test's result under `-x`.
"""
import ctypes

import pytest
import torch

from signrot_b200 import _lib
from signrot_b200.transformers import kv_cache as kvc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _decode_static(o, q, specs, layer, hq, hkv, page, batch, chunks):
    lib = _lib.load()
    rc = lib.sr_batch_decode_i4_static(
        o.data_ptr(), q.data_ptr(), specs["kv_data"].data_ptr(), specs["kv_param"].data_ptr(),
        specs["kv_indptr"].data_ptr(), specs["kv_indices"].data_ptr(), specs["last_page_offset"].data_ptr(),
        specs["kv_data"].size(1), layer, hq, hkv, page, 128, batch, chunks, 1,
        torch.cuda.current_stream().cuda_stream)
    return rc, lib.sr_last_error().decode()


def test_static_workspace_decode_matches_caller_workspace_twice():
    B, Hq, Hkv, page, T, chunks = 4, 8, 2, 64, 500, 5
    g = torch.Generator().manual_seed(11)
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, T + 8, DEV, 1, Hkv, 128, group_size=Hq // Hkv)
    k = torch.randn((B, T, Hkv, 128), generator=g).half().to(DEV)
    v = torch.randn((B, T, Hkv, 128), generator=g).half().to(DEV)
    cache.update(k, v, 0)
    specs = cache.refresh_specs()
    for trial in range(2):
        q = torch.randn((B, Hq, 128), generator=g).half().to(DEV)
        want = torch.empty_like(q)
        tmp = torch.empty((B, Hq, chunks, 132), dtype=torch.float32, device=DEV)
        kvc.batch_decode_i4(want, q, **specs, layer_idx=0, tmp=tmp, num_chunks=chunks, hadamard_q=True)
        got = torch.full_like(q, float("nan"))
        rc, msg = _decode_static(got, q, specs, 0, Hq, Hkv, page, B, chunks)
        assert rc == 0, msg
        torch.cuda.synchronize()
        # same kernels, same chunking, same arithmetic: the same bits (a partial left over from the previous call
        # and read by mistake would show up here)
        assert torch.isfinite(got).all()
        assert torch.equal(got, want), f"call {trial}"


def test_static_workspace_rejects_oversized_requests():
    B, Hq, Hkv, page = 64, 32, 8, 16
    cache = kvc.MultiLayerPagedKVCache4Bit(B, page, 64, DEV, 1, Hkv, 128, group_size=Hq // Hkv)
    k = torch.zeros((B, 32, Hkv, 128), dtype=torch.float16, device=DEV)
    cache.update(k, k, 0)
    q = torch.zeros((B, Hq, 128), dtype=torch.float16, device=DEV)
    o = torch.empty_like(q)
    rc, msg = _decode_static(o, q, cache.refresh_specs(), 0, Hq, Hkv, page, B, 8)  # 64*32*8*132 floats
    assert rc == 3 and "1081344" in msg and "2162688" in msg
    rc, msg = _decode_static(o, q, cache.refresh_specs(), 0, Hq, Hkv, page, B, 1)  # unsplit: no workspace
    assert rc == 0, msg
    torch.cuda.synchronize()
