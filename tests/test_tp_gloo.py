"""Plumbing of the tensor-parallel linears on CPU: two gloo ranks, arithmetic supplied by the
oracle.  Checks that the sharded result is bit-identical to the unsharded one (int32 all-reduce)
and that shard ranges tile the dimension."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def test_shard_range_tiles_the_dimension():
    from signrot_b200.tp import shard_range
    for total, world, align in [(14336, 8, 64), (4096, 3, 64), (1024, 2, 8), (64, 4, 64)]:
        edges = [shard_range(total, r, world, align) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == total
        for (b0, e0), (b1, e1) in zip(edges, edges[1:]):
            assert e0 == b1 and (e0 - b0) % align == 0
    with pytest.raises(ValueError):
        shard_range(100, 0, 2, 64)


class _OracleOps:
    """CPU stand-in for signrot_b200.functional.kernel, built from the oracle (tests only)."""

    def __init__(self):
        import oracle
        from signrot_b200.functional.kernel import PackedQuantizedTensor
        self.o, self.P = oracle, PackedQuantizedTensor

    def rotate_quant(self, x, hadK=None, K=1, sign=None, heads=0, clip_ratio=1.0):
        o = self.o
        rot = o.rotate_heads(x, heads, cast_in_to_f16=True) if heads else \
            o.rotate(x, hadK, K, sign, cast_in_to_f16=True, out_dtype=torch.float16)
        codes, s = o.sym_quant_dynamic(rot, clip_ratio)
        return self.P(o.pack_codes(codes), s)

    def matmul_si4_si4(self, a, b):
        return self.o.matmul_i4(a, b)

    def sym_dequant(self, acc, sr, sc):
        return self.o.sym_dequant(acc, sr, sc)

    def w4a4_linear(self, packed, w, ws):
        return self.o.w4a4_linear(packed.quantized_x, packed.scales_x, w, ws)


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from signrot_b200.tp import RowParallelLinear4bit, ColumnParallelLinear4bit, shard_range
        from signrot_b200.functional.hadamard import get_hadK
        ops = _OracleOps()
        g = torch.Generator().manual_seed(0)
        M, K, N = 6, 768, 40
        x = torch.randn((M, K), generator=g).half()
        w = oracle.pack_i4(torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int32))
        ws = (torch.rand((N, 1), generator=g) * 0.01).half()
        sign = (torch.randint(0, 2, (K,), generator=g) * 2 - 1).to(torch.int8)
        hadK, Kh = get_hadK(K)
        # unsharded answer
        full = ops.rotate_quant(x, hadK, Kh, sign=sign)
        want = oracle.w4a4_linear(full.quantized_x, full.scales_x, w, ws)
        row = RowParallelLinear4bit(w, ws, hadK, Kh, sign=sign, ops=ops)
        b, e = shard_range(K, rank, world, 64)
        got = row.forward(x[:, b:e].contiguous())
        assert torch.equal(got, want), "row-parallel result differs from the unsharded one"
        col = ColumnParallelLinear4bit(w, ws, ops=ops)
        got = col.forward(full, gather_output=True)
        assert torch.equal(got, want), "column-parallel result differs from the unsharded one"
        (Path(out_dir) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_tp_linears_two_ranks(tmp_path):
    world, port = 2, 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_decoder_head_slices_match_row_shards():
    """The tensor-parallel decoder slices q/k/v by heads and gate/up by MLP width; the row-parallel o_proj and
    down_proj of the same rank must own exactly the input channels those slices produce."""
    from signrot_b200.tp import shard_range
    for heads, kv_heads, d, ffn, world in [(32, 8, 128, 14336, 2), (32, 8, 128, 14336, 4), (32, 8, 128, 14336, 8),
                                           (8, 4, 128, 3072, 2)]:
        for rank in range(world):
            ql = heads // world * d
            assert shard_range(heads * d, rank, world, 64) == (rank * ql, (rank + 1) * ql)
            fl = ffn // world
            assert shard_range(ffn, rank, world, 64) == (rank * fl, (rank + 1) * fl)
            assert (kv_heads // world) * world == kv_heads


def _ep_worker(rank, world, port, out_dir):
    """Expert parallelism on CPU: routing replicated, each rank adds the weighted outputs of its own experts' rows
    (a contiguous range of the expert-sorted rows), fp32 all-reduce; equals the unsharded weighted sum."""
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        T, E, k, hid = 37, 8, 2, 64
        logits = torch.randn((T, E), generator=g).half()
        probs = torch.softmax(logits.float(), dim=1)
        pw, sel = torch.topk(probs, k, dim=-1)
        w = (pw / pw.sum(-1, keepdim=True)).half()
        flat = sel.reshape(-1)
        perm = torch.argsort(flat, stable=True)
        inv = torch.argsort(perm)
        counts = torch.bincount(flat, minlength=E)
        row_off = torch.cat([counts.new_zeros(1), counts.cumsum(0)])
        y = torch.randn((T * k, hid), generator=g).half()            # expert outputs in sorted row order
        want = (y[inv].view(T, k, hid) * w.unsqueeze(-1)).sum(dim=1)
        per = E // world
        lo, hi = int(row_off[rank * per]), int(row_off[(rank + 1) * per])
        part = torch.zeros((T, hid), dtype=torch.float32)
        for t in range(T):
            for j in range(k):
                r = int(inv[t * k + j])
                if lo <= r < hi:
                    part[t] += (y[r].float() * w[t, j].float()).half().float()
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        assert torch.equal(part.half(), want), "expert-parallel sum differs from the unsharded one"
        covered = [(int(row_off[r * per]), int(row_off[(r + 1) * per])) for r in range(world)]
        assert covered[0][0] == 0 and covered[-1][1] == T * k and all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
        (Path(out_dir) / f"ep{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


def test_expert_parallel_sum_two_ranks(tmp_path):
    world, port = 2, 29900 + os.getpid() % 90
    mp.spawn(_ep_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ep{r}").exists() for r in range(world))
