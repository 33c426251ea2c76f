"""Worker of the multi-GPU tensor-parallel check (one process per GPU, NCCL).  Launched by
tests/test_gpu_tp.py, or by hand:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 tests/tp_nccl_worker.py

Every rank builds the same seeded linear, computes the one-GPU result (fused rotation + quantizer,
W4A4 GEMM + dequant) and checks that the column-parallel and the row-parallel (int32 all-reduce)
forms reproduce it bit for bit."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from signrot_b200 import tp  # noqa: E402
from signrot_b200.functional import kernel  # noqa: E402
from signrot_b200.functional.hadamard import get_hadK  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from signrot_b200.comm import PeerGroup
    from signrot_b200 import _lib
    peer = PeerGroup()                               # 2 MB slots: the decode-size cases below go through it
    for (m, k, n) in [(64, 4096, 1024), (200, 14336, 512), (3, 768, 264)]:
        g = torch.Generator().manual_seed(1000 + k)
        x = torch.randn((m, k), generator=g).half().to(dev)
        w = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8).to(dev)
        ws = (torch.rand((n, 1), generator=g) * 0.01 + 0.001).half().to(dev)
        sign = (torch.randint(0, 2, (k,), generator=g) * 2 - 1).to(torch.int8).to(dev)
        hadK, K = get_hadK(k)
        hk = hadK.to(dev, torch.float16) if hadK is not None else None
        packed = kernel.rotate_quant(x, hk, K, sign=sign)
        want = kernel.w4a4_linear(packed, w, ws)

        col = tp.ColumnParallelLinear4bit(w, ws)
        got_c = col.forward(packed, gather_output=True)
        assert torch.equal(got_c, want), f"column-parallel mismatch at {(m, k, n)} on rank {rank}"

        row = tp.RowParallelLinear4bit(w, ws, hadK=hk, K_had=K, sign=sign)
        got_r = row.forward(x[:, row.begin:row.end].contiguous())
        assert torch.equal(got_r, want), f"row-parallel mismatch at {(m, k, n)} on rank {rank}"

        # the same through one-kernel exchanges over peer memory, several times in a row (both buffer parities,
        # and ranks that run ahead of each other)
        row_p = tp.RowParallelLinear4bit(w, ws, hadK=hk, K_had=K, sign=sign, peer=peer)
        x_local = x[:, row_p.begin:row_p.end].contiguous()
        for it in range(5):
            got_p = row_p.forward(x_local)
            assert torch.equal(got_p, want), f"peer-exchange row-parallel mismatch at {(m, k, n)}, call {it}, rank {rank}"
        if rank == 0:
            torch.cuda._sleep(20_000_000)            # one rank falls behind: the others wait inside the exchange
        got_p = row_p.forward(x_local)
        assert torch.equal(got_p, want), f"peer-exchange mismatch after a delayed rank at {(m, k, n)} on rank {rank}"
    # plain gather and fp32 sum
    xs = torch.full((8, 1024), float(rank + 1), dtype=torch.float16, device=dev)
    full = peer.all_gather_cols(xs)
    for r in range(world):
        assert bool((full[:, r * 1024:(r + 1) * 1024] == r + 1).all())
    part = torch.full((64, 4096), 0.5 + rank, dtype=torch.float32, device=dev)
    tot = peer.all_reduce_f32(part)
    assert bool((tot == sum(0.5 + r for r in range(world))).all())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "an exchange gave up waiting"
    dist.barrier()
    peer.close()
    if rank == 0:
        print(f"tp_nccl_worker: OK on {world} ranks")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
