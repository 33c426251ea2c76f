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
    dist.barrier()
    if rank == 0:
        print(f"tp_nccl_worker: OK on {world} ranks")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
