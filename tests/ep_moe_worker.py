"""Worker of the expert-parallel MoE check (one process per GPU, NCCL).  Launched by tests/test_gpu_tp.py, or:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29514 tests/ep_moe_worker.py

Every rank builds the same seeded sparse block, computes the one-GPU output, shards a second copy by experts
and checks that the expert-parallel block (local grouped GEMMs + fp32 all-reduce of the weighted partial sums)
reproduces it bit for bit (top-2: at most two addends per token)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from signrot_b200 import nn as snn  # noqa: E402


def block(E, hidden, inter, top_k, seed, dev, asym):
    g = torch.Generator().manual_seed(seed)
    def w(n, k):
        return torch.randint(0, 256, (E, n, k // 2), generator=g, dtype=torch.uint8).to(dev)
    def s(n, k):
        return (torch.rand((E, n), generator=g) * 0.5 / k + 0.5 / k).half().to(dev)
    gate = torch.nn.Linear(hidden, E, bias=False).half()
    gate.weight.data = torch.randn((E, hidden), generator=g).half()
    sg = (torch.randint(0, 2, (E, inter), generator=g) * 2 - 1).to(torch.int8).to(dev)
    return snn.SignRotMoEBlock(gate.to(dev), top_k=top_k, norm_topk_prob=True, w_gate=w(inter, hidden),
                               s_gate=s(inter, hidden), w_up=w(inter, hidden), s_up=s(inter, hidden),
                               w_down=w(hidden, inter), s_down=s(hidden, inter), sign_down=sg, asym=asym)


@torch.no_grad()
def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from signrot_b200.comm import PeerGroup
    peer = PeerGroup()
    def poison():
        # The rows of other ranks' experts are never written by an expert-parallel block; whatever the allocator hands
        # out for them must not matter.  Leave NaNs in the pool so that the next torch.empty is likely to hold them.
        t = torch.full((48 << 20,), float("nan"), dtype=torch.float16, device=dev)
        del t

    for (E, hidden, inter, tokens, asym) in [(8, 512, 768, 64, False), (8, 512, 768, 700, False), (4, 256, 1536, 33, True),
                                             (4, 256, 14336, 40, False)]:
        full = block(E, hidden, inter, 2, 11, dev, asym)
        ep = block(E, hidden, inter, 2, 11, dev, asym).shard_experts_()
        ep_peer = block(E, hidden, inter, 2, 11, dev, asym).shard_experts_(peer=peer)   # sum through peer memory
        assert ep.w_gate.shape[0] == E // world
        x = torch.randn((1, tokens, hidden), generator=torch.Generator().manual_seed(tokens)).half().to(dev)
        want, logits_a = full(x)
        poison()
        got, logits_b = ep(x)
        assert torch.equal(logits_a, logits_b)
        assert torch.equal(got, want), f"expert-parallel output differs at {(E, hidden, inter, tokens, asym)} on rank {rank}"
        for it in range(3):
            poison()
            got_p, _ = ep_peer(x)
            assert torch.equal(got_p, want), f"peer-exchange expert-parallel output differs, call {it}, rank {rank}"
    if "--time" in sys.argv:
        # Mixtral-shaped block (8 experts of 14336 x 4096, top-2), 64 and 4096 tokens: milliseconds per forward,
        # one GPU against expert-parallel, max over ranks
        for tokens in (64, 4096):
            full = block(8, 4096, 14336, 2, 1, dev, False)
            x = torch.randn((1, tokens, 4096), generator=torch.Generator().manual_seed(1)).half().to(dev)
            res = []
            for blk in (full, None):
                if blk is None:
                    blk = full.shard_experts_(peer=peer)      # shard the same block in place (saves memory)
                for _ in range(3):
                    blk(x)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                dist.barrier()
                e0.record()
                for _ in range(10):
                    blk(x)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / 10], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res.append(t.item())
            if rank == 0:
                print(f"ep_moe_worker: timing tokens={tokens} one_gpu_ms={res[0]:.3f} ep{world}_ms={res[1]:.3f}", flush=True)
            del full, blk
            torch.cuda.empty_cache()
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"ep_moe_worker: OK on {world} ranks", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
