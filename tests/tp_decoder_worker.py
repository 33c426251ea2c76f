"""Worker of the tensor-parallel decoder check (one process per GPU, NCCL).  Launched by
tests/test_gpu_tp.py, or by hand:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29512 tests/tp_decoder_worker.py [--time]

Every rank builds the same seeded decoder, computes the one-GPU logits (prefill, then decode steps), shards
a second copy of the model and checks that the tensor-parallel stack reproduces them bit for bit, eagerly
and replayed from a CUDA graph.  With --time it also prints decode milliseconds per step of both."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from signrot_b200.transformers import kernel_utils as ku  # noqa: E402


def build(cfg, dev, seed):
    with torch.device(dev):
        m = ku.KernelDecoderModel(cfg)
    return m.to(dev).random_init_(seed)


@torch.no_grad()
def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    timing = "--time" in sys.argv
    if timing:
        cfg = ku.DecoderConfig(num_hidden_layers=4, vocab_size=32000)
        B, T, steps, page = 8, 2048, 32, 256
    else:
        cfg = ku.DecoderConfig(hidden_size=1024, intermediate_size=3072, num_hidden_layers=2, num_attention_heads=8,
                               num_key_value_heads=4, head_dim=128, vocab_size=512)
        B, T, steps, page = 2, 37, 4, 16
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, cfg.vocab_size, (B, T), generator=g).to(dev)
    toks = [torch.randint(0, cfg.vocab_size, (B, 1), generator=g).to(dev) for _ in range(steps)]

    full = build(cfg, dev, 3)
    cache = ku.build_paged_cache(full, B, T + steps + 8, page_size=page)
    want = [full(prompt, past_key_values=cache, last_token_only=True).logits.clone()]
    want += [full(t, past_key_values=cache).logits.clone() for t in toks]

    shard = ku.shard_decoder_(build(cfg, dev, 3))
    assert shard.config.num_key_value_heads == cfg.num_key_value_heads // world
    cache_s = ku.build_paged_cache(shard, B, T + steps + 8, page_size=page)
    got = shard(prompt, past_key_values=cache_s, last_token_only=True).logits
    assert torch.equal(got, want[0]), f"prefill logits differ on rank {rank}"
    half = steps // 2
    for i in range(half):                                   # eager steps
        assert torch.equal(shard(toks[i], past_key_values=cache_s).logits, want[1 + i]), f"decode step {i}, rank {rank}"
    dec = ku.try_graph_decoder(shard, cache_s, B)           # the rest replayed from a graph (collectives inside)
    for i in range(half, steps):
        out = dec.step(toks[i]) if dec is not None else shard(toks[i], past_key_values=cache_s).logits
        assert torch.equal(out, want[1 + i]), f"graphed decode step {i}, rank {rank}"
    dist.barrier()
    if timing:
        def ms_per_step(model, c, d):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            tok = toks[0]
            torch.cuda.synchronize()
            dist.barrier()
            e0.record()
            for _ in range(32):
                (d.step(tok) if d is not None else model(tok, past_key_values=c))
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 32], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()
        full_dec = ku.try_graph_decoder(full, cache, B)
        a, b = ms_per_step(full, cache, full_dec), ms_per_step(shard, cache_s, dec)
        if rank == 0:
            print(f"tp_decoder_worker: timing layers={cfg.num_hidden_layers} batch={B} ctx={T} one_gpu_ms={a:.3f} "
                  f"tp{world}_ms={b:.3f} graph={dec is not None}")
    graphed = dec is not None
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"tp_decoder_worker: OK on {world} ranks (graph replay: {graphed})", flush=True)
    # Tearing the communicator down while CUDA graphs that captured its collectives are still alive blocks
    # forever in this NCCL version; nothing is in flight after the barrier and the synchronize above, so the
    # process simply ends here.
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
