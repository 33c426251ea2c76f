"""Megatron-style sharding of the quantized linears over `torch.distributed`
(one process per GPU; NCCL over NVLink on GPUs, gloo in the CPU tests of the plumbing).

The reference has no tensor parallelism on this path (fake_quant/kernel_utils.py:365-366: the
kernel model must live on one device).  The scheme here keeps every TP degree bit-identical
to one GPU:

  * column-parallel (q/k/v/gate/up): each rank owns N/tp output columns; the quantized input
    is replicated; no collective.
  * row-parallel (o_proj/down_proj): each rank owns K/tp input channels.  The online rotation
    and the per-token scale span the full K, so the fp16 input shards are all-gathered, every
    rank rotates + quantizes the full row (memory-bound, cheap), multiplies its K-slice of the
    codes with its weight shard, and the **int32** partial sums are all-reduced.  Integer
    addition is associative, so the result does not depend on the reduction order; the dequant
    epilogue runs after the reduce.

`ops` is the operator namespace used for the arithmetic; it defaults to the CUDA kernels
(`signrot_b200.functional.kernel`).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int, align: int = 1):
    """[begin, end) of the contiguous shard of `total` units owned by `rank`; shard sizes are
    multiples of `align` except possibly the last one."""
    if total % align:
        raise ValueError(f"{total} is not a multiple of {align}")
    units = total // align
    base, rem = divmod(units, world)
    begin = rank * base + min(rank, rem)
    end = begin + base + (1 if rank < rem else 0)
    return begin * align, end * align


def all_gather_cat(x: torch.Tensor, sizes, group=None) -> torch.Tensor:
    """Concatenation along the last dimension of every rank's `x` (rank r contributes sizes[r]
    columns).  Equal shards take one collective into one buffer; shards of unequal width are padded to
    the widest one first."""
    width = max(sizes)
    local = x.contiguous()
    if local.shape[-1] != width:
        local = torch.nn.functional.pad(local, (0, width - local.shape[-1]))
    world = len(sizes)
    stacked = torch.empty((world, *local.shape), dtype=local.dtype, device=local.device)
    if local.is_cuda:
        dist.all_gather_into_tensor(stacked, local, group=group)
    else:       # the CPU backend of the plumbing tests has only the list form
        dist.all_gather(list(stacked.unbind(0)), local, group=group)
    if min(sizes) == width:
        # [world, ..., w] -> [..., world * w]
        return stacked.movedim(0, -2).reshape(*local.shape[:-1], world * width)
    return torch.cat([stacked[r][..., :w] for r, w in enumerate(sizes)], dim=-1)


def _default_ops():
    from .functional import kernel
    return kernel


class ColumnParallelLinear4bit:
    """Output columns [begin, end) of a Linear4bit.  weight uint8 [N, K/2], scales fp16 [N, 1]."""

    def __init__(self, weight, weight_scales, group=None, ops=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ops = ops or _default_ops()
        n = weight.shape[0]
        self.n = n
        self.begin, self.end = shard_range(n, self.rank, self.world, align=8)
        self.weight = weight[self.begin:self.end].contiguous()
        self.weight_scales = weight_scales.reshape(-1)[self.begin:self.end].contiguous()

    def forward(self, packed, gather_output: bool = False):
        out = self.ops.w4a4_linear(packed, self.weight, self.weight_scales)
        if not gather_output:
            return out
        sizes = [e - b for b, e in (shard_range(self.n, r, self.world, 8) for r in range(self.world))]
        return all_gather_cat(out, sizes, self.group)


class RowParallelLinear4bit:
    """Input channels [begin, end) of a Linear4bit whose input goes through the online rotation.

    forward(x_local) takes this rank's fp16 activation shard [M, K/tp] (e.g. its slice of the
    SwiGLU output or of the attention output) and returns the full fp16 output [M, N] on every
    rank."""

    def __init__(self, weight, weight_scales, hadK=None, K_had=1, sign=None, heads=0, clip_ratio=1.0,
                 group=None, ops=None, peer=None):
        self.group = group
        self.peer = peer            # signrot_b200.comm.PeerGroup: one-kernel exchanges for messages that fit its slots
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ops = ops or _default_ops()
        self.k = weight.shape[1] * 2
        # shards are multiples of 64 values: 32 packed bytes, the GEMM's alignment unit
        self.begin, self.end = shard_range(self.k, self.rank, self.world, align=64)
        self.weight = weight[:, self.begin // 2:self.end // 2].contiguous()
        self.weight_scales = weight_scales.reshape(-1).contiguous()
        self.hadK, self.K_had, self.sign, self.heads, self.clip = hadK, K_had, sign, heads, clip_ratio

    def gather_input(self, x_local):
        sizes = [e - b for b, e in (shard_range(self.k, r, self.world, 64) for r in range(self.world))]
        peer = self.peer
        if (peer is not None and min(sizes) == max(sizes) and x_local.dim() == 2 and x_local.dtype == torch.float16
                and peer.fits(x_local.shape[0], x_local.shape[1], 0)):
            return peer.all_gather_cols(x_local)
        return all_gather_cat(x_local, sizes, self.group)

    def forward(self, x_local):
        x = self.gather_input(x_local) if self.world > 1 else x_local
        packed = self.ops.rotate_quant(x, self.hadK, self.K_had, sign=self.sign, heads=self.heads,
                                       clip_ratio=self.clip)
        codes = packed.quantized_x
        if hasattr(self.ops, "matmul_si4_cols") and codes.dim() == 2 and (self.begin // 2) % 16 == 0 and codes.shape[1] % 16 == 0:
            acc = self.ops.matmul_si4_cols(codes, self.begin // 2, self.end // 2, self.weight)   # no copy of the slice
        else:
            acc = self.ops.matmul_si4_si4(codes[..., self.begin // 2:self.end // 2].contiguous(), self.weight)
        peer = self.peer
        if self.world > 1 and peer is not None and acc.dim() == 2 and peer.fits(acc.shape[0], acc.shape[1], 1):
            # push the int32 partials to every peer, sum and dequantize in the same kernel
            return peer.all_reduce_dequant(acc, packed.scales_x.reshape(-1), self.weight_scales)
        if self.world > 1:
            dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)  # int32: exact, order-free
        return self.ops.sym_dequant(acc, packed.scales_x, self.weight_scales)
