"""Sparse MoE block over stacked int4 expert weights, interface of
`signrot.nn.SignRotMoEBlock` (signrot/nn/moe.py:28-236).

One forward is ten launches, all fixed-shape and free of host synchronisation (capturable):

  router linear -> `moe_route` (fp32 softmax, top-k, renormalisation, rows counted and placed per
  expert in token order) -> per-token quantizer -> `moe_gather` (packed codes + scales per routed
  row) -> grouped gate GEMM, grouped up GEMM (`grouped_linear`: int4 GEMM + expert-indexed dequant
  in one launch; the weight-streaming mma.sync kernel when the routed rows average at most 16 per
  expert, the CTA-pair tcgen05 kernel otherwise) -> SwiGLU -> rotation + per-expert sign +
  quantizer in one kernel (`rotate_quant` with expert ids) -> grouped down GEMM -> `moe_combine`
  (un-permute and routing-weighted sum with the reference's rounding points).

The reference also carries a host-synchronising per-expert loop over the dense kernels
(`use_grouped=False`) as the equivalence check of its grouped kernels.  Both give the same bits, so
this build has the grouped form only; the keyword is accepted and the loop lives in the tests as a
checker (tests/test_gpu_moe.py).
"""
from __future__ import annotations

import torch

from ..functional import kernel
from ..functional.hadamard import get_hadK

_WEIGHT_BUFFERS = ("w_gate", "w_up", "w_down", "s_gate", "s_up", "s_down", "wsum_gate", "wsum_up", "wsum_down")


class SignRotMoEBlock(torch.nn.Module):
    def __init__(self, gate, *, top_k, norm_topk_prob,
                 w_gate, s_gate, w_up, s_up, w_down, s_down,
                 sign_down=None, wsum_gate=None, wsum_up=None, wsum_down=None,
                 asym=False, clip_ratio=1.0, fp32_had=False, use_grouped=True):
        super().__init__()
        experts, inter, half_hidden = w_gate.shape
        if tuple(w_down.shape) != (experts, 2 * half_hidden, inter // 2):
            raise ValueError(f"w_down {tuple(w_down.shape)} does not match w_gate {tuple(w_gate.shape)}")
        if experts > 512 or top_k > 8:
            raise NotImplementedError(f"{experts} experts / top-{top_k}: the routing kernel takes up to 512 experts, top-8")
        self.gate = gate                    # router linear, 16-bit, untouched
        self.top_k, self.norm_topk_prob = top_k, norm_topk_prob
        self.asym, self.clip_ratio, self.fp32_had = asym, clip_ratio, fp32_had
        self.use_grouped = use_grouped      # kept for the reference's signature; see the module docstring
        self.num_experts, self.intermediate_size, self.hidden_size = experts, inter, 2 * half_hidden
        given = dict(w_gate=w_gate, w_up=w_up, w_down=w_down, s_gate=s_gate, s_up=s_up, s_down=s_down,
                     wsum_gate=wsum_gate, wsum_up=wsum_up, wsum_down=wsum_down, sign_down=sign_down)
        for name, value in given.items():
            self.register_buffer(name, value, persistent=False)
        had_K, self.K = get_hadK(inter)
        if had_K is not None:
            had_K = had_K.to(w_gate.device, torch.float32 if fp32_had else torch.float16)
        self.register_buffer("had_K", had_K, persistent=False)
        self._ep = None                     # (group, first expert, end expert, peer group) after shard_experts_

    @staticmethod
    def stack_experts(linears, need_wsum):
        """[E, ...] stacks of the experts' packed weights, fp16 scales [E, N] and, on request, int4 row sums."""
        weights = torch.stack([lin.weight for lin in linears]).contiguous()
        scales = torch.stack([lin.weight_scales.reshape(-1).half() for lin in linears]).contiguous()
        if not need_wsum:
            return weights, scales, None
        return weights, scales, kernel.sum_i4(weights).view(len(linears), -1)

    def _row_sums(self):
        """int4 row sums of the three stacks (asymmetric zero-point correction), computed on first use: the
        block may be built while the weights are still on the CPU."""
        if self.asym and self.wsum_gate is None:
            for tag in ("gate", "up", "down"):
                w = getattr(self, "w_" + tag)
                setattr(self, "wsum_" + tag, kernel.sum_i4(w).view(w.shape[0], -1))

    def forward(self, hidden_states: torch.Tensor):
        bsz, seq, hid = hidden_states.shape
        dtype = hidden_states.dtype
        x = hidden_states.reshape(-1, hid)
        self._row_sums()
        router_logits = self.gate(x)
        weights, _, tok, eid, inv, row_off = kernel.moe_route(router_logits.to(torch.float16), self.top_k,
                                                              self.norm_topk_prob)
        x16 = x if dtype == torch.float16 else x.to(torch.float16)
        if self.asym:
            codes, scales, zeros = kernel.asym_quant_dynamic(x16, self.clip_ratio)
            per_token = kernel.PackedQuantizedTensor(codes, scales, zeros.to(torch.int8))
        else:
            per_token = kernel.PackedQuantizedTensor(*kernel.sym_quant_dynamic(x16, self.clip_ratio))
        routed = kernel.moe_gather(per_token, tok)      # a token's experts, and gate/up, read the same codes
        ep = self._ep
        covered = 0                             # rows the offsets passed below cover: all of them
        if ep is None:
            eid_w, off_w, rng = eid, row_off, None
        else:
            # expert parallel: this rank holds experts [e0, e1); the rows are sorted by expert, so its rows are
            # the contiguous range row_off[e0] .. row_off[e1] and the grouped GEMMs touch nothing else.  Expert
            # ids index the local weight stacks; the sign table stays global.
            e0, e1 = ep[1], ep[2]
            eid_w, off_w, rng = eid - e0, row_off[e0:e1 + 1], row_off[e0:e1 + 1:e1 - e0].contiguous()
            # about this share of the routed rows (the counts live on the device): picks the decode or the prefill kernel
            covered = max(1, routed.quantized_x.shape[0] * (e1 - e0) // self.num_experts)
        gate_h = kernel.grouped_linear(routed, eid_w, off_w, self.w_gate, self.s_gate, self.wsum_gate, covered)
        up_h = kernel.grouped_linear(routed, eid_w, off_w, self.w_up, self.s_up, self.wsum_up, covered)
        inter = kernel.swiglu(gate_h, up_h)
        sign_ids = eid if self.sign_down is not None else None
        if self.fp32_had:
            # fp32 rotation keeps the reference's operator chain: transform, one rounding, expert-indexed quantizer
            h = kernel.hadamard(inter, self.had_K, self.K, fp32_mode=True, out_dtype=torch.float16)
            signs = self.sign_down if self.sign_down is not None else \
                torch.ones((1, self.intermediate_size), dtype=torch.int8, device=h.device)
            ids = eid if self.sign_down is not None else torch.zeros_like(eid)
            if self.asym:
                q, s, z = kernel.asym_quant_dynamic_moe(h, signs, ids, self.clip_ratio)
                pk = kernel.PackedQuantizedTensor(q, s, z.to(torch.int8))
            else:
                pk = kernel.PackedQuantizedTensor(*kernel.sym_quant_dynamic_moe(h, signs, ids, self.clip_ratio))
        else:
            pk = kernel.rotate_quant(inter, self.had_K, self.K, sign=self.sign_down, expert_ids=sign_ids,
                                     clip_ratio=self.clip_ratio, asym=self.asym)
        y = kernel.grouped_linear(pk, eid_w, off_w, self.w_down, self.s_down, self.wsum_down, covered)
        if ep is None:
            out = kernel.moe_combine(y, weights, inv)
        else:
            import torch.distributed as dist
            part = kernel.moe_combine(y, weights, inv, row_range=rng, out_fp32=True)
            peer = ep[3]
            if peer is not None and peer.fits(part.shape[0], part.shape[1], 2):
                out = peer.all_reduce_f32(part)      # one kernel: push, sum in rank order, round
            else:
                dist.all_reduce(part, op=dist.ReduceOp.SUM, group=ep[0])
                out = part.to(torch.float16)
        if dtype != torch.float16:
            out = out.to(dtype)
        return out.view(bsz, seq, hid), router_logits

    def shard_experts_(self, group=None, peer=None):
        """Expert parallelism, in place: this rank keeps a contiguous block of num_experts / world experts
        (weights, scales, row sums); router, tokens and the sign table stay replicated.  Every rank routes all
        tokens, computes the rows of its own experts and the weighted partial sums are added across ranks in
        fp32 (with top-2 a token has at most two non-zero addends, so the result has the bits of one GPU)."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if self.num_experts % world:
            raise ValueError(f"{self.num_experts} experts do not split {world} ways")
        per = self.num_experts // world
        e0, e1 = rank * per, (rank + 1) * per
        self._row_sums()
        for name in _WEIGHT_BUFFERS:
            t = getattr(self, name)
            if t is not None:
                setattr(self, name, t[e0:e1].contiguous())
        self._ep = (group, e0, e1, peer)     # peer: signrot_b200.comm.PeerGroup for decode-size sums, or None
        return self
