"""Sparse MoE block over stacked int4 expert weights, interface of
`signrot.nn.SignRotMoEBlock` (signrot/nn/moe.py:28-236).

Data flow per forward (all fixed-shape, no host synchronisation, so the block can be
captured in a CUDA graph):

  router (fp linear, fp32 softmax, top-k) -> rows sorted by expert -> every token quantized
  once, packed codes gathered per routed row -> grouped gate/up GEMM + expert-indexed
  dequant -> SwiGLU -> rotation + per-expert sign + quantization in ONE kernel
  (`rotate_quant` with expert_ids) -> grouped down GEMM + dequant -> weighted un-permute.

`use_grouped=False` runs the per-expert loop over the dense kernels (host-synchronising);
it is the equivalence check for the grouped path, bit-identical by construction.

The grouped GEMM + dequant pair runs as ONE launch (`kernel.grouped_linear`): the library takes the
weight-streaming mma.sync kernel when the routed rows average at most 16 per expert (decode) and
the CTA-pair tcgen05 kernel otherwise.  With `fused_routing` (default, fp16, at most 512 experts,
top-8) the softmax / top-k / sort-by-expert chain, the gathers and the final weighted un-permute
are one launch each (`kernel.moe_route / moe_gather / moe_combine`).  The reference's two calls (`matmul_grouped` followed by
`sym_dequant_moe`) remain for more than 512 experts.  All of them produce the same bits: the int32
accumulators are exact either way and the dequant arithmetic is shared.
"""
from __future__ import annotations

import torch

from ..functional import kernel
from ..functional.hadamard import get_hadK


class SignRotMoEBlock(torch.nn.Module):
    def __init__(self, gate, *, top_k, norm_topk_prob,
                 w_gate, s_gate, w_up, s_up, w_down, s_down,
                 sign_down=None, wsum_gate=None, wsum_up=None, wsum_down=None,
                 asym=False, clip_ratio=1.0, fp32_had=False, use_grouped=True, fused_routing=True):
        super().__init__()
        self.fused_routing = fused_routing
        self._ep = None                 # (group, first expert, end expert) after shard_experts_
        self.gate = gate
        self.top_k = top_k
        self.norm_topk_prob = norm_topk_prob
        self.asym = asym
        self.clip_ratio = clip_ratio
        self.fp32_had = fp32_had
        self.use_grouped = use_grouped

        self.num_experts, self.intermediate_size = w_gate.shape[0], w_gate.shape[1]
        self.hidden_size = w_gate.shape[2] * 2
        assert w_down.shape == (self.num_experts, self.hidden_size, self.intermediate_size // 2)

        for name, t in (("w_gate", w_gate), ("w_up", w_up), ("w_down", w_down),
                        ("s_gate", s_gate), ("s_up", s_up), ("s_down", s_down),
                        ("sign_down", sign_down),
                        ("wsum_gate", wsum_gate), ("wsum_up", wsum_up), ("wsum_down", wsum_down)):
            self.register_buffer(name, t, persistent=False)

        had_K, self.K = get_hadK(self.intermediate_size)
        if had_K is not None:
            had_K = had_K.to(w_gate.device, torch.float32 if fp32_had else torch.float16)
        self.register_buffer("had_K", had_K, persistent=False)
        self._consts_dev = None

    @staticmethod
    def stack_experts(linears, need_wsum):
        """Stacks per-expert Linear4bit weights, scales and (optionally) int4 row sums."""
        w = torch.stack([m.weight for m in linears]).contiguous()
        s = torch.stack([m.weight_scales.view(-1).to(torch.float16) for m in linears]).contiguous()
        wsum = torch.stack([kernel.sum_i4(m.weight).view(-1) for m in linears]) if need_wsum else None
        return w, s, wsum

    def _ensure_wsum(self):
        if not self.asym or self.wsum_gate is not None:
            return
        e = self.num_experts
        self.wsum_gate = kernel.sum_i4(self.w_gate).view(e, -1)
        self.wsum_up = kernel.sum_i4(self.w_up).view(e, -1)
        self.wsum_down = kernel.sum_i4(self.w_down).view(e, -1)

    def _quantize(self, x):
        if self.asym:
            q, s, z = kernel.asym_quant_dynamic(x, self.clip_ratio)
            return q, s, z.to(torch.int8)
        q, s = kernel.sym_quant_dynamic(x, self.clip_ratio)
        return q, s, None

    # ------------------------------------------------------------------ grouped path

    def _consts(self, device):
        """Device-resident constants of the three grouped calls: weight base addresses,
        leading dimensions, and (m, n, k) rows whose m column is rewritten every forward."""
        if self._consts_dev == device:
            return self._gc
        e, h, i = self.num_experts, self.hidden_size, self.intermediate_size
        idx = torch.arange(e, dtype=torch.int64, device=device)

        def make(w, n, k):
            ps = torch.empty((e, 3), dtype=torch.int32, device=device)
            ps[:, 1] = n
            ps[:, 2] = k
            return {"ps": ps, "ptr_b": w.data_ptr() + idx * w.stride(0), "k": k,
                    "ld_ab": torch.full((e,), k, dtype=torch.int64, device=device),
                    "ld_c": torch.full((e,), n, dtype=torch.int64, device=device)}

        self._gc = {"gate": make(self.w_gate, i, h), "up": make(self.w_up, i, h), "down": make(self.w_down, h, i)}
        self._consts_dev = device
        return self._gc

    def _gemm_dequant_grouped(self, q, s, z, eid, row_off, w, s_w, wsum, gc):
        m, n = q.shape[0], w.shape[1]
        if self.num_experts <= 512:
            return kernel.grouped_linear(kernel.PackedQuantizedTensor(q, s, z), eid, self._row_off32, w, s_w, wsum)
        c = torch.empty((m, n), dtype=torch.int32, device=q.device)
        ptr_a = q.data_ptr() + row_off * q.shape[1]
        ptr_c = c.data_ptr() + row_off * (n * 4)
        kernel.matmul_grouped(gc["ps"], ptr_a, gc["ptr_b"], ptr_c, gc["ld_ab"], gc["ld_ab"], gc["ld_c"],
                              signed_a=z is None, max_k=gc["k"])
        return kernel.sym_dequant_moe(c, s, s_w, eid, z, wsum)

    # ------------------------------------------------------------------ per-expert loop

    def _gemm_dequant_loop(self, q, s, z, counts, w, s_w, wsum):
        out = torch.empty(q.shape[0], w.shape[1], dtype=torch.float16, device=q.device)
        start = 0
        for e, m in enumerate(counts.tolist()):
            if m == 0:
                continue
            sl = slice(start, start + m)
            start += m
            if z is not None:
                acc = kernel.matmul_ui4_si4(q[sl], w[e])
                acc -= kernel.matmul_colrow_i8_i32(z[sl], wsum[e].view(1, -1))
            else:
                acc = kernel.matmul_si4_si4(q[sl], w[e])
            out[sl] = kernel.sym_dequant(acc, s[sl], s_w[e].view(-1, 1))
        return out

    # ------------------------------------------------------------------ forward

    def _forward_fused_routing(self, hidden_states):
        """The grouped path with the routing glue as three launches (`moe_route`, `moe_gather`,
        `moe_combine`) instead of the tensor-library chain below: ten launches per block."""
        bsz, seq, hid = hidden_states.shape
        x = hidden_states.reshape(-1, hid)
        router_logits = self.gate(x)
        weights, _, tok, eid, inv, row_off = kernel.moe_route(router_logits, self.top_k, self.norm_topk_prob)
        q_tok, s_tok, z_tok = self._quantize(x)
        routed = kernel.moe_gather(kernel.PackedQuantizedTensor(q_tok, s_tok, z_tok), tok)
        ep = self._ep
        if ep is None:
            eid_w, off_w, rng = eid, row_off, None
        else:
            # expert parallel: this rank holds experts [e0, e1); the rows are sorted by expert, so its rows are
            # the contiguous range row_off[e0] .. row_off[e1] and the grouped GEMMs touch nothing else.  Expert
            # ids index the local weight stacks; the sign table stays global.
            e0, e1 = ep[1], ep[2]
            eid_w, off_w, rng = eid - e0, row_off[e0:e1 + 1], row_off[e0:e1 + 1:e1 - e0].contiguous()
        gate_h = kernel.grouped_linear(routed, eid_w, off_w, self.w_gate, self.s_gate, self.wsum_gate)
        up_h = kernel.grouped_linear(routed, eid_w, off_w, self.w_up, self.s_up, self.wsum_up)
        inter = kernel.swiglu(gate_h, up_h)
        pk = kernel.rotate_quant(inter, self.had_K, self.K, sign=self.sign_down,
                                 expert_ids=eid if self.sign_down is not None else None,
                                 clip_ratio=self.clip_ratio, asym=self.asym)
        y = kernel.grouped_linear(pk, eid_w, off_w, self.w_down, self.s_down, self.wsum_down)
        if ep is None:
            out = kernel.moe_combine(y, weights, inv)
        else:
            import torch.distributed as dist
            part = kernel.moe_combine(y, weights, inv, row_range=rng, out_fp32=True)
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=ep[0])
            out = part.to(torch.float16)
        return out.view(bsz, seq, hid), router_logits

    def shard_experts_(self, group=None):
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
        self._ensure_wsum()
        for name in ("w_gate", "w_up", "w_down", "s_gate", "s_up", "s_down", "wsum_gate", "wsum_up", "wsum_down"):
            t = getattr(self, name)
            if t is not None:
                setattr(self, name, t[e0:e1].contiguous())
        self._ep = (group, e0, e1)
        self.fused_routing = True
        return self

    def forward(self, hidden_states: torch.Tensor):
        bsz, seq, hid = hidden_states.shape
        x = hidden_states.view(-1, hid)
        dt = x.dtype
        self._ensure_wsum()
        if (self.fused_routing and self.use_grouped and not self.fp32_had and dt == torch.float16
                and self.num_experts <= 512 and self.top_k <= 8 and hid % 8 == 0
                and self.gate.weight.dtype == torch.float16):
            return self._forward_fused_routing(hidden_states)
        if self._ep is not None:
            raise RuntimeError("an expert-parallel block runs the fused-routing path only (fp16, grouped)")

        router_logits = self.gate(x)
        probs = torch.softmax(router_logits, dim=1, dtype=torch.float)
        probs, chosen = torch.topk(probs, self.top_k, dim=-1)
        if self.norm_topk_prob:
            probs /= probs.sum(dim=-1, keepdim=True)
        probs = probs.to(dt)

        # sort the (token, choice) rows by expert with fixed-shape, sync-free ops
        flat_e = chosen.reshape(-1)
        perm = torch.argsort(flat_e, stable=True)
        counts = torch.zeros(self.num_experts, dtype=torch.int32, device=x.device)
        counts.index_add_(0, flat_e, torch.ones_like(flat_e, dtype=torch.int32))
        tok = perm // self.top_k
        eid = flat_e[perm].to(torch.int32)

        q_tok, s_tok, z_tok = self._quantize(x.to(torch.float16))
        q_a, s_a = q_tok[tok], s_tok[tok]
        z_a = z_tok[tok] if z_tok is not None else None

        if self.use_grouped:
            gc = self._consts(x.device)
            row_off = torch.zeros(self.num_experts, dtype=torch.int64, device=x.device)
            row_off[1:] = torch.cumsum(counts[:-1], 0)
            self._row_off32 = torch.zeros(self.num_experts + 1, dtype=torch.int32, device=x.device)
            self._row_off32[1:] = torch.cumsum(counts, 0)
            for key in ("gate", "up", "down"):
                gc[key]["ps"][:, 0] = counts
            gate_h = self._gemm_dequant_grouped(q_a, s_a, z_a, eid, row_off, self.w_gate, self.s_gate,
                                                self.wsum_gate, gc["gate"])
            up_h = self._gemm_dequant_grouped(q_a, s_a, z_a, eid, row_off, self.w_up, self.s_up, self.wsum_up,
                                              gc["up"])
        else:
            gate_h = self._gemm_dequant_loop(q_a, s_a, z_a, counts, self.w_gate, self.s_gate, self.wsum_gate)
            up_h = self._gemm_dequant_loop(q_a, s_a, z_a, counts, self.w_up, self.s_up, self.wsum_up)
        inter = kernel.swiglu(gate_h, up_h)

        if self.use_grouped and not self.fp32_had:
            # rotation, per-expert sign and quantization in one pass over each row
            pk = kernel.rotate_quant(inter, self.had_K, self.K, sign=self.sign_down,
                                     expert_ids=eid if self.sign_down is not None else None,
                                     clip_ratio=self.clip_ratio, asym=self.asym)
            y = self._gemm_dequant_grouped(pk.quantized_x, pk.scales_x, pk.zeros_x, eid, row_off, self.w_down,
                                           self.s_down, self.wsum_down, gc["down"])
        else:
            h = kernel.hadamard(inter, self.had_K, self.K, fp32_mode=self.fp32_had, out_dtype=torch.float16)
            if self.use_grouped:
                if self.asym:
                    q_d, s_d, z_d = kernel.asym_quant_dynamic_moe(h, self.sign_down, eid, self.clip_ratio)
                    z_d = z_d.to(torch.int8)
                else:
                    q_d, s_d = kernel.sym_quant_dynamic_moe(h, self.sign_down, eid, self.clip_ratio)
                    z_d = None
                y = self._gemm_dequant_grouped(q_d, s_d, z_d, eid, row_off, self.w_down, self.s_down,
                                               self.wsum_down, gc["down"])
            else:
                if self.sign_down is not None:
                    h = h * self.sign_down[eid]
                q_d, s_d, z_d = self._quantize(h)
                y = self._gemm_dequant_loop(q_d, s_d, z_d, counts, self.w_down, self.s_down, self.wsum_down)

        # deterministic un-permute and weighted sum (no atomics)
        inv = torch.argsort(perm)
        y = y.to(dt)[inv].view(-1, self.top_k, hid)
        out = (y * probs.unsqueeze(-1)).sum(dim=1)
        return out.view(bsz, seq, hid), router_logits
