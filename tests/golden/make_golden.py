"""Generates tests/golden/*.npz by running the REFERENCE's own Python on the CPU.

    SIGNROT_REFERENCE=<SignRot checkout> python tests/golden/make_golden.py

The reference has no stored golden vectors for this path; these files pin the oracle (and,
through it, the CUDA kernels) to what the reference's code computes on fixed seeded inputs.
Every array is produced by a reference function imported through oracle/ref_shim.py; inputs
are stored next to outputs so the tests do not depend on RNG stability across torch versions.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import ref_shim  # noqa: E402

OUT = Path(__file__).resolve().parent


def npy(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.detach().cpu().numpy()


def main():
    torch.manual_seed(0)
    had = ref_shim.module("signrot.functional.hadamard")
    qz = ref_shim.module("signrot.functional.quantization")
    kvc = ref_shim.module("signrot.transformers.kv_cache")
    qu = ref_shim.module("quant_utils")
    norm = ref_shim.module("signrot.nn.normalization")
    g = torch.Generator().manual_seed(20240607)

    # 1. Hadamard butterfly (signrot/functional/hadamard.py:43-65) incl. the Kronecker cases
    d = {}
    for n, rows in ((128, 3), (768, 2), (4096, 2), (14336, 1), (2048, 1)):
        x = torch.randn((rows, n), generator=g, dtype=torch.float32)
        d[f"x_{n}"] = npy(x)
        d[f"y_{n}"] = npy(had.matmul_hadU(x))
        d[f"K_{n}"] = np.int64(had.get_hadK(n)[1])
    torch.manual_seed(7)
    d["randhad_64_seed7"] = npy(had.random_hadamard_matrix(64, "cpu"))
    np.savez_compressed(OUT / "hadamard.npz", **d)

    # 2. nibble packing (signrot/functional/quantization.py:45-101)
    q = torch.randint(-8, 8, (5, 64), generator=g, dtype=torch.int8)
    packed = qz.pack_i4(q)
    np.savez_compressed(OUT / "pack.npz", q=npy(q), packed=npy(packed), unpack_i4=npy(qz.unpack_i4(packed)),
                        unpack_ui4=npy(qz.unpack_ui4(packed)))

    # 3. KV quantizer (signrot/transformers/kv_cache.py:12-68)
    x = torch.randn((2, 3, 4, 128), generator=g).half()
    x[0, 0, 0] = 0.5          # constant vector: diff clamps to 1e-5
    x[1, 2, 3] *= 30.0
    pq, ps, pz = kvc.asym_quantize_and_pack_i4(x)
    deq = kvc.unpack_i4_and_asym_dequantize(pq, ps, pz)
    np.savez_compressed(OUT / "kv_quant.npz", x=npy(x), q=npy(pq), scale=npy(ps), zero=npy(pz), deq=npy(deq))

    # 4. fake-quant wrapper incl. SignRot sign derivation (fake_quant/quant_utils.py:316-386)
    d = {}
    def wrapper_case(tag, in_f, out_f, dtype, full=False, partial_dim=0, adj=False, tokens=24, sym=True, clip=1.0):
        lin = torch.nn.Linear(in_f, out_f, bias=False)
        lin.weight.data = (torch.randn((out_f, in_f), generator=g) * 0.05)
        lin = lin.to(dtype)
        w0 = lin.weight.data.clone()
        wrp = qu.ActQuantWrapper(lin)
        wrp.quantizer.configure(bits=4, groupsize=-1, sym=sym, clip_ratio=clip)
        if full:
            hk, K = had.get_hadK(in_f)
            wrp.online_full_had = True
            wrp.had_K, wrp.K = hk, K
        if partial_dim:
            hk, K = had.get_hadK(in_f // partial_dim)
            wrp.online_partial_had = True
            wrp.had_K, wrp.K, wrp.had_dim = hk, K, partial_dim
        if adj:
            wrp.had_adj_sign = torch.ones(in_f, dtype=torch.int8)
        x = torch.randn((1, tokens, in_f), generator=g)
        x[0, 5, 3] = 60.0  # a massive-activation token
        x[0, 5, 17] = -45.0
        x = x.to(dtype)
        with torch.no_grad():
            y = wrp(x)
        d[f"{tag}_x"], d[f"{tag}_w0"], d[f"{tag}_y"] = npy(x), npy(w0), npy(y)
        d[f"{tag}_w1"] = npy(lin.weight.data)
        if adj:
            d[f"{tag}_sign"] = npy(wrp.had_adj_sign)
    wrapper_case("plain512_f16", 512, 32, torch.float16)
    wrapper_case("plain512_bf16", 512, 32, torch.bfloat16)
    wrapper_case("full768_adj_f16", 768, 32, torch.float16, full=True, adj=True)
    wrapper_case("full1024_adj_bf16", 1024, 16, torch.bfloat16, full=True, adj=True)
    wrapper_case("heads256_f16", 256, 32, torch.float16, partial_dim=64)
    wrapper_case("asym512_clip_f16", 512, 16, torch.float16, sym=False, clip=0.9)
    np.savez_compressed(OUT / "fake_quant_wrapper.npz", **d)

    # 5. RTN weight quantizer (fake_quant/quant_utils.py:408-560)
    d = {}
    W = (torch.randn((16, 64), generator=g) * 0.03).half()
    for tag, mse, symgrid in (("rtn", False, False), ("rtn_mse", True, False), ("rtn_symgrid", False, True)):
        wq = qu.WeightQuantizer()
        wq.configure(4, perchannel=True, sym=True, mse=mse)
        wq.sym_symmetric_grid = symgrid
        wq.find_params(W)
        d[f"{tag}_scale"], d[f"{tag}_wq"] = npy(wq.scale), npy(wq(W))
    d["W"] = npy(W)
    np.savez_compressed(OUT / "rtn.npz", **d)

    # 6. RMSNorm reference statement (signrot/nn/normalization.py:24-30)
    x = torch.randn((3, 256), generator=g).half()
    m = norm.RMSNorm(256, eps=1e-5)
    np.savez_compressed(OUT / "rmsnorm.npz", x=npy(x), y=npy(m.forward_reference(x)))

    # 7. activation fake quantizer edge rows (fake_quant/quant_utils.py:95-144)
    x = torch.randn((6, 128), generator=g).half()
    x[1] = 0
    x[2] = 1.25
    x[3] *= 1e3
    x[4] *= 1e-4
    x[5] = -x[5].abs()
    d = {"x": npy(x)}
    for tag, sym, clip in (("sym", True, 1.0), ("asym", False, 1.0), ("asym_clip", False, 0.9)):
        aq = qu.ActQuantizer()
        aq.configure(bits=4, sym=sym, clip_ratio=clip)
        aq.find_params(x)
        d[tag] = npy(aq(x))
    np.savez_compressed(OUT / "act_fake_quant.npz", **d)
    extra(g)
    print("golden vectors written to", OUT)


def _reference_function(path: Path, name: str, namespace: dict):
    """Compiles ONE function of a reference script without importing the script (its module level
    imports the CUDA extension and runs on a GPU)."""
    import ast
    tree = ast.parse(path.read_text())
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
    code = compile(ast.Module(body=[fn], type_ignores=[]), str(path), "exec")
    exec(code, namespace)
    return namespace[name]


def extra(g):
    """Vectors for the statements that exist only as CUDA kernels in the reference, taken from the
    pure-torch code the reference itself tests those kernels against."""
    import math
    import types
    import oracle
    kern = ref_shim.module("signrot.functional.kernel")
    qn = ref_shim.module("signrot.nn.quantization")
    kvc = ref_shim.module("signrot.transformers.kv_cache")

    # 8. scale order of the quantizer modules' torch statements (signrot/nn/quantization.py:23-28, 44-48,
    #    67-76).  Their code decision is a CUDA call; it is answered by the oracle here, so only the scales
    #    (and the asymmetric zero point) written by the reference's lines are stored.
    seen = {}
    def grab_sym(x, scales):
        seen["scale"] = scales.clone()
        return oracle.sym_quant(x, scales)
    def grab_asym(x, scales, zeros):
        seen["scale"], seen["zero"] = scales.clone(), zeros.clone()
        return oracle.pack_codes(oracle.asym_quant_codes(x, scales.half(), zeros.half(), 0, 15))
    kern.sym_quant, kern.asym_quant_f16_ui4 = grab_sym, grab_asym
    x = torch.randn((7, 256), generator=g).half()
    x[2] *= 40.0
    x[5] = x[5].abs() + 0.5
    d = {"x": npy(x)}
    for clip in (1.0, 0.9):
        tag = f"clip{int(clip * 100)}"
        qn.Quantizer(clip_ratio=clip).forward_reference(x)
        d[f"quantizer_{tag}"] = npy(seen["scale"])
        qn.SymQuantizer(clip_ratio=clip).forward_reference(x)
        d[f"symquantizer_{tag}"] = npy(seen["scale"])
        qn.AsymQuantizer(clip_ratio=clip).forward_reference(x)
        d[f"asym_scale_{tag}"], d[f"asym_zero_{tag}"] = npy(seen["scale"]), npy(seen["zero"])
    np.savez_compressed(OUT / "quantizer_scales.npz", **d)

    # 9. rotary embedding: the HF function the reference checks rope_qk against
    #    (benchmarks/test_fused_equivalence.py:102-115)
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb
    d = {}
    for tag, (b, t_, hq, hk, cos_b) in {"b4t3": (4, 3, 32, 8, 4), "b2t5_shared": (2, 5, 8, 8, 1)}.items():
        q = torch.randn((b, t_, hq, 128), generator=g).half()
        k = torch.randn((b, t_, hk, 128), generator=g).half()
        cos = torch.randn((cos_b, t_, 128), generator=g).half()
        sin = torch.randn((cos_b, t_, 128), generator=g).half()
        qr, kr = apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=2)
        for name, val in (("q", q), ("k", k), ("cos", cos), ("sin", sin), ("q_out", qr), ("k_out", kr)):
            d[f"{tag}_{name}"] = npy(val)
    np.savez_compressed(OUT / "rope.npz", **d)

    # 10. decode attention: the reference's fp32 statement over its own dequantized paged cache
    #     (benchmarks/test_split_decode.py:22-46 with kv_cache.py:12-68), K rotated as the cache does
    #     (kv_cache.py:70-73)
    ref_attn = _reference_function(ref_shim.REF / "benchmarks" / "test_split_decode.py", "reference_attention",
                                   {"torch": torch, "math": math,
                                    "unpack_i4_and_asym_dequantize": kvc.unpack_i4_and_asym_dequantize})
    B, L, Hh, page, T = 2, 2, 4, 16, 37
    k = torch.randn((B, T, Hh, 128), generator=g).half()
    v = torch.randn((B, T, Hh, 128), generator=g).half()
    q = torch.randn((B, Hh, 128), generator=g).half()
    kq, ks, kz = kvc.asym_quantize_and_pack_i4(kvc.matmul_had_cuda(k, torch.float16))
    vq, vs, vz = kvc.asym_quantize_and_pack_i4(v)
    n_pages = (T + page - 1) // page
    pages = torch.zeros((n_pages * B, L, 2, Hh, page, 64), dtype=torch.uint8)
    scales = torch.zeros((n_pages * B, L, 2, Hh, page, 2), dtype=torch.float16)
    for b in range(B):
        for pos in range(T):
            pg, slot = (pos // page) * B + b, pos % page
            pages[pg, 1, 0, :, slot], pages[pg, 1, 1, :, slot] = kq[b, pos], vq[b, pos]
            scales[pg, 1, 0, :, slot] = torch.cat((ks[b, pos], kz[b, pos]), -1)
            scales[pg, 1, 1, :, slot] = torch.cat((vs[b, pos], vz[b, pos]), -1)
    cache = types.SimpleNamespace(page_size=page, pages=pages, scales=scales, batch_size=B)
    q_rot = kvc.matmul_had_cuda(q, torch.float16)
    out = ref_attn(cache, q_rot, 1, T)
    np.savez_compressed(OUT / "attention.npz", k=npy(k), v=npy(v), q=npy(q), out=npy(out), page=np.int64(page))

    # 11. sparse block: the reference's forward (signrot/nn/moe.py:160-236, per-expert loop branch) with its
    #     CUDA calls answered by the integer oracle; router, stable sort, gathers, un-permute and weighted
    #     sum are the reference's own lines
    moe = ref_shim.module("signrot.nn.moe")
    kern.sym_quant_dynamic = lambda x, clip: (lambda c, s: (oracle.pack_codes(c), s))(*oracle.sym_quant_dynamic(x, clip))
    kern.matmul_si4_si4 = lambda a, b: oracle.matmul_i4(a, b)
    kern.sym_dequant = lambda acc, sr, sc: oracle.sym_dequant(acc, sr, sc)
    kern.swiglu = lambda a, b: oracle.swiglu(a, b)
    E, hidden, inter, top_k, tokens = 4, 64, 96, 2, 10
    def w(n, kk):
        return oracle.pack_i4(torch.randint(-8, 8, (E * n, kk), generator=g, dtype=torch.int32)).view(E, n, kk // 2)
    def sc(n, kk):
        return (torch.rand((E, n), generator=g) * 0.5 / kk + 0.5 / kk).half()
    gate = torch.nn.Linear(hidden, E, bias=False).half()
    gate.weight.data = torch.randn((E, hidden), generator=g).half()
    sign = (torch.randint(0, 2, (E, inter), generator=g) * 2 - 1).to(torch.int8)
    tensors = dict(w_gate=w(inter, hidden), s_gate=sc(inter, hidden), w_up=w(inter, hidden), s_up=sc(inter, hidden),
                   w_down=w(hidden, inter), s_down=sc(hidden, inter), sign_down=sign)
    blk = moe.SignRotMoEBlock(gate, top_k=top_k, norm_topk_prob=True, use_grouped=False, **tensors)
    x = torch.randn((1, tokens, hidden), generator=g).half()
    with torch.no_grad():
        y, logits = blk(x)
    d = {kk: npy(vv) for kk, vv in tensors.items()}
    d.update(x=npy(x), gate_w=npy(gate.weight.data), y=npy(y), logits=npy(logits), top_k=np.int64(top_k))
    np.savez_compressed(OUT / "moe_block.npz", **d)


if __name__ == "__main__":
    main()
