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
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
