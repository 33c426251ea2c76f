"""CPU oracle for the SignRot online quantized-linear path.

TEST INFRASTRUCTURE ONLY.  This package restates, on the CPU with torch/numpy tensor
arithmetic, what the reference computes on this path; each function cites the reference
file:line it follows.  It exists to check the CUDA library and to time a CPU baseline.  It
is imported by tests/, by `__graft_entry__.smoke()` and by the `cpu_baseline` / reference
arm of bench.py, and by nothing else: the product package `signrot_b200` never imports it
and has no CPU path.

Pinning.  The reference ships no golden vectors for this path, so the oracle is pinned
against outputs of the reference's own Python, imported on the CPU through `ref_shim.py`
and stored under tests/golden/ by tests/golden/make_golden.py (Hadamard tables and
butterfly, nibble packing, fake-quant wrapper with sign derivation, RTN weight quantizer,
KV quantizer, RMSNorm).  The parts of the path that exist only as CUDA in the reference
(fused quantizers' `__hdiv` rounding, decode attention, grouped GEMM) are restated from the
kernel sources; for those, parity is pinned only through the Python twins the reference keeps
beside them (`forward_reference`, `asym_quantize_and_pack_i4`, `_gemm_dequant_loop`).

fp16 arithmetic: torch CPU half ops compute in fp32 and round to nearest even once, which is
the `rn_h(op)` of the kernels.  The one deliberate difference from the GPU reference is the
code decision `x / scale`: the device `__hdiv` multiplies by an approximate reciprocal, the
oracle divides exactly (as the host branch of `__hdiv` does), so codes can differ by one at
exact rounding ties.
"""
from .quant import *  # noqa: F401,F403
from .hadamard import *  # noqa: F401,F403
from .gemm import *  # noqa: F401,F403
from .misc import *  # noqa: F401,F403
from .attention import *  # noqa: F401,F403
from .moe import *  # noqa: F401,F403
