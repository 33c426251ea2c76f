"""signrot_b200: SignRot's online quantized-linear path on B200 (sm_100a).

The package mirrors the reference's public layout for this path:

    signrot_b200.functional   pack/unpack, Hadamard helpers, `kernel` operators
    signrot_b200.nn           Linear4bit, Quantizer, AsymQuantizer, OnlineHadamard, RMSNorm,
                              SignRotMoEBlock
    signrot_b200.transformers MultiLayerPagedKVCache4Bit, HFCacheAdapter

All GPU work goes through the C ABI of libsignrot_b200.so (include/signrot_b200.h); there is
no CPU or library fallback.  `install_as_signrot()` registers the package under the name
`signrot`, so code written against the reference (`import signrot.nn`, `signrot._CUDA`-free
call sites such as fake_quant/quant_utils.py:214-296) picks up these kernels unchanged.
"""
from __future__ import annotations

import importlib
import sys

from . import _lib
from .functional.quantization import pack_i4, unpack_i4, asym_quant_dequant, sym_quant_dequant
from .functional.hadamard import matmul_hadU_cuda, random_hadamard_matrix, apply_exact_had_to_linear
from . import functional
from . import nn

__version__ = "0.1.0"


def __getattr__(name):
    if name == "transformers":  # imported lazily: it pulls in Hugging Face transformers
        return importlib.import_module(__name__ + ".transformers")
    raise AttributeError(name)


def install_as_signrot() -> None:
    """Makes `import signrot`, `signrot.nn`, `signrot.functional[.kernel|.hadamard|...]` and
    `signrot.transformers` resolve to this package."""
    me = sys.modules[__name__]
    sys.modules["signrot"] = me
    for sub in ("functional", "functional.kernel", "functional.quantization", "functional.hadamard",
                "functional.hadamard_matrices", "nn", "nn.linear", "nn.quantization", "nn.hadamard",
                "nn.normalization", "nn.moe"):
        sys.modules["signrot." + sub] = importlib.import_module(__name__ + "." + sub)
    class _Lazy:  # signrot.transformers on first use
        pass
    try:
        sys.modules["signrot.transformers"] = importlib.import_module(__name__ + ".transformers")
        sys.modules["signrot.transformers.kv_cache"] = importlib.import_module(__name__ + ".transformers.kv_cache")
    except Exception:  # Hugging Face transformers missing: the kernels still work
        pass
