"""Functional layer: same names as `signrot.functional` (signrot/functional/__init__.py:1-5)."""
from .quantization import pack_i4, unpack_i4, unpack_ui4, asym_quant_dequant, sym_quant_dequant
from .hadamard import matmul_hadU, matmul_hadU_cuda, random_hadamard_matrix, apply_exact_had_to_linear, get_hadK
from . import kernel
