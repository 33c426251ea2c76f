"""Modules with the names of `signrot.nn` (signrot/nn/__init__.py:1-5)."""
from .linear import Linear4bit, AsymSymmLinear4bit
from .normalization import RMSNorm
from .quantization import Quantizer, SymQuantizer, AsymQuantizer
from .hadamard import OnlineHadamard
from .moe import SignRotMoEBlock
