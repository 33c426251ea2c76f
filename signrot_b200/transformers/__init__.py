"""Same names as `signrot.transformers` (signrot/transformers/__init__.py:1)."""
from .kv_cache import MultiLayerPagedKVCache4Bit, HFCacheAdapter
from . import kernel_utils
