"""Hadamard matrices of order 12 ... 172 as float32 tensors (`get_had12()` ... `get_had172()`),
the same matrices as signrot/functional/hadamard_matrices.py:8-4200, decoded from the
bit-packed tables in hadamard_tables.py."""
from __future__ import annotations

import functools

import numpy as np
import torch

from .hadamard_tables import PACKED

ORDERS = tuple(sorted(PACKED))


@functools.lru_cache(maxsize=None)
def _decode(k: int) -> torch.Tensor:
    bits = PACKED[k]
    raw = bits.to_bytes((k * k + 7) // 8, "little")
    flat = np.unpackbits(np.frombuffer(raw, dtype=np.uint8), bitorder="little")[: k * k]
    h = torch.from_numpy(flat.astype(np.float32) * 2.0 - 1.0).reshape(k, k)
    return h


def get_had(k: int) -> torch.Tensor:
    """A fresh float32 [k, k] copy of the order-k matrix."""
    return _decode(k).clone()


def _getter(k):
    def get():
        return get_had(k)
    get.__name__ = f"get_had{k}"
    return get


for _k in ORDERS:
    globals()[f"get_had{_k}"] = _getter(_k)
