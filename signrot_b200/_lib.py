"""ctypes binding of libsignrot_b200.so (the C ABI declared in include/signrot_b200.h).

The library is loaded from the package directory.  There is no fallback: if the
shared object is missing, or a call is made without a CUDA tensor, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import re
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libsignrot_b200.so"
HEADER_PATH = _PKG.parent / "include" / "signrot_b200.h"

SR_F16, SR_BF16, SR_F32 = 0, 1, 2
DTYPE_TAG = {torch.float16: SR_F16, torch.bfloat16: SR_BF16, torch.float32: SR_F32}

_lib = None

_P = ctypes.c_void_p
_I64 = ctypes.c_int64
_I = ctypes.c_int
_F = ctypes.c_float

# argument types of every entry point, in header order
_SIGNATURES = {
    "sr_device_status": [ctypes.POINTER(ctypes.c_int), _I],
    "sr_matmul_i4": [_P, _P, _I64, _I64, _I64, _I, _P, _P],
    "sr_matmul_i4_ld": [_P, _I64, _P, _I64, _I64, _I64, _I, _P, _P],
    "sr_w4a4_linear": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P],
    "sr_w4a4_linear_ws_bytes": [_I64, _I64, _I64, _P],
    "sr_w4a4_linear_ws": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _I64, _P, _P],
    "sr_w4a4_swiglu": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P],
    "sr_grouped_linear": [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _P, _P],
    "sr_matmul_grouped": [_P, _I64, _P, _P, _P, _P, _P, _P, _I, _I64, _P],
    "sr_selftest_bounded_wait": [_I64, _P],
    "sr_sym_quant_dynamic": [_P, _I64, _I64, _F, _P, _P, _P],
    "sr_asym_quant_dynamic": [_P, _I64, _I64, _F, _P, _P, _P, _P],
    "sr_sym_quant_dynamic_moe": [_P, _P, _P, _I64, _I64, _F, _P, _P, _P],
    "sr_asym_quant_dynamic_moe": [_P, _P, _P, _I64, _I64, _F, _P, _P, _P, _P],
    "sr_sym_quant": [_P, _P, _I64, _I64, _P, _P],
    "sr_asym_quant_f16_si4": [_P, _P, _P, _I64, _I64, _P, _P],
    "sr_asym_quant_f16_ui4": [_P, _P, _P, _I64, _I64, _P, _P],
    "sr_sym_dequant": [_P, _P, _P, _I64, _I64, _P, _P],
    "sr_sym_dequant_moe": [_P, _P, _P, _P, _P, _P, _I64, _I64, _P, _P],
    "sr_sum_i4": [_P, _I64, _I64, _I, _P, _P],
    "sr_matmul_colrow_i8_i32": [_P, _P, _I64, _I64, _P, _P],
    "sr_hadamard": [_P, _I, _I64, _I64, _P, _I64, _F, _P, _I, _P, _I, _P],
    "sr_hadamard_heads": [_P, _I, _I64, _I64, _I64, _F, _I, _P, _I, _P],
    "sr_rotate_quant": [_P, _I, _I64, _I64, _P, _I64, _F, _P, _P, _I64, _F, _I, _P, _P, _P, _P, _P],
    "sr_moe_route": [_P, _I64, _I64, _I64, _I, _P, _P, _P, _P, _P, _P, _P],
    "sr_moe_gather": [_P, _P, _P, _P, _I64, _I64, _P, _P, _P, _P],
    "sr_moe_combine": [_P, _P, _P, _P, _I64, _I64, _I64, _I, _P, _P],
    "sr_rtn_pack": [_P, _I, _I64, _I64, _P, _I, _P, _P, _P],
    "sr_rmsnorm": [_P, _I64, _I64, _F, _I64, _P, _P],
    "sr_add_rmsnorm_quant": [_P, _P, _I64, _I64, _F, _I64, _F, _I, _P, _P, _P, _P, _P, _P],
    "sr_rope_qk": [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "sr_swiglu": [_P, _P, _I64, _P, _P],
    "sr_kv_quant_pack": [_P, _I64, _I64, _P, _P, _P],
    "sr_append_kv_i4": [_P] * 9 + [_I64] * 6 + [_P],
    "sr_init_kv_i4": [_P] * 10 + [_I64] * 7 + [_P],
    "sr_kv_append_quant": [_P] * 7 + [_I64] * 7 + [_I, _P],
    "sr_rope_kv_append": [_P] * 8 + [_I64] * 3 + [_P, _P, _I64, _P, _P] + [_I64] * 8 + [_I, _P],
    "sr_batch_decode_i4": [_P] * 7 + [_I64] * 7 + [_P, _I64, _I, _P],
    "sr_rope_decode_i4": [_P] * 4 + [_I64] * 3 + [_P, _P, _I64] + [_P] * 5 + [_I64] * 7 + [_P, _I64, _I, _I, _P],
    "sr_batch_decode_i4_merged": [_P] * 7 + [_I64] * 7 + [_P, _I64, _P, _I, _P],
    "sr_peer_region_bytes": [_I64, _I64, ctypes.POINTER(ctypes.c_int64)],
    "sr_peer_alloc": [_I64, ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p],
    "sr_peer_open": [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)],
    "sr_peer_close": [_P],
    "sr_peer_free": [_P],
    "sr_peer_exchange": [_I, ctypes.POINTER(ctypes.c_void_p), _I, _I, _I64, _P, _I64, _I64, _P, _P, _P, _P],
    "sr_decode_advance": [_P] * 5 + [_I64] * 3 + [_P],
    "sr_batch_decode_i4_static": [_P] * 7 + [_I64] * 7 + [_I64, _I, _P],
}


def declared_symbols() -> list[str]:
    """Names of all functions the public header declares."""
    text = HEADER_PATH.read_text()
    return sorted(set(re.findall(r"\b(sr_[a-z0-9_]+)\s*\(", text)))


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and attaches argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m signrot_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(os.fspath(LIB_PATH))
    lib.sr_last_error.restype = ctypes.c_char_p
    lib.sr_last_error.argtypes = []
    lib.sr_version.restype = ctypes.c_int
    lib.sr_version.argtypes = []
    for name, args in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = args
    _lib = lib
    return lib


def ptr(t: torch.Tensor | None):
    """Device address of a tensor (None -> NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def call(name: str, *args) -> None:
    """Calls an entry point on the current stream; raises RuntimeError on a non-zero status,
    as the reference's TORCH_CHECKs do."""
    lib = load()
    rc = getattr(lib, name)(*args, stream())
    if rc != 0:
        raise RuntimeError(lib.sr_last_error().decode() or f"{name} failed with status {rc}")


def run(dev: torch.device, name: str, *args) -> None:
    """`call` with the tensor's device made current (kernels launch on the current device)."""
    if dev is not None and dev.index is not None and dev.index != torch.cuda.current_device():
        with torch.cuda.device(dev):
            call(name, *args)
    else:
        call(name, *args)


def call_nostream(name: str, *args) -> None:
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise RuntimeError(lib.sr_last_error().decode() or f"{name} failed with status {rc}")


def device_status(clear: bool = True) -> int:
    lib = load()
    out = ctypes.c_int(0)
    rc = lib.sr_device_status(ctypes.byref(out), 1 if clear else 0)
    if rc != 0:
        raise RuntimeError(lib.sr_last_error().decode())
    return out.value


def require_cuda(name: str, *tensors: torch.Tensor | None, strided: tuple = ()) -> torch.device:
    """All given tensors must be contiguous CUDA tensors on one device
    (signrot/kernels/bindings.cpp:15-20).  Tensors also listed in `strided` may be views whose
    strides the caller passes to the library."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"{name}: expected a CUDA tensor, got {t.device} (no CPU fallback)")
        if not t.is_contiguous() and not any(t is s for s in strided):
            raise RuntimeError(f"{name}: tensor must be contiguous")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{name}: tensors are on different devices ({dev} and {t.device})")
    return dev
