"""The C-ABI library loads and exports what include/signrot_b200.h declares; host-side
argument validation answers before anything is launched.  CPU only (no compute calls)."""
import ctypes
import subprocess

import pytest
import torch

from signrot_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert len(declared) >= 29
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    nm = subprocess.run(["nm", "-D", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in nm.splitlines() if " T sr_" in l}
    assert exported == set(declared), exported ^ set(declared)


def test_signature_table_covers_header():
    typed = set(_lib._SIGNATURES) | {"sr_last_error", "sr_version"}
    assert typed == set(_lib.declared_symbols())


def test_version():
    assert _lib.load().sr_version() == 100


def _err():
    return _lib.load().sr_last_error().decode()


def test_argument_errors_are_reported_on_the_host():
    lib = _lib.load()
    # K not a multiple of 32: the reference asserts in functional/kernel.py:68
    rc = lib.sr_matmul_i4(ctypes.c_void_p(16), ctypes.c_void_p(16), 4, 4, 48, 0, ctypes.c_void_p(16), None)
    assert rc == 1 and "32" in _err()
    rc = lib.sr_rope_qk(None, None, None, None, 1, 1, 1, 1, 1, 7, None)
    assert rc == 1 and "even head_dim" in _err()
    rc = lib.sr_kv_quant_pack(None, 4, 7, None, None, None)
    assert rc == 1 and "even last dimension" in _err()
    rc = lib.sr_batch_decode_i4(None, None, None, None, None, None, None, 1, 0, 8, 8, 16, 64, 2, None, 1, 0, None)
    assert rc == 1 and "head_dim" in _err()
    rc = lib.sr_hadamard(None, 0, 2, 96 * 3, None, 1, 1.0, None, 0, None, 0, None)
    assert rc == 1 and "power of two" in _err()
    rc = lib.sr_sym_dequant_moe(None, None, None, None, ctypes.c_void_p(8), None, 1, 1, None, None)
    assert rc == 1 and "together" in _err()
    rc = lib.sr_w4a4_linear(None, ctypes.c_void_p(8), ctypes.c_void_p(8), None, ctypes.c_void_p(8), None, None,
                            1, 1, 32, ctypes.c_void_p(8), None)
    assert rc == 1 and "row sums" in _err()
    # empty problems succeed without touching the device
    assert lib.sr_matmul_i4(None, None, 0, 16, 64, 0, None, None) == 0
    assert lib.sr_sym_quant_dynamic(None, 0, 128, 1.0, None, None, None) == 0
    assert lib.sr_swiglu(None, None, 0, None, None) == 0


def test_python_wrappers_refuse_cpu_tensors():
    from signrot_b200.functional import kernel
    x = torch.zeros(2, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        kernel.sym_quant_dynamic(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        kernel.matmul_si4_si4(torch.zeros(2, 32, dtype=torch.uint8), torch.zeros(2, 32, dtype=torch.uint8))
    with pytest.raises(AssertionError, match="multiplication of 32"):
        kernel.matmul_si4_si4(torch.zeros(2, 24, dtype=torch.uint8), torch.zeros(2, 24, dtype=torch.uint8))


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libsignrot_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()
