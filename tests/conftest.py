"""pytest configuration: the `gpu` marker, import path, shared helpers."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library must exist before any test touches it (build is incremental)."""
    from signrot_b200 import build
    build.build()


def load_golden(name: str):
    return np.load(GOLDEN / name)


def t(a: np.ndarray, bf16: bool = False) -> torch.Tensor:
    x = torch.from_numpy(np.ascontiguousarray(a))
    return x.view(torch.bfloat16) if bf16 else x


def code_mismatch(a: torch.Tensor, b: torch.Tensor):
    """(fraction of differing codes, max |difference|)."""
    d = (a.to(torch.int32) - b.to(torch.int32)).abs()
    return (d != 0).float().mean().item(), int(d.max().item()) if d.numel() else 0


def assert_codes_close(got, want, frac=1e-4):
    """Act-quant codes may differ only by +-1 (exact rounding ties), in at most `frac` of the
    elements."""
    f, m = code_mismatch(got, want)
    assert m <= 1, f"codes differ by {m}"
    assert f <= frac, f"{f:.2e} of the codes differ (limit {frac:.0e})"


def rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    g, w = got.double(), want.double()
    return ((g - w).norm() / w.norm().clamp_min(1e-30)).item()
