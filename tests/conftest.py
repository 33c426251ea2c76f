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


def assert_act_quant_matches(got_packed, got_scale, want_rot_h, clip: float = 1.0, scale_frac: float = 0.01):
    """Per-token symmetric int4 codes + scales of a fused kernel against the oracle, every row checked.

    The scale is rn_h(amax / 7): it equals the oracle's unless the row maximum itself moved by one
    fp16 ulp, and then the two scales must be ADJACENT fp16 values (at most `scale_frac` of the rows).
    The codes of every row are compared with the oracle's quantizer run on the oracle's rotated row
    with the scale the kernel wrote: +-1 at rounding ties, at most 1e-4 of the elements."""
    import oracle
    gs = got_scale.detach().cpu().reshape(-1).contiguous()
    codes_ref, scale_ref = oracle.sym_quant_dynamic(want_rot_h, clip)
    ws = scale_ref.reshape(-1).contiguous()
    step = (gs.view(torch.int16).int() - ws.view(torch.int16).int()).abs()
    assert int(step.max()) <= 1, f"a scale is {int(step.max())} fp16 steps from the oracle's"
    moved = int((step != 0).sum())
    frac = moved / max(1, step.numel())
    assert moved <= max(1, int(scale_frac * step.numel())), \
        f"{moved} of {step.numel()} row scales differ from the oracle's (limit {scale_frac:.0e} of the rows)"
    want = oracle.sym_quant_codes(want_rot_h.reshape(-1, want_rot_h.shape[-1]), gs)
    assert_codes_close(oracle.unpack_i4(got_packed.detach().cpu()).reshape(want.shape), want)
    return frac


def rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    g, w = got.double(), want.double()
    return ((g - w).norm() / w.norm().clamp_min(1e-30)).item()
