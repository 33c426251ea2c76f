"""Places the reference's own CPU code for this path under oracle/_ref/ (test infrastructure only).

    python -m oracle.build_ref          # needs a SignRot checkout ($SIGNROT_REFERENCE or ../reference)

The reference's CPU implementation of the quantized-linear path is Python: the fake-quant branch of
ActQuantWrapper.forward (fake_quant/quant_utils.py:322-386) with the functions it imports.  Those few
files are copied, unmodified, from the checkout where they lie into oracle/_ref/ -- a git-ignored
directory, so nothing of the reference enters this repository's history -- where oracle/ref_shim.py
finds them on a machine without the checkout.  bench.py's CPU legs then time the reference's own
forward (`cpu_baseline.kind` = "reference"); without the directory they time the oracle port.
"""
from __future__ import annotations

import os
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"

FILES = [
    "fake_quant/quant_utils.py", "fake_quant/utils.py", "fake_quant/hadamard_utils.py",
    "signrot/functional/hadamard.py", "signrot/functional/hadamard_matrices.py",
    "signrot/functional/quantization.py", "signrot/functional/kernel.py",
]


def checkout() -> Path | None:
    for c in (os.environ.get("SIGNROT_REFERENCE"), HERE.parents[1] / "reference"):
        if c and (Path(c) / "fake_quant" / "quant_utils.py").exists():
            return Path(c)
    return None


def populate(verbose: bool = False) -> bool:
    """Copies FILES from the checkout; returns False (and leaves oracle/_ref alone) without one."""
    src = checkout()
    if src is None:
        return DEST.exists()
    for rel in FILES:
        out = DEST / rel
        out.parent.mkdir(parents=True, exist_ok=True)
        if not out.exists() or out.stat().st_mtime < (src / rel).stat().st_mtime:
            shutil.copy2(src / rel, out)
            if verbose:
                print("copied", rel)
    return True


if __name__ == "__main__":
    print("oracle/_ref ready" if populate(True) else "no SignRot checkout found: oracle/_ref not populated")
