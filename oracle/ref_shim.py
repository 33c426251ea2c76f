"""Imports the reference's own Python on the CPU (test infrastructure only).

Works only where the reference's files are present: a SignRot checkout (its path in
$SIGNROT_REFERENCE, else the directory `reference` beside this repository's parent), else the
handful of its Python files that oracle/build_ref.py placed under oracle/_ref/ (git-ignored; that
directory travels to a GPU box with the built libraries).  Used by tests/golden/make_golden.py to
produce the committed golden vectors and by the CPU legs of bench.py to time the reference's own
fake-quant forward.

`import signrot` itself fails (signrot/__init__.py:5 imports the unbuilt CUDA extension), so
empty package objects named `signrot`, `signrot.functional`, ... are registered with
`__path__` pointing into the checkout; submodules then resolve normally.  Dependencies that
are absent from this image get stubs: `fast_hadamard_transform` (dense Sylvester product in
fp32 cast back to the input dtype: the contract of hadamard_transform(x, scale) as used at
signrot/functional/hadamard.py:81,85), `accelerate`, `termcolor`, and `signrot._CUDA`.
"""
from __future__ import annotations

import importlib
import os
import sys
import types
from pathlib import Path

import torch

def _find_reference() -> Path:
    cands = [os.environ.get("SIGNROT_REFERENCE"), Path(__file__).resolve().parents[2] / "reference",
             Path(__file__).resolve().parent / "_ref"]
    for c in cands:
        if c and (Path(c) / "signrot" / "functional" / "hadamard.py").exists():
            return Path(c)
    return Path(cands[1])


REF = _find_reference()


def available() -> bool:
    return (REF / "signrot" / "functional" / "hadamard.py").exists()


def _sylvester(n: int) -> torch.Tensor:
    h = torch.ones((1, 1), dtype=torch.float32)
    while h.shape[0] < n:
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return h


def _hadamard_transform(x, scale=1.0):
    """Stand-in for fast_hadamard_transform.hadamard_transform: fp32 sums, one rounding to the input
    dtype.  Up to 2048 points a dense Sylvester product; longer rows as H_a (x) H_b (two dense
    products of sqrt-size factors), which is the same transform with fewer operations."""
    n = x.shape[-1]
    if n <= 2048:
        y = torch.nn.functional.linear(x.float(), _sylvester(n)) * float(scale)
        return y.to(x.dtype)
    a = 1 << ((n.bit_length() - 1) // 2)
    b = n // a
    xf = x.float().reshape(-1, a, b)
    y = torch.matmul(_sylvester(a), torch.matmul(xf, _sylvester(b))) * float(scale)
    return y.reshape(x.shape).to(x.dtype)


_installed = False


def install():
    """Registers the stubs and package shells (idempotent)."""
    global _installed
    if _installed:
        return
    if not available():
        raise RuntimeError(f"no SignRot checkout at {REF}")
    import transformers  # noqa: F401  (must precede the accelerate stub)
    import transformers.models.llama.modeling_llama  # noqa: F401

    fht = types.ModuleType("fast_hadamard_transform")
    fht.hadamard_transform = _hadamard_transform
    sys.modules.setdefault("fast_hadamard_transform", fht)

    if "accelerate" not in sys.modules:
        acc = types.ModuleType("accelerate")

        class PartialState:
            device = torch.device("cpu")
            num_processes = 1
            process_index = 0
            is_main_process = True
            local_process_index = 0

            def wait_for_everyone(self):
                pass

        acc.PartialState = PartialState
        acc.Accelerator = type("Accelerator", (), {})
        acc.dispatch_model = lambda m, **k: m
        acc.infer_auto_device_map = lambda *a, **k: {}
        acc.__path__ = []
        utils = types.ModuleType("accelerate.utils")
        utils.gather_object = lambda x: x
        utils.broadcast = lambda x, **k: x
        utils.get_max_memory = lambda *a, **k: {}
        utils.get_balanced_memory = lambda *a, **k: {}
        utils.wait_for_everyone = lambda: None
        hooks = types.ModuleType("accelerate.hooks")
        hooks.attach_align_device_hook = lambda *a, **k: None
        acc.utils, acc.hooks = utils, hooks
        sys.modules["accelerate"] = acc
        sys.modules["accelerate.utils"] = utils
        sys.modules["accelerate.hooks"] = hooks
    if "termcolor" not in sys.modules:
        tc = types.ModuleType("termcolor")
        tc.colored = lambda s, *a, **k: s
        sys.modules["termcolor"] = tc

    for name, sub in (("signrot", "signrot"), ("signrot.functional", "signrot/functional"),
                      ("signrot.nn", "signrot/nn"), ("signrot.transformers", "signrot/transformers")):
        if name in sys.modules and getattr(sys.modules[name], "__file__", None):
            raise RuntimeError(f"a real module named {name} is already imported; the shim needs the name free")
        m = types.ModuleType(name)
        m.__path__ = [str(REF / sub)]
        sys.modules[name] = m
    cuda = types.ModuleType("signrot._CUDA")  # never called on the CPU paths used here
    sys.modules["signrot._CUDA"] = cuda
    sys.modules["signrot"]._CUDA = cuda
    sys.path.insert(0, str(REF / "fake_quant"))
    _installed = True


def module(name: str):
    """Imports a reference module, e.g. 'signrot.functional.hadamard' or 'quant_utils'."""
    install()
    return importlib.import_module(name)
