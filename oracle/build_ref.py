"""Places the reference's own CPU code for this path under oracle/_ref/ (test infrastructure only).

    python -m oracle.build_ref          # needs a SignRot checkout ($SIGNROT_REFERENCE or ../reference)

The reference's CPU implementation of the quantized-linear path is Python: the fake-quant branch of
ActQuantWrapper.forward (fake_quant/quant_utils.py:322-386) with the functions it imports.  Those few
files are copied, unmodified, from the checkout where they lie into oracle/_ref/ -- a git-ignored
directory, so nothing of the reference enters this repository's history -- where oracle/ref_shim.py
finds them on a machine without the checkout.  bench.py's CPU legs then time the reference's own
forward (`cpu_baseline.kind` = "reference"); without the directory they time the oracle port.

build_native() also compiles the reference's CUDA extension (signrot/kernels/*.cu + bindings.cpp, the
module the reference imports as signrot._CUDA) for sm_100a, straight from the checkout, into
oracle/_ref/native/_CUDA.so.  The sources need CUTLASS, whose submodule is empty in the checkout; the
header tree that ships inside the flashinfer wheel of this image is used instead (a build without that
wheel skips this step).  The module is a second, GPU-side checker: tests/test_gpu_reference_native.py
runs the reference's own kernels beside this library's on the same device buffers.  It is never on a
product path and never timed.
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


NATIVE = DEST / "native" / "_CUDA.so"
NATIVE_SOURCES = ["gemm.cu", "gemm_grouped.cu", "moe.cu", "quant.cu", "fused.cu", "flashinfer.cu", "bindings.cpp"]


def build_native(verbose: bool = False) -> bool:
    """Compiles the reference's extension module; returns whether oracle/_ref/native/_CUDA.so exists afterwards."""
    import subprocess
    import sysconfig
    from concurrent.futures import ThreadPoolExecutor
    src = checkout()
    if src is None:
        return NATIVE.exists()
    kdir = src / "signrot" / "kernels"
    newest = max((kdir / f).stat().st_mtime for f in NATIVE_SOURCES)
    if NATIVE.exists() and NATIVE.stat().st_mtime >= newest:
        return True
    try:
        import flashinfer
        import torch
        from torch.utils.cpp_extension import include_paths
    except ImportError:
        return False
    cutlass = Path(flashinfer.__file__).parent / "data" / "cutlass"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not (cutlass / "include" / "cutlass" / "cutlass.h").exists() or not Path(nvcc).exists():
        return False
    obj = NATIVE.parent / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{kdir / 'include'}", f"-I{cutlass / 'include'}", f"-I{cutlass / 'tools' / 'util' / 'include'}",
           *[f"-I{p}" for p in include_paths("cuda")], f"-I{sysconfig.get_paths()['include']}"]
    defs = ["-DTORCH_EXTENSION_NAME=_CUDA", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]

    def compile_one(name: str):
        out = obj / (name.rsplit(".", 1)[0] + ".o")
        if name.endswith(".cu"):
            cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
                   "--expt-extended-lambda", "-Xcompiler", "-fPIC", *defs, *inc, "-c", str(kdir / name), "-o", str(out)]
        else:
            cmd = ["g++", "-O2", "-std=c++17", "-fPIC", *defs, *inc, "-I/usr/local/cuda/include", "-c", str(kdir / name),
                   "-o", str(out)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{name}: {r.stderr[-2000:]}")
        return str(out)

    try:
        with ThreadPoolExecutor(max_workers=4) as pool:
            objs = list(pool.map(compile_one, NATIVE_SOURCES))
        tlib = Path(torch.__file__).parent / "lib"
        cmd = ["g++", "-shared", "-o", str(NATIVE), *objs, f"-L{tlib}", f"-Wl,-rpath,{tlib}", "-lc10", "-lc10_cuda",
               "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-L/usr/local/cuda/lib64", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(r.stderr[-2000:])
    except RuntimeError as e:
        if verbose:
            print("reference extension not built:", e)
        return False
    if verbose:
        print("built", NATIVE)
    return True


def load_native():
    """The reference's extension module (signrot._CUDA), or None when it was not built."""
    if not NATIVE.exists():
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location("_CUDA", str(NATIVE))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print("oracle/_ref ready" if populate(True) else "no SignRot checkout found: oracle/_ref not populated")
    print("reference extension:", "present" if build_native(True) else "not built")
