"""Hadamard transforms with the interface of `signrot.functional.hadamard`
(signrot/functional/hadamard.py:14-133).

`matmul_hadU` is the device-agnostic butterfly used offline (weight rotation, random
rotation matrices); `matmul_hadU_cuda` is the online transform and runs on the library's
rotation kernel (it replaces fast_hadamard_transform plus the had-K matmul)."""
from __future__ import annotations

import math
from collections import OrderedDict

import torch

from . import hadamard_matrices as _hm
from . import kernel as _kernel

# largest known order first, as signrot/functional/hadamard.py:14-32
KNOWN_HADAMARD_MATRICES = OrderedDict(
    (k, getattr(_hm, f"get_had{k}")) for k in (172, 156, 148, 140, 108, 60, 52, 40, 36, 28, 20, 12))


def is_pow2(n):
    return n > 0 and (n & (n - 1)) == 0


def get_hadK(n, transpose=False):
    """(hadK, K): the first table order K with n % K == 0 and n / K a power of two, else
    (None, 1) for power-of-two n (hadamard.py:33-40)."""
    for K, getter in KNOWN_HADAMARD_MATRICES.items():
        if n % K == 0 and is_pow2(n // K):
            h = getter()
            return (h.T if transpose else h), K
    assert is_pow2(n), "No known Hadamard matrix factor found and n is not a power of 2!"
    return None, 1


def matmul_hadU(X, transpose=False, hadK=None, K=None) -> torch.Tensor:
    """(hadK (x) H_{n/K}) X / sqrt(n) over the last dimension by radix-2 butterflies in X's
    dtype; any device (hadamard.py:43-65)."""
    n = X.shape[-1]
    if K is None:
        hadK, K = get_hadK(n, transpose)
    y = X.reshape(-1, K, n // K).clone()
    h = 1
    seg = n // K
    while h < seg:
        y = y.view(y.shape[0], K, seg // (2 * h), 2, h)
        a, b = y[:, :, :, 0, :], y[:, :, :, 1, :]
        y = torch.stack((a + b, a - b), dim=3)
        h *= 2
    y = y.reshape(-1, K, seg)
    if K > 1:
        y = hadK.to(y).view(1, K, K) @ y
    return y.reshape(X.shape) / torch.tensor(n).sqrt()


def matmul_hadUt(X):
    return matmul_hadU(X, transpose=True)


def random_hadamard_matrix(size, device):
    """Randomized Hadamard matrix H diag(+-1) in float64 (hadamard.py:70-75); the diagonal
    comes from torch.randint, so torch.manual_seed fixes it."""
    d = torch.randint(low=0, high=2, size=(size,)).to(torch.float64) * 2 - 1
    return matmul_hadU(torch.diag(d)).to(device)


def matmul_hadU_cuda(X, hadK, K):
    """Online transform on the GPU (hadamard.py:78-87): Walsh-Hadamard over each of the K
    segments with scale 1/sqrt(n) (fp32 sums, rounded to X's dtype), then the K x K factor."""
    return _kernel.hadamard(X, hadK, K)


def matmul_hadUt_cuda(X, hadK, K):
    """Transposed variant; only symmetric factors are supported online (the reference's
    version of this function passes an unsupported keyword and cannot be called)."""
    if K > 1:
        return _kernel.hadamard(X, hadK.T.contiguous(), K)
    return _kernel.hadamard(X, None, 1)


def apply_exact_had_to_linear(module, had_dim=-1, output=False):
    """Folds an exact Hadamard into a Linear's weight, offline (hadamard.py:95-128), in fp32 on the
    weight's own device."""
    assert isinstance(module, torch.nn.Linear)
    in_features, out_features = module.in_features, module.out_features
    if had_dim != -1:
        assert is_pow2(had_dim), "Hadamard dimension must be a power of 2!"
    W = module.weight.data
    dtype = W.dtype
    Wf = W.float()

    def transform(x, hadK, K):
        # on the GPU the fold runs through the library's fp32 transform (one launch per matrix),
        # on the CPU through the torch butterfly
        if x.is_cuda:
            return _kernel.hadamard(x.contiguous(), hadK, K, fp32_mode=True)
        return matmul_hadU(x, hadK=hadK, K=K)

    if had_dim == -1:
        if output:
            hadK, K = get_hadK(out_features)
            Wf = transform(Wf.t().contiguous(), hadK, K).t()
        else:
            hadK, K = get_hadK(in_features)
            Wf = transform(Wf, hadK, K)
    else:
        if not output:
            raise NotImplementedError("Not implemented (or tested) yet!")
        Wt = Wf.t().contiguous()
        shape = Wt.shape
        Wt = transform(Wt.reshape(-1, shape[-1] // had_dim, had_dim), None, 1)
        Wf = Wt.reshape(shape).t()
    module.weight.data = Wf.contiguous().to(dtype=dtype)
