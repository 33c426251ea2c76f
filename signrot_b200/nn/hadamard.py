"""Online Hadamard module (signrot/nn/hadamard.py:8-56): rotation, optional +-1 sign vector
(`had_adj_sign`, the SignRot adjustment) and cast back, in one kernel launch."""
from __future__ import annotations

import torch

from ..functional import kernel
from ..functional.hadamard import get_hadK


class OnlineHadamard(torch.nn.Module):
    had_adj_sign: torch.Tensor | None

    def __init__(self, hadamard_dim, tied_module=None, force_fp32=False, had_adj=False, dynamic_adj=False):
        super().__init__()
        self.fp32_had = force_fp32
        had_rem_dim, self.rem_dim = get_hadK(hadamard_dim)
        if had_rem_dim is not None:
            self.register_buffer("had_rem_dim", had_rem_dim)
            if not self.fp32_had:
                self.had_rem_dim = self.had_rem_dim.to(torch.float16)
        else:
            self.had_rem_dim = None
        self.register_buffer("had_adj_sign", None)
        if had_adj:
            self.register_buffer("had_adj_sign", torch.ones(hadamard_dim, dtype=torch.int8))
        self.dynamic_adj = dynamic_adj
        self.module = tied_module

    def forward(self, x: torch.Tensor):
        sign = self.had_adj_sign
        if sign is not None and not self._had_adj_ready_cached:
            raise RuntimeError("Dynamic hadamard adjustment not implemented yet.")
        return kernel.hadamard(x, self.had_rem_dim, self.rem_dim, sign=sign, fp32_mode=self.fp32_had,
                               out_dtype=x.dtype)

    @property
    def _had_adj_ready_cached(self):
        # reading the device tensor is a host sync, so the answer is cached (the sign vector
        # is frozen once the kernel modules exist)
        ready = getattr(self, "_had_adj_ready_flag", None)
        if ready is None:
            ready = self.had_adj_ready()
            self._had_adj_ready_flag = ready
        return ready

    def had_adj_ready(self):
        return bool(self.had_adj_sign is not None and torch.all(self.had_adj_sign != 0))
