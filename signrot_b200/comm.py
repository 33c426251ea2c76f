"""Exchanges between the GPUs of a tensor- or expert-parallel group over peer memory.

`PeerGroup` gives every rank of a `torch.distributed` group (one process per GPU, one node) a region of
device memory that all peers map through CUDA inter-process handles; `torch.distributed` is used once, at
set-up, to pass the handles around.  After that an exchange is ONE kernel launch per rank
(`sr_peer_exchange`: push with peer stores, flag, bounded wait, combine), with no host synchronisation, so a
decode step that contains exchanges can be captured in a CUDA graph.  Messages that do not fit the slots
(prefill-size tensors) go through the collective library instead: `fits()` tells which.

The reference has no multi-GPU form of this path (fake_quant/kernel_utils.py:365-366).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib

GATHER, REDUCE_I32_DEQUANT, REDUCE_F32 = 0, 1, 2
_ELEM = {GATHER: 2, REDUCE_I32_DEQUANT: 4, REDUCE_F32: 4}


class PeerGroup:
    def __init__(self, group=None, slot_bytes: int = 2 << 20, device=None):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("peer exchanges take groups of up to 8 ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.slot_bytes = int(slot_bytes)
        lib = _lib.load()
        total = ctypes.c_int64(0)
        self._check(lib.sr_peer_region_bytes(self.world, self.slot_bytes, ctypes.byref(total)))
        handle = ctypes.create_string_buffer(64)
        own = ctypes.c_void_p(0)
        with torch.cuda.device(self.device):
            self._check(lib.sr_peer_alloc(total.value, ctypes.byref(own), handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self._regions = (ctypes.c_void_p * self.world)()
            self._opened = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self._regions[r] = own.value
                    continue
                p = ctypes.c_void_p(0)
                self._check(lib.sr_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
                self._regions[r] = p.value
                self._opened.append(p.value)
        self._own = own.value
        dist.barrier(group=group)        # every region is zeroed and mapped before the first exchange

    @staticmethod
    def _check(rc):
        if rc != 0:
            raise RuntimeError(_lib.load().sr_last_error().decode())

    def fits(self, rows: int, cols: int, mode: int) -> bool:
        return rows * cols * _ELEM[mode] <= self.slot_bytes

    def _exchange(self, mode, src, rows, cols, out, row_scale=None, col_scale=None):
        _lib.run(self.device, "sr_peer_exchange", mode, self._regions, self.rank, self.world, self.slot_bytes,
                 _lib.ptr(src), rows, cols, _lib.ptr(row_scale), _lib.ptr(col_scale), _lib.ptr(out))
        return out

    def all_gather_cols(self, x_local: torch.Tensor) -> torch.Tensor:
        """fp16 [rows, cols] on every rank -> fp16 [rows, world * cols], rank r's columns at [r * cols, (r + 1) * cols)."""
        assert x_local.dtype == torch.float16 and x_local.dim() == 2
        x_local = x_local.contiguous()
        rows, cols = x_local.shape
        out = torch.empty((rows, self.world * cols), dtype=torch.float16, device=x_local.device)
        return self._exchange(GATHER, x_local, rows, cols, out)

    def all_reduce_dequant(self, acc: torch.Tensor, row_scale: torch.Tensor, col_scale: torch.Tensor) -> torch.Tensor:
        """int32 partial sums [rows, cols] of a row-parallel W4A4 linear -> its fp16 output: exact integer sum over
        the ranks, then rn_h((float(sum) * row_scale) * col_scale) as on one GPU."""
        assert acc.dtype == torch.int32 and acc.dim() == 2 and acc.is_contiguous()
        rows, cols = acc.shape
        out = torch.empty((rows, cols), dtype=torch.float16, device=acc.device)
        return self._exchange(REDUCE_I32_DEQUANT, acc, rows, cols, out, row_scale.contiguous(), col_scale.contiguous())

    def all_reduce_f32(self, part: torch.Tensor) -> torch.Tensor:
        """fp32 [rows, cols] partial outputs -> fp16 of their sum, added in rank order on every rank."""
        assert part.dtype == torch.float32 and part.dim() == 2 and part.is_contiguous()
        rows, cols = part.shape
        out = torch.empty((rows, cols), dtype=torch.float16, device=part.device)
        return self._exchange(REDUCE_F32, part, rows, cols, out)

    def close(self):
        """Unmaps the peers' regions and frees the own one.  Collective: every rank calls it, none may have an
        exchange in flight."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        lib = _lib.load()
        with torch.cuda.device(self.device):
            for p in self._opened:
                lib.sr_peer_close(p)
            dist.barrier(group=self.group)
            lib.sr_peer_free(self._own)
        self._own, self._opened = None, []
