"""Fused matvec + all-gather over NVLink peer memory (one process per GPU).

``PeerGather`` owns the symmetric buffers: ``slots`` full-length y vectors and one flag row per
slot on every rank, mapped into every rank's address space by torch's symmetric memory
(plumbing only; the stores, flags and waits are in the CUDA kernel).  ``matvec`` launches the
row-sharded Q4_K_M matvec whose epilogue writes this rank's slice into every rank's vector and
returns the assembled local vector (valid for later work in the same stream).
With ``world == 1`` it needs no process group and degenerates to a plain matvec into the buffer.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _ffi
from .runtime import _raise_for
from .sharding import shard_rows


class PeerGather:
    def __init__(self, rows_global: int, slots: int, device, group=None):
        self.rows_global, self.slots = int(rows_global), int(slots)
        self.device = torch.device(device)
        self.world, self.rank = 1, 0
        n_y = self.slots * self.rows_global
        if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()
                                 and torch.distributed.get_world_size() > 1):
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            self.y_store = symm_mem.empty(n_y, dtype=torch.float32, device=self.device)
            self.flags = symm_mem.empty(self.slots * self.world, dtype=torch.int32, device=self.device)
            self.y_store.zero_()
            self.flags.zero_()
            hy = symm_mem.rendezvous(self.y_store, group)
            hf = symm_mem.rendezvous(self.flags, group)
            y_ptrs, f_ptrs = list(hy.buffer_ptrs), list(hf.buffer_ptrs)
            self._handles = (hy, hf)
            torch.cuda.synchronize(self.device)
            dist.barrier(group)   # every rank's zeroing is done before anyone stores into it
        else:
            self.y_store = torch.zeros(n_y, dtype=torch.float32, device=self.device)
            self.flags = torch.zeros(self.slots, dtype=torch.int32, device=self.device)
            y_ptrs, f_ptrs = [self.y_store.data_ptr()], [self.flags.data_ptr()]
        self.y_ptr_table = torch.tensor(y_ptrs, dtype=torch.int64, device=self.device)
        self.f_ptr_table = torch.tensor(f_ptrs, dtype=torch.int64, device=self.device)
        self.local_words = torch.zeros(2 * self.slots, dtype=torch.int32, device=self.device)
        self.row_offset, self.rows_local = shard_rows(self.rows_global, self.world, self.rank)

    def vector(self, slot: int) -> torch.Tensor:
        """This rank's copy of the assembled vector of `slot`."""
        return self.y_store[slot * self.rows_global:(slot + 1) * self.rows_global]

    def matvec(self, q: torch.Tensor, x: torch.Tensor, n_superblocks: int, slot: int,
               status: Optional[torch.Tensor] = None, tuning=None) -> torch.Tensor:
        """y[row_offset : row_offset + rows_local] = this rank's rows; returns the full vector."""
        if not (q.is_cuda and x.is_cuda):
            raise ValueError("q and x must be CUDA tensors (this backend has no CPU path)")
        if q.numel() < self.rows_local * n_superblocks * 144 or x.numel() < n_superblocks * 256:
            raise ValueError("q or x too small for this rank's shard")
        g = _ffi.AxcGather(self.y_ptr_table.data_ptr(), self.f_ptr_table.data_ptr(),
                           slot * self.rows_global * 4, slot * self.world * 4,
                           self.local_words.data_ptr() + slot * 8, self.world, self.rank, self.row_offset)
        with torch.cuda.device(self.device):
            rc = _ffi.lib().axc_cuda_q4k_matvec_allgather(
                q.data_ptr(), x.data_ptr(), self.rows_local, n_superblocks, C.byref(g),
                int(torch.cuda.current_stream().cuda_stream),
                status.data_ptr() if status is not None else None,
                C.byref(tuning) if tuning is not None else None)
        _raise_for(rc)
        return self.vector(slot)
