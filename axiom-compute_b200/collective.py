"""Fused matvec + all-gather over NVLink peer memory (one process per GPU).

``PeerGather`` owns the buffers: on every rank two alternating copies of ``slots`` full-length
vectors of (value, epoch) words and a small ``done`` array, all mapped into every rank's address
space by torch's symmetric memory (plumbing only; the stores and the waits are in the CUDA
kernels), plus a local fp32 copy and the epoch counter.  One step is any number of ``matvec()``
calls into distinct slots followed by ``finish()``:

* ``matvec`` launches the row-sharded Q4_K_M matvec whose epilogue stores this rank's slice into
  every rank's vector (the copy selected by the low bit of the step's epoch) without waiting for
  anyone;
* ``finish`` waits until every word of every slot carries the step's epoch and unpacks the values,
  after which ``vector(slot)`` is complete for later work in the same stream.  Its last CTA then
  ends the step: it tells every rank that this rank has consumed the step, waits until every rank
  has consumed the step before, and advances the epoch.  A rank can therefore run at most one step
  ahead of the slowest one, and the copy it writes next is free on every rank; a word from a later
  step than the reader's own would set bit 8 of the status word instead of being accepted.

With ``world == 1`` no process group is needed and the same kernels run on local memory.
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
        n = self.slots * self.rows_global
        self._n = n
        # [copy 0 | copy 1 | done words (one uint32 per rank, padded to 16 int64)]
        total = 2 * n + 16
        if group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()
                                 and torch.distributed.get_world_size() > 1):
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            if self.world > 16:
                raise ValueError("at most 16 ranks")
            self.pairs = symm_mem.empty(total, dtype=torch.int64, device=self.device)
            self.pairs.zero_()
            self._handle = symm_mem.rendezvous(self.pairs, group)
            ptrs = list(self._handle.buffer_ptrs)
            torch.cuda.synchronize(self.device)
            dist.barrier(group)   # every rank's zeroing is done before anyone stores into it
        else:
            self.pairs = torch.zeros(total, dtype=torch.int64, device=self.device)
            ptrs = [self.pairs.data_ptr()]
        self.parity_stride = n * 8
        self.ptr_table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        self.done_table = torch.tensor([p + 2 * n * 8 for p in ptrs], dtype=torch.int64, device=self.device)
        self.epoch = torch.ones(1, dtype=torch.int32, device=self.device)     # the first step is epoch 1
        self.arrive = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.values = torch.zeros(n, dtype=torch.float32, device=self.device)
        self.row_offset, self.rows_local = shard_rows(self.rows_global, self.world, self.rank)
        self._sync = _ffi.AxcGatherSync(self.done_table.data_ptr(), self.pairs.data_ptr() + 2 * n * 8,
                                        self.arrive.data_ptr(), self.epoch.data_ptr(), self.world, self.rank)

    def _stream(self) -> int:
        return int(torch.cuda.current_stream(self.device).cuda_stream)

    def vector(self, slot: int) -> torch.Tensor:
        """This rank's copy of the assembled vector of `slot` (complete after ``finish``)."""
        return self.values[slot * self.rows_global:(slot + 1) * self.rows_global]

    def matvec(self, q: torch.Tensor, x: torch.Tensor, n_superblocks: int, slot: int,
               status: Optional[torch.Tensor] = None, tuning=None) -> None:
        """Rows [row_offset, row_offset + rows_local) of `slot`, stored on every rank."""
        if not (q.is_cuda and x.is_cuda):
            raise ValueError("q and x must be CUDA tensors (this backend has no CPU path)")
        if q.numel() < self.rows_local * n_superblocks * 144 or x.numel() < n_superblocks * 256:
            raise ValueError("q or x too small for this rank's shard")
        if not 0 <= slot < self.slots:
            raise ValueError("slot out of range")
        g = _ffi.AxcGather(self.ptr_table.data_ptr(), slot * self.rows_global * 8, self.epoch.data_ptr(),
                           self.world, self.rank, self.row_offset, self.parity_stride)
        with torch.cuda.device(self.device):
            rc = _ffi.lib().axc_cuda_q4k_matvec_allgather(
                q.data_ptr(), x.data_ptr(), self.rows_local, n_superblocks, C.byref(g), self._stream(),
                status.data_ptr() if status is not None else None,
                C.byref(tuning) if tuning is not None else None)
        _raise_for(rc)

    def finish(self, status: Optional[torch.Tensor] = None, slots: Optional[int] = None,
               let_next_start: bool = False) -> None:
        """Wait for the step's words of the first `slots` slots (default all), unpack them, and end
        the step (handshake with the other ranks, epoch advanced): one launch.  `let_next_start`:
        the launches behind this one (the next step's matvecs, declared independent) may be
        scheduled while it still waits, so a stream or graph of several steps does not drain at
        the end of each; they must not read ``vector()`` before an ordered launch."""
        n = (self.slots if slots is None else int(slots)) * self.rows_global
        flags = _ffi.AXC_FINISH_LET_NEXT_START if let_next_start else 0
        with torch.cuda.device(self.device):
            rc = _ffi.lib().axc_cuda_gather_finish(
                self.pairs.data_ptr(), self.epoch.data_ptr(), self.values.data_ptr(), n, self._stream(),
                status.data_ptr() if status is not None else None, flags, self.parity_stride,
                C.byref(self._sync))
        _raise_for(rc)
