"""Device-layer entry points on torch CUDA tensors (weights and activations resident in HBM).

torch is used for device memory and streams only; every function forwards raw device pointers
and the current stream to ``libaxc_cuda.so``.  No function here computes anything itself and
none has a CPU path: a non-CUDA tensor is an error.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _ffi
from .runtime import _raise_for

Q4K_SB_BYTES, Q4K_SB_ELEMS = 144, 256
Q4_0_BLK_BYTES, Q4_0_BLK_ELEMS = 18, 32


def _stream_ptr() -> int:
    return int(torch.cuda.current_stream().cuda_stream)


def _chk(t: torch.Tensor, dtype, name: str, min_elems: int) -> int:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this backend has no CPU path)")
    if t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous {dtype}")
    if t.numel() < min_elems:
        raise ValueError(f"{name} has {t.numel()} elements, needs >= {min_elems}")
    return t.data_ptr()


def make_tuning(ctas_per_sm: int = 0, tile_rows: int = 0, stages: int = 0, threads: int = 0,
                evict_first: int = -1, pdl: int = 2, resident: int = 0) -> _ffi.AxcTuning:
    return _ffi.AxcTuning(ctas_per_sm, tile_rows, stages, threads, evict_first, pdl, resident)


def new_status(device=None) -> torch.Tensor:
    """Device word that receives kernel error bits (0 = clean)."""
    return torch.zeros(1, dtype=torch.int32, device=device or "cuda")


def _matvec(fn_name, blk_bytes, blk_elems, q, x, rows, n, y, status, tuning):
    qp = _chk(q, torch.uint8, "q", rows * n * blk_bytes)
    xp = _chk(x, torch.float32, "x", n * blk_elems)
    if y is None:
        y = torch.empty(rows, dtype=torch.float32, device=q.device)
    yp = _chk(y, torch.float32, "y", rows)
    sp = _chk(status, torch.int32, "status", 1) if status is not None else None
    with torch.cuda.device(q.device):
        rc = getattr(_ffi.lib(), fn_name)(qp, xp, yp, rows, n, _stream_ptr(), sp,
                                          C.byref(tuning) if tuning is not None else None)
    _raise_for(rc)
    return y


def q4k_matvec(q: torch.Tensor, x: torch.Tensor, rows: int, n_superblocks: int,
               y: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
               tuning: Optional[_ffi.AxcTuning] = None) -> torch.Tensor:
    """y[r] = q4km_dequant_matvec(q row r, x): ``rows`` reference calls
    (examples/q4km_dequant_matvec.axc) in one launch."""
    return _matvec("axc_cuda_q4k_matvec", Q4K_SB_BYTES, Q4K_SB_ELEMS, q, x, rows, n_superblocks,
                   y, status, tuning)


def q4_0_matvec(q: torch.Tensor, x: torch.Tensor, rows: int, n_blocks: int,
                y: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
                tuning: Optional[_ffi.AxcTuning] = None) -> torch.Tensor:
    """y[r] = q4_0_dequant_matvec(q row r, x) (examples/q4_0_dequant_matvec.axc)."""
    return _matvec("axc_cuda_q4_0_matvec", Q4_0_BLK_BYTES, Q4_0_BLK_ELEMS, q, x, rows, n_blocks,
                   y, status, tuning)


def _matvec_seq(fn_name, blk_bytes, blk_elems, q, x, rows, n, y):
    qp = _chk(q, torch.uint8, "q", rows * n * blk_bytes)
    xp = _chk(x, torch.float32, "x", n * blk_elems)
    if y is None:
        y = torch.empty(rows, dtype=torch.float32, device=q.device)
    yp = _chk(y, torch.float32, "y", rows)
    with torch.cuda.device(q.device):
        rc = getattr(_ffi.lib(), fn_name)(qp, xp, yp, rows, n, _stream_ptr())
    _raise_for(rc)
    return y


def q4k_matvec_seq(q, x, rows: int, n_superblocks: int, y=None) -> torch.Tensor:
    """Reference operation order; y is bit-identical to ``q4km_dequant_matvec_cpu``."""
    return _matvec_seq("axc_cuda_q4k_matvec_seq", Q4K_SB_BYTES, Q4K_SB_ELEMS, q, x, rows,
                       n_superblocks, y)


def q4_0_matvec_seq(q, x, rows: int, n_blocks: int, y=None) -> torch.Tensor:
    """Reference operation order; y is bit-identical to ``q4_0_dequant_matvec_cpu``."""
    return _matvec_seq("axc_cuda_q4_0_matvec_seq", Q4_0_BLK_BYTES, Q4_0_BLK_ELEMS, q, x, rows,
                       n_blocks, y)


def _dequant(fn_name, blk_bytes, blk_elems, q, rows, n):
    qp = _chk(q, torch.uint8, "q", rows * n * blk_bytes)
    w = torch.empty((rows, n * blk_elems), dtype=torch.float32, device=q.device)
    with torch.cuda.device(q.device):
        rc = getattr(_ffi.lib(), fn_name)(qp, w.data_ptr(), rows, n, _stream_ptr())
    _raise_for(rc)
    return w


def q4k_dequant(q: torch.Tensor, rows: int, n_superblocks: int) -> torch.Tensor:
    """Bit-exact dequantised weights, shape (rows, n_superblocks * 256)."""
    return _dequant("axc_cuda_q4k_dequant", Q4K_SB_BYTES, Q4K_SB_ELEMS, q, rows, n_superblocks)


def q4_0_dequant(q: torch.Tensor, rows: int, n_blocks: int) -> torch.Tensor:
    """Bit-exact dequantised weights, shape (rows, n_blocks * 32)."""
    return _dequant("axc_cuda_q4_0_dequant", Q4_0_BLK_BYTES, Q4_0_BLK_ELEMS, q, rows, n_blocks)


def q4k_matvec_plan(rows: int, n_superblocks: int, tuning=None, sm_count: int = 148) -> dict:
    """Launch geometry the Q4_K_M matvec would use (no GPU needed)."""
    out = (C.c_int32 * 5)()
    rc = _ffi.lib().axc_cuda_q4k_matvec_plan(rows, n_superblocks,
                                             C.byref(tuning) if tuning is not None else None,
                                             sm_count, out)
    _raise_for(rc)
    return {"grid": out[0], "block": out[1], "smem": out[2], "tile_rows": out[3], "stages": out[4]}


def q4k_prefill(q: torch.Tensor, a_bf16: torch.Tensor, m_tokens: int, n_rows: int, n_superblocks: int,
                c: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None, form: int = 0,
                independent: bool = False) -> torch.Tensor:
    """C[m, n] = sum_k A[m, k] * bf16(W[n, k]) on the tensor cores (tcgen05); A is a bf16 tensor of
    shape (m_tokens, n_superblocks * 256), the result fp32 of shape (m_tokens, n_rows).  `form`:
    0 = the library's choice, 1 = one CTA per tile, 2 = a CTA pair per 256 rows.  `independent`: q and a
    are not written and c not touched by the launch directly before (lets the call overlap it)."""
    qp = _chk(q, torch.uint8, "q", n_rows * n_superblocks * Q4K_SB_BYTES)
    ap = _chk(a_bf16, torch.bfloat16, "a", m_tokens * n_superblocks * Q4K_SB_ELEMS)
    if c is None:
        c = torch.empty((m_tokens, n_rows), dtype=torch.float32, device=q.device)
    cp = _chk(c, torch.float32, "c", m_tokens * n_rows)
    with torch.cuda.device(q.device):
        rc = _ffi.lib().axc_cuda_q4k_prefill_form(qp, ap, cp, m_tokens, n_rows, n_superblocks, _stream_ptr(),
                                                  status.data_ptr() if status is not None else None, int(form),
                                                  1 if independent else 0)
    _raise_for(rc)
    return c
