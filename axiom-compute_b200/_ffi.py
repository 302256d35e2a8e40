"""ctypes binding of ``libaxc_cuda.so`` (the C ABI declared in ``include/axc_cuda.h``).

There is no fallback: if the shared library is missing or cannot be loaded, ``lib()`` raises.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libaxc_cuda.so")

_lock = threading.Lock()
_lib = None

# axc_status (include/axc_cuda.h)
AXC_OK = 0
AXC_ERR_NO_SUPPORTED_DEVICE = 3
AXC_ERR_DEVICE_CREATION_FAILED = 5
AXC_ERR_PIPELINE_CREATION_FAILED = 10
AXC_ERR_BUFFER_ALLOCATION_FAILED = 11
AXC_ERR_QUEUE_SUBMIT_FAILED = 15
AXC_ERR_FENCE_TIMEOUT = 16
AXC_ERR_READBACK_FAILED = 17
AXC_ERR_BINDING_COUNT_MISMATCH = 18
AXC_ERR_PUSH_CONSTANT_SIZE_MISMATCH = 19
AXC_ERR_WORKGROUP_COUNT_EXCEEDS_LIMIT = 20
AXC_ERR_STAGING_COPY_FAILED = 25
AXC_ERR_INVALID_ARGUMENT = 100

AXC_FINISH_OVERLAP_PREVIOUS = 1
AXC_FINISH_LET_NEXT_START = 2
AXC_TY_OTHER, AXC_TY_U8, AXC_TY_F32, AXC_TY_U32 = 0, 1, 2, 3
AXC_ACCESS_READ_ONLY, AXC_ACCESS_READ_WRITE, AXC_ACCESS_WRITE_ONLY = 1, 2, 3


class AxcErrorFields(C.Structure):
    _fields_ = [("binding", C.c_uint32), ("direction", C.c_uint32), ("size", C.c_uint64),
                ("expected", C.c_uint64), ("provided", C.c_uint64), ("timeout_ns", C.c_uint64),
                ("requested", C.c_uint32 * 3), ("max", C.c_uint32 * 3)]


class AxcCtxOpts(C.Structure):
    _fields_ = [("physical_device_index", C.c_int32), ("fence_timeout_ms", C.c_uint64),
                ("pipeline_cache_path", C.c_char_p)]


class AxcBufDesc(C.Structure):
    _fields_ = [("elem_ty", C.c_uint32), ("access", C.c_uint32), ("buffer_position", C.c_uint32),
                ("position", C.c_uint32)]


class AxcDispatchStats(C.Structure):
    _fields_ = [("h2d_ns", C.c_uint64), ("kernel_ns", C.c_uint64), ("d2h_ns", C.c_uint64),
                ("total_device_ns", C.c_uint64), ("rows_effective", C.c_uint32),
                ("blocks_per_row", C.c_uint32)]


class AxcTuning(C.Structure):
    _fields_ = [("ctas_per_sm", C.c_int32), ("tile_rows", C.c_int32), ("stages", C.c_int32),
                ("threads", C.c_int32), ("evict_first", C.c_int32), ("pdl", C.c_int32), ("resident", C.c_int32)]


class AxcGather(C.Structure):
    _fields_ = [("y_peer_bases", C.c_void_p), ("y_offset_bytes", C.c_uint64), ("epoch", C.c_void_p),
                ("world", C.c_uint32), ("rank", C.c_uint32), ("row_offset", C.c_uint32),
                ("parity_stride_bytes", C.c_uint64)]


class AxcGatherSync(C.Structure):
    _fields_ = [("done_peer_bases", C.c_void_p), ("done_local", C.c_void_p), ("arrive_counter", C.c_void_p),
                ("epoch", C.c_void_p), ("world", C.c_uint32), ("rank", C.c_uint32)]


class AxcXSrc(C.Structure):
    _fields_ = [("x", C.c_void_p), ("x2", C.c_void_p), ("x_pairs", C.c_void_p), ("x2_pairs", C.c_void_p),
                ("epoch", C.c_void_p), ("unit_rms", C.c_uint32), ("parity_stride_bytes", C.c_uint64)]


# Every symbol include/axc_cuda.h declares: name -> (restype, argtypes)
_VP = C.c_void_p
_U32P = C.POINTER(C.c_uint32)
_U64P = C.POINTER(C.c_uint64)
_SZP = C.POINTER(C.c_size_t)
_VPP = C.POINTER(C.c_void_p)
_DISPATCH_TAIL = [_U32P, _VPP, _SZP, C.c_uint32, _VPP, _SZP, C.c_uint32, _VP, C.c_size_t]

SYMBOLS = {
    "axc_cuda_probe": (C.c_int, []),
    "axc_cuda_gpu_tests_enabled": (C.c_int, []),
    "axc_cuda_device_count": (C.c_int, []),
    "axc_cuda_ctx_create": (C.c_int, [C.POINTER(AxcCtxOpts), C.POINTER(_VP)]),
    "axc_cuda_ctx_destroy": (None, [_VP]),
    "axc_cuda_ctx_device_name": (C.c_size_t, [_VP, C.c_char_p, C.c_size_t]),
    "axc_cuda_ctx_max_grid": (None, [_VP, _U32P]),
    "axc_cuda_ctx_device_index": (C.c_int, [_VP]),
    "axc_cuda_ctx_sm_count": (C.c_int, [_VP]),
    "axc_cuda_prepare_kernel": (C.c_int, [_VP, C.c_char_p, C.POINTER(AxcBufDesc), C.c_uint32,
                                          C.c_uint32, C.c_uint64, C.c_uint64, C.POINTER(_VP)]),
    "axc_cuda_kernel_retain": (None, [_VP]),
    "axc_cuda_kernel_release": (None, [_VP]),
    "axc_cuda_kernel_buffer_sizes": (C.c_uint32, [_VP, _U64P, C.c_uint32]),
    "axc_cuda_kernel_cache_key": (None, [_VP, _U64P, _U64P, _U32P]),
    "axc_cuda_kernel_set_strict_order": (None, [_VP, C.c_int]),
    "axc_cuda_kernel_set_tuning": (None, [_VP, C.POINTER(AxcTuning)]),
    "axc_cuda_dispatch": (C.c_int, [_VP, _VP] + _DISPATCH_TAIL + [C.POINTER(AxcDispatchStats)]),
    "axc_cuda_dispatch_oneshot": (C.c_int, [_VP, C.c_char_p, C.POINTER(AxcBufDesc), C.c_uint32,
                                            C.c_uint32, C.c_uint64, C.c_uint64] + _DISPATCH_TAIL +
                                  [C.POINTER(AxcDispatchStats)]),
    "axc_cuda_bench_dispatch": (C.c_int, [_VP, _VP] + _DISPATCH_TAIL +
                                [C.c_uint32, _U64P, _U64P, _U64P]),
    "axc_cuda_strerror": (C.c_char_p, [C.c_int]),
    "axc_cuda_last_error_detail": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "axc_cuda_last_error_fields": (None, [C.POINTER(AxcErrorFields)]),
    "axc_cuda_q4k_matvec": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, _VP, _VP,
                                      C.POINTER(AxcTuning)]),
    "axc_cuda_q4_0_matvec": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, _VP, _VP,
                                       C.POINTER(AxcTuning)]),
    "axc_cuda_q4k_matvec_seq": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, _VP]),
    "axc_cuda_q4_0_matvec_seq": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, _VP]),
    "axc_cuda_q4k_dequant": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _VP]),
    "axc_cuda_q4_0_dequant": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _VP]),
    "axc_cuda_q4k_matvec_plan": (C.c_int, [C.c_uint32, C.c_uint32, C.POINTER(AxcTuning), C.c_int32,
                                           C.POINTER(C.c_int32)]),
    "axc_cuda_q4k_matvec_allgather": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, C.POINTER(AxcGather), _VP, _VP,
                                                C.POINTER(AxcTuning)]),
    "axc_cuda_q4k_prefill": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, C.c_uint32, _VP, _VP]),
    "axc_cuda_q4k_prefill_form": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, C.c_uint32, _VP, _VP, C.c_int,
                                            C.c_uint32]),
    "axc_cuda_q4k_matvec_fused": (C.c_int, [_VP, C.POINTER(AxcXSrc), _VP, C.c_uint32, C.c_uint32,
                                            C.POINTER(AxcGather), _VP, _VP, C.POINTER(AxcTuning)]),
    "axc_cuda_q4k_prepared_x_bytes": (C.c_size_t, [C.c_uint32]),
    "axc_cuda_q4k_prepare_x": (C.c_int, [C.POINTER(AxcXSrc), _VP, _VP, C.c_uint32, _VP, _VP, C.c_uint32]),
    "axc_cuda_q4k_matvec_prepared": (C.c_int, [_VP, _VP, C.c_uint32, _VP, C.c_uint32, C.c_uint32,
                                               C.POINTER(AxcGather), _VP, _VP, C.POINTER(AxcTuning)]),
    "axc_cuda_gather_next_epoch": (C.c_int, [_VP, _VP]),
    "axc_cuda_gather_finish": (C.c_int, [_VP, _VP, _VP, C.c_uint32, _VP, _VP, C.c_uint32, C.c_uint64,
                                         C.POINTER(AxcGatherSync)]),
    "axc_cuda_gather_reduce_finish": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, C.c_uint64, _VP, _VP, C.c_uint32,
                                                C.c_uint64]),
    "axc_cuda_q4k_matvec_static": (C.c_int, [_VP, _VP, _VP, C.c_uint32, C.c_uint32, _VP]),
    "axc_cuda_q4k_matvec_static_warmup": (C.c_int, []),
    "axc_cuda_version": (C.c_int, []),
}


def lib() -> C.CDLL:
    """The loaded shared library; raises if it has not been built (no CPU fallback exists)."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: the CUDA extension has not been built "
                    "(run __graft_entry__.build() or axiom-compute_b200/build.py); "
                    "this backend has no CPU fallback")
            L = C.CDLL(LIB_PATH)
            for name, (restype, argtypes) in SYMBOLS.items():
                fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = L
    return _lib


def last_error_detail() -> str:
    L = lib()
    n = L.axc_cuda_last_error_detail(None, 0)
    buf = C.create_string_buffer(n + 1)
    L.axc_cuda_last_error_detail(buf, n + 1)
    return buf.value.decode("utf-8", "replace")


def last_error_fields() -> AxcErrorFields:
    f = AxcErrorFields()
    lib().axc_cuda_last_error_fields(C.byref(f))
    return f
