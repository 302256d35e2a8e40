"""Host-side mirror of ``axc_runtime``'s public surface over the CUDA C ABI.

Same names, argument meaning and error behaviour as the reference crate
(crates/axc-runtime/src/lib.rs:57-62): ``VulkanContext`` / ``VulkanContextOptions`` (here also
exported under their honest names ``CudaContext`` / ``CudaContextOptions``), ``KernelHandle``,
``KernelCacheKey``, ``DispatchRequest``, ``DispatchError``, ``KernelMetadata``,
``load_kernel_metadata``, ``probe_vulkan_available``, ``gpu_tests_enabled``,
``captured_icd_path``; plus the binding-plan types of axc-hir that cross the boundary
(crates/axc-hir/src/param.rs:66-126).  Every method forwards to ``libaxc_cuda.so``; nothing is
computed on the host.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

from . import _ffi
from . import errors as E

CURRENT_SCHEMA_VERSION = 1  # crates/axc-runtime/src/metadata.rs:35
DEFAULT_FENCE_TIMEOUT_MS = 10_000  # crates/axc-runtime/src/dispatch.rs:26
MAX_PUSH_CONSTANT_BYTES = 128  # crates/axc-hir/src/param.rs:111

_ELEM_CODE = {"U8": _ffi.AXC_TY_U8, "F32": _ffi.AXC_TY_F32, "U32": _ffi.AXC_TY_U32}
_ACCESS_CODE = {"ReadOnly": _ffi.AXC_ACCESS_READ_ONLY, "ReadWrite": _ffi.AXC_ACCESS_READ_WRITE,
                "WriteOnly": _ffi.AXC_ACCESS_WRITE_ONLY}


# ---- binding plan (axc-hir) -------------------------------------------------------------------

@dataclass(frozen=True)
class BufferTy:
    """crates/axc-hir/src/buffer.rs:41-49; ``elem`` / ``access`` use serde's variant names."""
    elem: str
    access: str


@dataclass(frozen=True)
class BufferBindingSlot:
    """crates/axc-hir/src/param.rs:66-78 (``span`` is not serialised and is omitted)."""
    name: str
    ty: BufferTy
    position: int
    buffer_position: int


@dataclass(frozen=True)
class ScalarPushConstantSlot:
    """crates/axc-hir/src/param.rs:92-107."""
    name: str
    ty: str
    offset: int
    member_index: int
    position: int


@dataclass(frozen=True)
class ParamBindingPlan:
    """crates/axc-hir/src/param.rs:119-126."""
    buffers: tuple
    scalars: tuple
    push_constant_total_bytes: int

    def to_json_obj(self) -> dict:
        return {
            "buffers": [{"name": b.name, "ty": {"elem": b.ty.elem, "access": b.ty.access},
                         "position": b.position, "buffer_position": b.buffer_position}
                        for b in self.buffers],
            "scalars": [{"name": s.name, "ty": s.ty, "offset": s.offset,
                         "member_index": s.member_index, "position": s.position}
                        for s in self.scalars],
            "push_constant_total_bytes": self.push_constant_total_bytes,
        }

    @staticmethod
    def from_json_obj(o: dict) -> "ParamBindingPlan":
        return ParamBindingPlan(
            buffers=tuple(BufferBindingSlot(b["name"], BufferTy(b["ty"]["elem"], b["ty"]["access"]),
                                            int(b["position"]), int(b["buffer_position"]))
                          for b in o["buffers"]),
            scalars=tuple(ScalarPushConstantSlot(s["name"], s["ty"], int(s["offset"]),
                                                 int(s["member_index"]), int(s["position"]))
                          for s in o["scalars"]),
            push_constant_total_bytes=int(o["push_constant_total_bytes"]))

    def hash64(self) -> int:
        """64-bit digest of the serialised plan (the reference uses xxh3_64 of the same JSON;
        only equality of keys matters, kernel_handle.rs:216-246)."""
        blob = json.dumps(self.to_json_obj(), separators=(",", ":")).encode()
        return int.from_bytes(hashlib.blake2b(blob, digest_size=8).digest(), "little")


def q4_matvec_binding_plan(kernel: str = "q4km_dequant_matvec") -> ParamBindingPlan:
    """The plan ``compute_binding_plan`` yields for both Q4 kernels
    (examples/q4km_dequant_matvec.axc:7-12, examples/q4_0_dequant_matvec.axc:7-12): q, x, y at
    bindings 0..2 and one u32 push constant at offset 0."""
    scalar = "n_superblocks" if kernel == "q4km_dequant_matvec" else "n_blocks"
    return ParamBindingPlan(
        buffers=(BufferBindingSlot("q", BufferTy("U8", "ReadOnly"), 0, 0),
                 BufferBindingSlot("x", BufferTy("F32", "ReadOnly"), 1, 1),
                 BufferBindingSlot("y", BufferTy("F32", "ReadWrite"), 2, 2)),
        scalars=(ScalarPushConstantSlot(scalar, "U32", 0, 0, 3),),
        push_constant_total_bytes=4)


# ---- metadata sidecar (crates/axc-runtime/src/metadata.rs) -------------------------------------

@dataclass
class KernelMetadata:
    kernel_name: str
    workgroup_size: list
    binding_plan: ParamBindingPlan
    entry_point: str
    schema_version: int = CURRENT_SCHEMA_VERSION
    push_constant_total_bytes: int = field(default=-1)

    def __post_init__(self):
        if self.push_constant_total_bytes < 0:
            self.push_constant_total_bytes = self.binding_plan.push_constant_total_bytes

    @staticmethod
    def new(kernel_name: str, workgroup_size, binding_plan: ParamBindingPlan,
            entry_point: str) -> "KernelMetadata":
        return KernelMetadata(kernel_name, list(workgroup_size), binding_plan, entry_point)

    def save(self, path) -> None:
        obj = {"schema_version": self.schema_version, "kernel_name": self.kernel_name,
               "workgroup_size": list(self.workgroup_size),
               "binding_plan": self.binding_plan.to_json_obj(),
               "push_constant_total_bytes": self.push_constant_total_bytes,
               "entry_point": self.entry_point}
        try:
            with open(path, "w") as f:
                json.dump(obj, f, indent=2)
        except OSError as e:
            raise E.MetadataIoError(f"metadata I/O error: {e}") from e


def load_kernel_metadata(path) -> KernelMetadata:
    """metadata.rs:107-122: read, parse, then check the schema version."""
    try:
        with open(path) as f:
            text = f.read()
    except OSError as e:
        raise E.MetadataIoError(f"metadata I/O error: {e}") from e
    try:
        o = json.loads(text)
        meta = KernelMetadata(
            kernel_name=o["kernel_name"], workgroup_size=[int(v) for v in o["workgroup_size"]],
            binding_plan=ParamBindingPlan.from_json_obj(o["binding_plan"]),
            entry_point=o["entry_point"], schema_version=int(o["schema_version"]),
            push_constant_total_bytes=int(o["push_constant_total_bytes"]))
        if len(meta.workgroup_size) != 3:
            raise ValueError("workgroup_size must have 3 entries")
    except (ValueError, KeyError, TypeError) as e:
        raise E.MetadataParseError(f"metadata parse error: {e}") from e
    if meta.schema_version != CURRENT_SCHEMA_VERSION:
        raise E.MetadataSchemaMismatch(
            f"metadata schema v{meta.schema_version} is not supported (runtime supports "
            f"v{CURRENT_SCHEMA_VERSION})", got=meta.schema_version, supported=CURRENT_SCHEMA_VERSION)
    return meta


# ---- availability (crates/axc-runtime/src/icd.rs) ----------------------------------------------

def probe_cuda_available() -> bool:
    return bool(_ffi.lib().axc_cuda_probe())


probe_vulkan_available = probe_cuda_available  # name the reference's callers use


def gpu_tests_enabled() -> bool:
    return os.environ.get("AXC_ENABLE_GPU_TESTS", "") == "1"


def captured_icd_path() -> str:
    """No installable client driver exists for CUDA; the reference's field stays empty."""
    return ""


# ---- errors ------------------------------------------------------------------------------------

def _raise_for(status: int) -> None:
    if status == _ffi.AXC_OK:
        return
    msg = _ffi.last_error_detail()
    f = _ffi.last_error_fields()
    reason = msg.split(": ", 1)[-1] if ": " in msg else msg
    if status == _ffi.AXC_ERR_NO_SUPPORTED_DEVICE:
        raise E.NoSupportedDevice(msg)
    if status == _ffi.AXC_ERR_DEVICE_CREATION_FAILED:
        raise E.DeviceCreationFailed(msg)
    if status == _ffi.AXC_ERR_PIPELINE_CREATION_FAILED:
        raise E.PipelineCreationFailed(msg)
    if status == _ffi.AXC_ERR_BUFFER_ALLOCATION_FAILED:
        raise E.BufferAllocationFailed(msg, binding=f.binding, size=f.size, reason=reason)
    if status == _ffi.AXC_ERR_QUEUE_SUBMIT_FAILED:
        raise E.QueueSubmitFailed(msg)
    if status == _ffi.AXC_ERR_FENCE_TIMEOUT:
        raise E.FenceTimeout(msg, timeout_ns=f.timeout_ns)
    if status == _ffi.AXC_ERR_READBACK_FAILED:
        raise E.ReadbackFailed(msg, binding=f.binding, reason=reason)
    if status == _ffi.AXC_ERR_BINDING_COUNT_MISMATCH:
        raise E.BindingCountMismatch(msg, expected=f.expected, provided=f.provided)
    if status == _ffi.AXC_ERR_PUSH_CONSTANT_SIZE_MISMATCH:
        raise E.PushConstantSizeMismatch(msg, expected=f.expected, provided=f.provided)
    if status == _ffi.AXC_ERR_WORKGROUP_COUNT_EXCEEDS_LIMIT:
        raise E.WorkgroupCountExceedsDeviceLimit(msg, requested=list(f.requested), max=list(f.max))
    if status == _ffi.AXC_ERR_STAGING_COPY_FAILED:
        raise E.StagingCopyFailed(msg, binding=f.binding, direction=E.CopyDirection(f.direction),
                                  reason=reason)
    raise E.InvalidArgument(msg or f"status {status}")


# ---- context / handle / dispatch ---------------------------------------------------------------

@dataclass
class CudaContextOptions:
    """crates/axc-runtime/src/context.rs:76-109."""
    pipeline_cache_path: Optional[str] = None   # accepted and ignored (kernels are AOT)
    physical_device_index: Optional[int] = None
    fence_timeout_ms: Optional[int] = None

    @staticmethod
    def from_env() -> "CudaContextOptions":
        def _int(name):
            try:
                return int(os.environ[name])
            except (KeyError, ValueError):
                return None
        return CudaContextOptions(None, _int("AXC_PHYSICAL_DEVICE_INDEX"),
                                  _int("AXC_FENCE_TIMEOUT_MS"))


@dataclass(frozen=True, order=True)
class KernelCacheKey:
    """crates/axc-runtime/src/kernel_handle.rs:44-51."""
    spirv_hash: int
    binding_plan_hash: int
    push_constant_bytes: int


@dataclass
class DispatchStats:
    h2d_ns: int
    kernel_ns: int
    d2h_ns: int
    total_device_ns: int
    rows_effective: int
    blocks_per_row: int


class KernelHandle:
    """crates/axc-runtime/src/kernel_handle.rs:123-151.  ``clone()`` shares the inner object."""

    def __init__(self, ptr: int, spirv_words: int):
        self._ptr = ptr
        self._spirv_words = spirv_words

    def clone(self) -> "KernelHandle":
        _ffi.lib().axc_cuda_kernel_retain(self._ptr)
        return KernelHandle(self._ptr, self._spirv_words)

    def spirv_word_count(self) -> int:
        return self._spirv_words

    def cache_key(self) -> KernelCacheKey:
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint32()
        _ffi.lib().axc_cuda_kernel_cache_key(self._ptr, C.byref(a), C.byref(b), C.byref(c))
        return KernelCacheKey(a.value, b.value, c.value)

    def buffer_sizes(self) -> list:
        out = (C.c_uint64 * 16)()
        n = _ffi.lib().axc_cuda_kernel_buffer_sizes(self._ptr, out, 16)
        return [int(out[i]) for i in range(min(n, 16))]

    def inner_id(self) -> int:
        """Address of the shared inner object (``Arc::ptr_eq`` in the reference's tests)."""
        return int(self._ptr)

    def set_strict_order(self, strict: bool) -> None:
        """Run the reference-order kernel (bit-identical y, slow) instead of the fast one."""
        _ffi.lib().axc_cuda_kernel_set_strict_order(self._ptr, 1 if strict else 0)

    def set_tuning(self, tuning) -> None:
        """Launch tunables (an ``_ffi.AxcTuning`` or None = defaults) for later dispatches."""
        _ffi.lib().axc_cuda_kernel_set_tuning(self._ptr, C.byref(tuning) if tuning is not None else None)

    def drop(self) -> None:
        if self._ptr:
            _ffi.lib().axc_cuda_kernel_release(self._ptr)
            self._ptr = 0

    def __del__(self):
        try:
            self.drop()
        except Exception:
            pass


@dataclass
class DispatchRequest:
    """crates/axc-runtime/src/dispatch.rs:33-50."""
    spirv: Sequence[int]
    binding_plan: ParamBindingPlan
    workgroups: Sequence[int]
    inputs: Sequence[bytes]
    output_sizes: Sequence[int]
    push_constants: bytes
    entry_point: str


def _spirv_hash(spirv) -> int:
    import array
    blob = array.array("I", [int(w) & 0xFFFFFFFF for w in spirv]).tobytes()
    return int.from_bytes(hashlib.blake2b(blob, digest_size=8).digest(), "little")


def _buf_descs(plan: ParamBindingPlan):
    n = len(plan.buffers)
    arr = (_ffi.AxcBufDesc * max(n, 1))()
    for i, b in enumerate(plan.buffers):
        arr[i].elem_ty = _ELEM_CODE.get(b.ty.elem, _ffi.AXC_TY_OTHER)
        arr[i].access = _ACCESS_CODE.get(b.ty.access, 0)
        arr[i].buffer_position = b.buffer_position
        arr[i].position = b.position
    return arr, n


def _as_buffer(b):
    """(address, length, keepalive) of a bytes-like input; zero-copy for bytes, bytearray and
    writable contiguous buffers (numpy arrays)."""
    if b is None:
        return None, 0, None
    if isinstance(b, bytes):
        if not b:
            return None, 0, None
        return C.cast(C.c_char_p(b), C.c_void_p).value, len(b), b
    mv = memoryview(b)
    if mv.nbytes == 0:
        return None, 0, None
    if mv.readonly or not mv.c_contiguous:
        return _as_buffer(mv.tobytes())
    flat = mv.cast("B")
    holder = (C.c_char * flat.nbytes).from_buffer(flat)
    return C.addressof(holder), flat.nbytes, (holder, flat, mv)


class CudaContext:
    """crates/axc-runtime/src/context.rs:160-547 -- the reference calls it ``VulkanContext``."""

    def __init__(self, options: Optional[CudaContextOptions] = None):
        opts = options if options is not None else CudaContextOptions.from_env()
        self._options = opts
        c_opts = _ffi.AxcCtxOpts(
            -1 if opts.physical_device_index is None else int(opts.physical_device_index),
            0 if opts.fence_timeout_ms is None else int(opts.fence_timeout_ms),
            None if opts.pipeline_cache_path is None else str(opts.pipeline_cache_path).encode())
        ptr = C.c_void_p()
        _raise_for(_ffi.lib().axc_cuda_ctx_create(C.byref(c_opts), C.byref(ptr)))
        self._ptr = ptr.value

    @staticmethod
    def new() -> "CudaContext":
        return CudaContext(CudaContextOptions.from_env())

    @staticmethod
    def new_with_options(options: CudaContextOptions) -> "CudaContext":
        return CudaContext(options)

    def physical_device_name(self) -> str:
        L = _ffi.lib()
        n = L.axc_cuda_ctx_device_name(self._ptr, None, 0)
        buf = C.create_string_buffer(n + 1)
        L.axc_cuda_ctx_device_name(self._ptr, buf, n + 1)
        return buf.value.decode()

    def max_compute_work_group_count(self) -> list:
        out = (C.c_uint32 * 3)()
        _ffi.lib().axc_cuda_ctx_max_grid(self._ptr, out)
        return [int(v) for v in out]

    def device_index(self) -> int:
        return int(_ffi.lib().axc_cuda_ctx_device_index(self._ptr))

    def sm_count(self) -> int:
        return int(_ffi.lib().axc_cuda_ctx_sm_count(self._ptr))

    def prepare_kernel(self, spirv, binding_plan: ParamBindingPlan, push_constant_total_bytes: int,
                       entry_point: str, *, spirv_hash: Optional[int] = None) -> KernelHandle:
        """context.rs:392-486.  ``spirv`` only feeds the cache key (the kernels are compiled
        ahead of time and selected by ``entry_point``)."""
        descs, n = _buf_descs(binding_plan)
        h = _spirv_hash(spirv) if spirv_hash is None else int(spirv_hash)
        out = C.c_void_p()
        _raise_for(_ffi.lib().axc_cuda_prepare_kernel(
            self._ptr, entry_point.encode(), descs, n, int(push_constant_total_bytes),
            h & 0xFFFFFFFFFFFFFFFF, binding_plan.hash64(), C.byref(out)))
        return KernelHandle(out.value, len(spirv))

    @staticmethod
    def _marshal(inputs, output_sizes, push_constants):
        n_in, n_out = len(inputs), len(output_sizes)
        in_ptrs = (C.c_void_p * max(n_in, 1))()
        in_lens = (C.c_size_t * max(n_in, 1))()
        keep = []
        for i, b in enumerate(inputs):
            addr, ln, holder = _as_buffer(b)
            in_ptrs[i], in_lens[i] = addr, ln
            keep.append(holder)
        out_bufs = [bytearray(int(sz)) for sz in output_sizes]
        out_ptrs = (C.c_void_p * max(n_out, 1))()
        out_lens = (C.c_size_t * max(n_out, 1))()
        for i, ob in enumerate(out_bufs):
            out_lens[i] = len(ob)
            if len(ob):
                h = (C.c_char * len(ob)).from_buffer(ob)
                keep.append(h)
                out_ptrs[i] = C.addressof(h)
        pc = bytes(push_constants)
        pc_buf = C.create_string_buffer(pc, max(len(pc), 1))
        return in_ptrs, in_lens, n_in, out_ptrs, out_lens, n_out, pc_buf, len(pc), out_bufs, keep

    def dispatch_handle(self, handle: KernelHandle, workgroups, inputs, output_sizes,
                        push_constants, *, stats: bool = False):
        """context.rs:498-547.  Returns one ``bytearray`` per binding (empty for size 0); with
        ``stats=True`` returns ``(outputs, DispatchStats)``."""
        (in_ptrs, in_lens, n_in, out_ptrs, out_lens, n_out, pc_buf, pc_len, out_bufs,
         keep) = self._marshal(inputs, output_sizes, push_constants)
        wg = (C.c_uint32 * 3)(*[int(v) for v in workgroups])
        st = _ffi.AxcDispatchStats()
        rc = _ffi.lib().axc_cuda_dispatch(
            self._ptr, handle._ptr, wg, in_ptrs, in_lens, n_in, out_ptrs, out_lens, n_out,
            C.cast(pc_buf, C.c_void_p), pc_len, C.byref(st) if stats else None)
        del keep
        _raise_for(rc)
        if stats:
            return out_bufs, DispatchStats(st.h2d_ns, st.kernel_ns, st.d2h_ns, st.total_device_ns,
                                           st.rows_effective, st.blocks_per_row)
        return out_bufs

    def bind(self, handle: KernelHandle, workgroups, inputs, output_sizes, push_constants) -> "BoundDispatch":
        """``dispatch_handle`` with its arguments marshalled once: ``run()`` repeats the same
        dispatch (same host input buffers, read again on every run; outputs land in the same
        reusable bytearrays).  A Rust caller pays nothing for marshalling; this gives a Python
        caller the same per-call cost (one foreign call)."""
        return BoundDispatch(self, handle, workgroups, inputs, output_sizes, push_constants)

    def dispatch(self, req: DispatchRequest):
        """dispatch.rs:109-132: validate, prepare, dispatch once, drop the handle."""
        (in_ptrs, in_lens, n_in, out_ptrs, out_lens, n_out, pc_buf, pc_len, out_bufs,
         keep) = self._marshal(req.inputs, req.output_sizes, req.push_constants)
        descs, n = _buf_descs(req.binding_plan)
        wg = (C.c_uint32 * 3)(*[int(v) for v in req.workgroups])
        rc = _ffi.lib().axc_cuda_dispatch_oneshot(
            self._ptr, req.entry_point.encode(), descs, n,
            int(req.binding_plan.push_constant_total_bytes), _spirv_hash(req.spirv),
            req.binding_plan.hash64(), wg, in_ptrs, in_lens, n_in, out_ptrs, out_lens, n_out,
            C.cast(pc_buf, C.c_void_p), pc_len, None)
        del keep
        _raise_for(rc)
        return out_bufs

    def bench_dispatch(self, handle: KernelHandle, workgroups, inputs, output_sizes,
                       push_constants, sample_count: int):
        """The timing loop of bench_variant (bench_variant.rs:284-301) run natively:
        returns (median_ns, samples_ns, device_kernel_ns, last outputs)."""
        (in_ptrs, in_lens, n_in, out_ptrs, out_lens, n_out, pc_buf, pc_len, out_bufs,
         keep) = self._marshal(inputs, output_sizes, push_constants)
        wg = (C.c_uint32 * 3)(*[int(v) for v in workgroups])
        n = max(int(sample_count), 0)
        samples = (C.c_uint64 * max(n, 1))()
        dev = (C.c_uint64 * max(n, 1))()
        median = C.c_uint64()
        rc = _ffi.lib().axc_cuda_bench_dispatch(
            self._ptr, handle._ptr, wg, in_ptrs, in_lens, n_in, out_ptrs, out_lens, n_out,
            C.cast(pc_buf, C.c_void_p), pc_len, n, samples, C.byref(median), dev)
        del keep
        _raise_for(rc)
        return int(median.value), [int(samples[i]) for i in range(n)], \
            [int(dev[i]) for i in range(n)], out_bufs

    def drop(self) -> None:
        if getattr(self, "_ptr", None):
            _ffi.lib().axc_cuda_ctx_destroy(self._ptr)
            self._ptr = None

    def __del__(self):
        try:
            self.drop()
        except Exception:
            pass


class BoundDispatch:
    """One dispatch whose C arguments are built once (see ``CudaContext.bind``)."""

    def __init__(self, ctx: CudaContext, handle: KernelHandle, workgroups, inputs, output_sizes, push_constants):
        self._ctx, self._handle = ctx, handle
        (self._in_ptrs, self._in_lens, self._n_in, self._out_ptrs, self._out_lens, self._n_out, self._pc_buf,
         self._pc_len, self.outputs, self._keep) = CudaContext._marshal(inputs, output_sizes, push_constants)
        self._wg = (C.c_uint32 * 3)(*[int(v) for v in workgroups])
        self._pc_ptr = C.cast(self._pc_buf, C.c_void_p)
        self._fn = _ffi.lib().axc_cuda_dispatch

    def run(self):
        """Dispatch once; returns the (reused) output buffers, one per binding."""
        rc = self._fn(self._ctx._ptr, self._handle._ptr, self._wg, self._in_ptrs, self._in_lens, self._n_in,
                      self._out_ptrs, self._out_lens, self._n_out, self._pc_ptr, self._pc_len, None)
        if rc:
            _raise_for(rc)
        return self.outputs


VulkanContext = CudaContext
VulkanContextOptions = CudaContextOptions
