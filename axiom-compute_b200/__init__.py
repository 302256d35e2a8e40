"""B200 (sm_100a) backend for AXIOM-Compute's Q4_K_M / Q4_0 dequant-matvec path.

Layers: ``libaxc_cuda.so`` (hand-written CUDA kernels + runtime, C ABI in
``include/axc_cuda.h``) -> ``runtime`` (mirror of axc-runtime's context / handle / dispatch
API) and ``ops`` (device-resident entry points on torch tensors) -> ``hooks`` (the
bench_variant / grid_search timing hooks).  Importing the package loads nothing native; the
first call into the library does, and fails loudly if it has not been built.
"""
from . import errors, runtime, synth  # noqa: F401
from .errors import CopyDirection, DispatchError  # noqa: F401
from .runtime import (  # noqa: F401
    CURRENT_SCHEMA_VERSION, BufferBindingSlot, BufferTy, CudaContext, CudaContextOptions,
    DispatchRequest, KernelCacheKey, KernelHandle, KernelMetadata, ParamBindingPlan,
    ScalarPushConstantSlot, VulkanContext, VulkanContextOptions, captured_icd_path,
    gpu_tests_enabled, load_kernel_metadata, probe_cuda_available, probe_vulkan_available,
    q4_matvec_binding_plan,
)

__all__ = [n for n in dir() if not n.startswith("_")]


def library_path() -> str:
    from . import _ffi
    return _ffi.LIB_PATH
