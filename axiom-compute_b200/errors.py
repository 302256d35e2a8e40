"""``DispatchError`` -- the typed error set of axc-runtime (crates/axc-runtime/src/error.rs:27-195).

One exception class per Rust variant, same names and fields, same ``Display`` text.  The CUDA
backend raises the subset listed in ``include/axc_cuda.h``; the others exist so that code
written against the reference's enum keeps its shape (the Vulkan-only ones are never raised).
"""
from __future__ import annotations

from enum import Enum


class CopyDirection(Enum):
    """crates/axc-runtime/src/error.rs:14-20."""
    HostToDevice = 0
    DeviceToHost = 1


class DispatchError(Exception):
    """Base of all variants; ``variant`` is the Rust variant name."""
    variant = "DispatchError"

    def __init__(self, message: str, **fields):
        super().__init__(message)
        self.message = message
        for k, v in fields.items():
            setattr(self, k, v)
        self.fields = fields


def _variant(name: str, doc: str):
    return type(name, (DispatchError,), {"variant": name, "__doc__": doc})


VulkanEntryFailed = _variant("VulkanEntryFailed", "Vulkan only; never raised by the CUDA backend.")
NoVulkanInstance = _variant("NoVulkanInstance", "Vulkan only; never raised by the CUDA backend.")
NoSupportedDevice = _variant("NoSupportedDevice", "No compute-capability-10.x CUDA device.")
NoComputeQueue = _variant("NoComputeQueue", "Vulkan only; never raised by the CUDA backend.")
DeviceCreationFailed = _variant("DeviceCreationFailed", "Device / stream bring-up failed.")
ShaderModuleCreationFailed = _variant("ShaderModuleCreationFailed", "Vulkan only.")
DescriptorSetLayoutFailed = _variant("DescriptorSetLayoutFailed", "Vulkan only.")
DescriptorPoolFailed = _variant("DescriptorPoolFailed", "Vulkan only.")
PipelineLayoutFailed = _variant("PipelineLayoutFailed", "Vulkan only.")
PipelineCreationFailed = _variant("PipelineCreationFailed", "Unsupported kernel / plan shape.")
BufferAllocationFailed = _variant("BufferAllocationFailed", "fields: binding, size, reason")
MemoryMapFailed = _variant("MemoryMapFailed", "Vulkan only.")
NoCompatibleMemoryType = _variant("NoCompatibleMemoryType", "Vulkan only.")
CommandBufferRecordFailed = _variant("CommandBufferRecordFailed", "Vulkan only.")
QueueSubmitFailed = _variant("QueueSubmitFailed", "Kernel launch or stream operation failed.")
FenceTimeout = _variant("FenceTimeout", "fields: timeout_ns")
ReadbackFailed = _variant("ReadbackFailed", "fields: binding, reason")
BindingCountMismatch = _variant("BindingCountMismatch", "fields: expected, provided")
PushConstantSizeMismatch = _variant("PushConstantSizeMismatch", "fields: expected, provided")
WorkgroupCountExceedsDeviceLimit = _variant("WorkgroupCountExceedsDeviceLimit",
                                            "fields: requested, max")
MetadataIoError = _variant("MetadataIoError", "Sidecar file I/O failed.")
MetadataParseError = _variant("MetadataParseError", "Sidecar JSON malformed.")
MetadataSchemaMismatch = _variant("MetadataSchemaMismatch", "fields: got, supported")
PipelineCacheLoadFailed = _variant("PipelineCacheLoadFailed", "Vulkan only.")
StagingCopyFailed = _variant("StagingCopyFailed", "fields: binding, direction, reason")


class InvalidArgument(DispatchError):
    """A null / malformed argument at the C boundary; has no Rust counterpart."""
    variant = "InvalidArgument"


ALL_VARIANTS = [
    VulkanEntryFailed, NoVulkanInstance, NoSupportedDevice, NoComputeQueue, DeviceCreationFailed,
    ShaderModuleCreationFailed, DescriptorSetLayoutFailed, DescriptorPoolFailed,
    PipelineLayoutFailed, PipelineCreationFailed, BufferAllocationFailed, MemoryMapFailed,
    NoCompatibleMemoryType, CommandBufferRecordFailed, QueueSubmitFailed, FenceTimeout,
    ReadbackFailed, BindingCountMismatch, PushConstantSizeMismatch,
    WorkgroupCountExceedsDeviceLimit, MetadataIoError, MetadataParseError, MetadataSchemaMismatch,
    PipelineCacheLoadFailed, StagingCopyFailed,
]  # 25, the count error.rs asserts in at_801
