// axc_cuda_q4k_matvec_static -- a Q4_K_M matvec entry point that allocates nothing.
//
// Who needs it: code that is not allowed to create device memory at the moment it wants a
// matvec.  Examples are a plug-in living inside a host application that handed the whole GPU
// to its own pool at start-up and forbids driver allocations afterwards, and a latency-critical
// decode thread for which cudaMalloc / cudaFree are off limits because they synchronise the
// device and stall every other stream.  Such callers bring q, x and y; the one piece of
// scratch the computation needs besides them -- x quantised into digit words, which the
// allocating path builds per CTA or a caller could keep in a buffer of its own -- lives here
// in a fixed array inside the library image.
//
// Cost and limits: the array occupies 139 520 bytes on every GPU that loads this library, for
// the life of the process, whether or not the entry point is ever called.  It bounds the row
// length: at most AXC_STATIC_MAX_SUPERBLOCKS (128) superblocks per row, K <= 32768.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/axc_cuda.h"
#include "axc_kernels.h"

namespace {

constexpr uint32_t kMaxSuperblocks = 128;                        // K = 32768
constexpr uint32_t kMaxPositions = kMaxSuperblocks * 4;          // 64-column positions
constexpr size_t kScratchBytes = (size_t)17 * kMaxPositions * 16 + 256;  // digits + metadata + slack

// The scratch.  In host code this name is only a handle for the runtime's symbol table, not a
// device address: it must never be passed to a kernel as is.  device_scratch() asks the
// runtime for the address on the current device.
static __device__ __align__(256) unsigned char g_static_x_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};

cudaError_t device_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_x_scratch);  // per device: each GPU has its own copy
        if (e != cudaSuccess) return e;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int axc_cuda_q4k_matvec_static_warmup(void) {
    void* scratch = nullptr;
    cudaError_t e = device_scratch(&scratch);   // loads the module that holds the array on this device
    if (e == cudaSuccess) e = axc::preload_q4k_prepared_path();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return AXC_ERR_DEVICE_CREATION_FAILED;
    }
    return AXC_OK;
}

extern "C" int axc_cuda_q4k_matvec_static(const void* q, const float* x, float* y, uint32_t rows,
                                          uint32_t n_superblocks, void* stream) {
    if (rows == 0) return AXC_OK;
    if (!q || !x || !y) return AXC_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)q | (uintptr_t)x | (uintptr_t)y) & 15u) return AXC_ERR_INVALID_ARGUMENT;
    if (n_superblocks == 0 || n_superblocks > kMaxSuperblocks)
        return AXC_ERR_BUFFER_ALLOCATION_FAILED;  // the fixed scratch cannot hold this row length
    void* scratch = nullptr;
    if (device_scratch(&scratch) != cudaSuccess) {
        cudaGetLastError();
        return AXC_ERR_DEVICE_CREATION_FAILED;
    }
    cudaStream_t st = (cudaStream_t)stream;
    // Every word of the scratch this call reads is rewritten by the quantiser first, so nothing
    // left over from an earlier call (or from another row length) can leak into the result.
    cudaError_t e = axc::launch_q4_quantize_x(x, scratch, n_superblocks * 4, st);
    if (e == cudaSuccess) {
        axc::MatvecTuning tune;
        tune.x_prepared = scratch;
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        e = axc::launch_q4k_matvec((const uint8_t*)q, x, y, rows, n_superblocks, nullptr, st, tune, sms, nullptr);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return AXC_ERR_QUEUE_SUBMIT_FAILED;
    }
    return AXC_OK;
}
