// libaxc_cuda.so -- runtime layer: the CUDA counterpart of axc-runtime's VulkanContext /
// KernelHandle / dispatch_handle (crates/axc-runtime/src/{context,kernel_handle,dispatch,
// buffers,error}.rs), exported with a C ABI (include/axc_cuda.h).
//
// Device buffers are cudaMalloc'ed per binding slot and grow to the next power of two; each
// slot has a pinned host staging twin; copies and the kernel go on the context's stream; the
// host waits on a CUDA event with a bounded poll (the "fence").
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

#include "../../include/axc_cuda.h"
#include "axc_kernels.h"

namespace {

constexpr uint64_t kDefaultFenceTimeoutMs = 10000;  // dispatch.rs:26
constexpr uint32_t kMaxGrid[3] = {2147483647u, 65535u, 65535u};

thread_local std::string g_detail;
thread_local axc_error_fields g_fields;

int fail(int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_detail = buf;
    return status;
}

void clear_error() {
    g_detail.clear();
    std::memset(&g_fields, 0, sizeof g_fields);
}

uint64_t round_up_pow2(uint64_t size) {  // buffers.rs:195-204
    if (size <= 4) return 4;
    if (size > (1ull << 62)) return UINT64_MAX;
    uint64_t p = 1;
    while (p < size) p <<= 1;
    return p;
}

enum class KernelKind { Q4K, Q4_0 };

struct Slot {
    void* dev = nullptr;
    void* staging = nullptr;  // pinned
    uint64_t size = 0;        // allocated bytes (power of two)
    uint64_t valid = 0;       // bytes of the most recent upload
    bool mapped = false;      // dev is the device view of the pinned host buffer (no copies)
    void* staging_dev = nullptr;  // device view of `staging` when it was allocated mapped (small inputs)
    bool dev_stale = false;   // staging holds a newer upload than dev (the copy was skipped)
};

// Output bindings up to this size live in mapped pinned host memory: the kernel's stores go
// straight to the host over PCIe and the device-to-host copy (a second DMA after the kernel,
// several microseconds of latency for a few tens of KB) disappears.  Larger outputs keep a
// device buffer and one bulk copy.
constexpr uint64_t kMappedOutputMax = 1u << 20;
// Activation vectors up to this size keep their staging buffer mapped as well: on the fast path a
// small kernel reads x from it over PCIe and quantises it once for every CTA of the matvec, so no
// copy-engine transfer (and no hand-over between the copy and compute engines) precedes the launch.
constexpr uint64_t kMappedInputMax = 1u << 18;

struct CacheKey {
    uint64_t spirv_hash, plan_hash;
    uint32_t pc_bytes;
    bool operator<(const CacheKey& o) const {
        return std::tie(spirv_hash, plan_hash, pc_bytes) <
               std::tie(o.spirv_hash, o.plan_hash, o.pc_bytes);
    }
};

struct CacheTable {
    std::mutex mu;
    std::map<CacheKey, axc_kernel*> live;
};

}  // namespace

struct axc_kernel {
    std::atomic<int> refs{1};
    std::shared_ptr<CacheTable> table;
    CacheKey key{};
    KernelKind kind = KernelKind::Q4K;
    int device = 0;
    int sm_count = 148;
    uint32_t n_bufs = 0;
    uint32_t pc_total = 0;
    std::atomic<int> strict{0};
    axc::MatvecTuning tune;  // guarded by mu
    std::mutex mu;  // serialises dispatches on this handle (context.rs:494-519)
    std::vector<Slot> slots;
    uint32_t* status_dev = nullptr;
    uint32_t* status_host = nullptr;  // pinned, mapped: [0] kernel error bits, [4] completion sequence number
    void* fast_scratch = nullptr;     // device: quantised x image, then the CTA counter of the completion signal
    size_t fast_image_bytes = 0;
    uint32_t fast_seq = 0;
    cudaEvent_t ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
};

struct axc_ctx {
    int device = 0;
    int sm_count = 148;
    std::string name;
    uint64_t fence_timeout_ms = 0;  // 0 = read AXC_FENCE_TIMEOUT_MS per dispatch
    cudaStream_t stream = nullptr;
    std::shared_ptr<CacheTable> table;
};

namespace {

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

void free_slot(Slot& s) {
    if (s.dev && !s.mapped) cudaFree(s.dev);
    if (s.staging) cudaFreeHost(s.staging);
    s = Slot{};
}

void destroy_kernel(axc_kernel* k) {
    DeviceGuard g(k->device);
    for (auto& s : k->slots) free_slot(s);
    if (k->status_host) cudaFreeHost(k->status_host);   // status_dev is its device view
    if (k->fast_scratch) cudaFree(k->fast_scratch);
    for (auto& e : k->ev)
        if (e) cudaEventDestroy(e);
    delete k;
}

uint64_t fence_timeout_ms_for(const axc_ctx* ctx) {
    if (ctx->fence_timeout_ms) return ctx->fence_timeout_ms;
    if (const char* s = std::getenv("AXC_FENCE_TIMEOUT_MS")) {
        char* end = nullptr;
        unsigned long long v = std::strtoull(s, &end, 10);
        if (end && end != s && *end == '\0') return (uint64_t)v;
    }
    return kDefaultFenceTimeoutMs;
}

// Bounded wait on an event: the fence of kernel_handle.rs:658-687.
bool wait_event(cudaEvent_t ev, uint64_t timeout_ms, cudaError_t* err) {
    using clock = std::chrono::steady_clock;
    const auto t0 = clock::now();
    const auto limit = std::chrono::milliseconds(timeout_ms);
    uint32_t spins = 0;
    for (;;) {
        const cudaError_t q = cudaEventQuery(ev);
        if (q == cudaSuccess) return true;
        if (q != cudaErrorNotReady) {
            *err = q;
            return false;
        }
        if ((++spins & 63u) == 0) {
            const auto el = clock::now() - t0;
            if (el > limit) {
                *err = cudaErrorNotReady;
                return false;
            }
            if (el > std::chrono::milliseconds(2)) std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
    }
}

int ensure_slots(axc_kernel* k, const size_t* input_lens, const size_t* output_sizes, const bool* writable,
                 int mapped_input = -1) {
    if (k->slots.size() < k->n_bufs) k->slots.resize(k->n_bufs);
    for (uint32_t i = 0; i < k->n_bufs; ++i) {
        const uint64_t need = std::max<uint64_t>(std::max<uint64_t>(input_lens[i], output_sizes[i]), 4);
        Slot& s = k->slots[i];
        if (s.dev && s.size >= need) continue;
        const uint64_t new_size = round_up_pow2(need);
        g_fields.binding = i;
        g_fields.size = need;
        if (new_size == UINT64_MAX)
            return fail(AXC_ERR_BUFFER_ALLOCATION_FAILED, "buffer #%u allocation failed (%llu bytes): requested size too large (> 2^62 bytes)", i, (unsigned long long)need);
        free_slot(s);
        if (writable && writable[i] && new_size <= kMappedOutputMax) {
            cudaError_t em = cudaHostAlloc(&s.staging, new_size, cudaHostAllocMapped);
            if (em == cudaSuccess) em = cudaHostGetDevicePointer(&s.dev, s.staging, 0);
            if (em == cudaSuccess) {
                std::memset(s.staging, 0, new_size);
                s.size = new_size, s.valid = 0, s.mapped = true;
                continue;
            }
            if (s.staging) cudaFreeHost(s.staging);
            s = Slot{};
            cudaGetLastError();   // fall back to a device buffer + staging copy
        }
        cudaError_t e = cudaMalloc(&s.dev, new_size);
        if (e != cudaSuccess) {
            s = Slot{};
            cudaGetLastError();
            return fail(AXC_ERR_BUFFER_ALLOCATION_FAILED, "buffer #%u allocation failed (%llu bytes): cudaMalloc: %s", i, (unsigned long long)need, cudaGetErrorString(e));
        }
        const bool map_in = (int)i == mapped_input && new_size <= kMappedInputMax;
        e = cudaHostAlloc(&s.staging, new_size, map_in ? cudaHostAllocMapped : cudaHostAllocDefault);
        if (e == cudaSuccess && map_in && cudaHostGetDevicePointer(&s.staging_dev, s.staging, 0) != cudaSuccess) {
            s.staging_dev = nullptr;   // not fatal: the copy path still works
            cudaGetLastError();
        }
        if (e != cudaSuccess) {
            cudaFree(s.dev);
            s = Slot{};
            cudaGetLastError();
            return fail(AXC_ERR_BUFFER_ALLOCATION_FAILED, "buffer #%u allocation failed (%llu bytes): cudaHostAlloc (staging): %s", i, (unsigned long long)need, cudaGetErrorString(e));
        }
        s.size = new_size;
        s.valid = 0;
    }
    g_fields.binding = 0;
    g_fields.size = 0;
    return AXC_OK;
}

int validate_counts(uint32_t n_bufs, uint32_t pc_total, const uint32_t wg[3], uint32_t n_inputs,
                    uint32_t n_outputs, size_t pc_len) {
    // Order of dispatch.rs:60-92: inputs, output_sizes, push constants, workgroup limits.
    if (n_inputs != n_bufs) {
        g_fields.expected = n_bufs, g_fields.provided = n_inputs;
        return fail(AXC_ERR_BINDING_COUNT_MISMATCH, "binding count mismatch: expected %u, got %u", n_bufs, n_inputs);
    }
    if (n_outputs != n_bufs) {
        g_fields.expected = n_bufs, g_fields.provided = n_outputs;
        return fail(AXC_ERR_BINDING_COUNT_MISMATCH, "binding count mismatch: expected %u, got %u", n_bufs, n_outputs);
    }
    if (pc_len != pc_total) {
        g_fields.expected = pc_total, g_fields.provided = pc_len;
        return fail(AXC_ERR_PUSH_CONSTANT_SIZE_MISMATCH, "push constant size mismatch: expected %u bytes, got %zu", pc_total, pc_len);
    }
    for (int a = 0; a < 3; ++a) {
        if (wg[a] > kMaxGrid[a]) {
            for (int b = 0; b < 3; ++b) g_fields.requested[b] = wg[b], g_fields.max[b] = kMaxGrid[b];
            return fail(AXC_ERR_WORKGROUP_COUNT_EXCEEDS_LIMIT, "workgroup count [%u, %u, %u] exceeds device limit [%u, %u, %u]", wg[0], wg[1], wg[2], kMaxGrid[0], kMaxGrid[1], kMaxGrid[2]);
        }
    }
    return AXC_OK;
}

int classify_kernel(const char* entry_point, const axc_buf_desc* bufs, uint32_t n_bufs,
                    uint32_t pc_total, KernelKind* kind) {
    const bool q4k = std::strcmp(entry_point, "q4km_dequant_matvec") == 0;
    const bool q40 = std::strcmp(entry_point, "q4_0_dequant_matvec") == 0;
    if (!q4k && !q40)
        return fail(AXC_ERR_PIPELINE_CREATION_FAILED, "failed to create compute pipeline: unsupported kernel for CUDA backend: %s", entry_point);
    bool shape_ok = n_bufs == 3 && pc_total == 4 && bufs;
    if (shape_ok) {
        shape_ok = bufs[0].elem_ty == AXC_TY_U8 && bufs[1].elem_ty == AXC_TY_F32 &&
                   bufs[2].elem_ty == AXC_TY_F32 && bufs[0].buffer_position == 0 &&
                   bufs[1].buffer_position == 1 && bufs[2].buffer_position == 2 &&
                   bufs[2].access != AXC_ACCESS_READ_ONLY;
    }
    if (!shape_ok)
        return fail(AXC_ERR_PIPELINE_CREATION_FAILED, "failed to create compute pipeline: unsupported kernel for CUDA backend: %s expects bindings [q: u8 readonly, x: f32 readonly, y: f32] and a 4-byte push constant", entry_point);
    *kind = q4k ? KernelKind::Q4K : KernelKind::Q4_0;
    return AXC_OK;
}

// Bounded wait for the completion word the matvec's last CTA writes to mapped host memory.
// Cheaper than an event (no extra command behind the kernel, no driver call per poll).  The
// stream is queried now and then so that a failed launch surfaces as an error, not a timeout.
bool wait_flag(const volatile uint32_t* flag, uint32_t seq, uint64_t timeout_ms, cudaStream_t st, cudaError_t* err) {
    using clock = std::chrono::steady_clock;
    const auto t0 = clock::now();
    const auto limit = std::chrono::milliseconds(timeout_ms);
    for (uint32_t spins = 1;; ++spins) {
        if (*flag == seq) {
            std::atomic_thread_fence(std::memory_order_acquire);   // y and the status word are read after the flag
            return true;
        }
#if defined(__x86_64__) || defined(__i386__)
        __builtin_ia32_pause();
#endif
        if ((spins & 1023u) == 0) {
            const cudaError_t q = cudaStreamQuery(st);
            if (q == cudaSuccess) {           // everything queued has finished
                if (*flag == seq) {
                    std::atomic_thread_fence(std::memory_order_acquire);
                    return true;
                }
                *err = cudaErrorUnknown;      // the kernel ended without signalling
                return false;
            }
            if (q != cudaErrorNotReady) {
                *err = q;
                return false;
            }
            const auto el = clock::now() - t0;
            if (el > limit) {
                *err = cudaErrorNotReady;
                return false;
            }
            if (el > std::chrono::milliseconds(2)) std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
    }
}

int dispatch_locked(axc_ctx* ctx, axc_kernel* k, const uint32_t wg[3], const void* const* inputs,
                    const size_t* input_lens, void* const* outputs, const size_t* output_sizes,
                    const void* pc, axc_dispatch_stats* stats) {
    DeviceGuard g(k->device);
    const bool writable[3] = {false, false, true};   // both kernels: [q, x] read-only, y written
    int rc = ensure_slots(k, input_lens, output_sizes, k->n_bufs == 3 ? writable : nullptr, k->n_bufs == 3 ? 1 : -1);
    if (rc != AXC_OK) return rc;
    cudaStream_t st = ctx->stream;
    const bool timed = stats != nullptr;
    cudaError_t e;

    // ---- host side of the uploads: into the pinned staging buffers ----
    for (uint32_t i = 0; i < k->n_bufs; ++i) {
        if (input_lens[i] == 0) continue;  // resident: keep device contents
        Slot& s = k->slots[i];
        std::memcpy(s.staging, inputs[i], input_lens[i]);
        s.valid = input_lens[i];
        if (!s.mapped) s.dev_stale = true;
    }

    // ---- geometry: rows from the grid, blocks per row from the push constant ----
    uint32_t n = 0;
    std::memcpy(&n, pc, 4);
    const uint64_t rows_req = std::min<uint64_t>((uint64_t)wg[0] * wg[1] * wg[2], 0xFFFFFFFFull);
    const uint32_t blk_bytes = k->kind == KernelKind::Q4K ? 144u : 18u;
    const uint32_t blk_elems = k->kind == KernelKind::Q4K ? 256u : 32u;
    const Slot& sq = k->slots[0];
    Slot& sx = k->slots[1];
    Slot& sy = k->slots[2];
    const uint64_t q_have = sq.valid ? sq.valid : sq.size;
    const uint64_t x_have = sx.valid ? sx.valid : sx.size;
    uint64_t y_have = std::max<uint64_t>(input_lens[2], output_sizes[2]);
    if (y_have == 0) y_have = sy.size;
    uint64_t rows = std::min<uint64_t>(rows_req, y_have / 4);
    if (n > 0) {
        const uint64_t row_bytes = (uint64_t)n * blk_bytes;
        rows = std::min<uint64_t>(rows, q_have / row_bytes);
        if (rows_req > 0 && rows == 0) {
            g_fields.binding = 0, g_fields.size = row_bytes;
            return fail(AXC_ERR_BUFFER_ALLOCATION_FAILED, "buffer #0 allocation failed (%llu bytes): q holds %llu bytes, one row of %u blocks needs %llu", (unsigned long long)row_bytes, (unsigned long long)q_have, n, (unsigned long long)row_bytes);
        }
        const uint64_t x_need = (uint64_t)n * blk_elems * 4;
        if (rows > 0 && x_have < x_need) {
            g_fields.binding = 1, g_fields.size = x_need;
            return fail(AXC_ERR_BUFFER_ALLOCATION_FAILED, "buffer #1 allocation failed (%llu bytes): x holds %llu bytes, %u blocks need %llu", (unsigned long long)x_need, (unsigned long long)x_have, n, (unsigned long long)x_need);
        }
    }

    // ---- the fast path: one launch, no copy-engine transfer for x, no event ----
    // x stays in its mapped staging buffer; the matvec's first CTAs read it over PCIe and quantise
    // it once for all CTAs (which meanwhile stream their weights), every CTA stores its rows of y
    // straight into mapped host memory, and the last CTA publishes a sequence number there, which
    // this thread polls.  Taken whenever the streaming kernel serves the shape and no device
    // timing was asked for.
    // (Inputs that are also read back take the copy path: x then has to be in device memory.)
    static const bool fast_enabled = [] {
        const char* v = std::getenv("AXC_DISPATCH_FAST");   // "0" forces the copy-and-event path
        return !(v && v[0] == '0' && v[1] == '\0');
    }();
    bool fast = fast_enabled && !timed && rows > 0 && n > 0 && !k->strict.load() && sx.staging_dev && sy.mapped &&
                output_sizes[0] == 0 && output_sizes[1] == 0 && !k->tune.x_prepared &&
                rows >= 64 &&   // enough CTAs for one producer per 64 x 64 columns of x (at most eight)
                (k->kind == KernelKind::Q4K ? axc::q4k_uses_stream_kernel(n) : axc::q4_0_uses_stream_kernel(n));
    if (fast && !k->fast_scratch) {
        // [quantised x image for rows of up to 32768 columns | 256 B of counters | y, up to the mapped-output limit]
        const size_t image = (axc::q4_prepared_x_bytes(512) + 255) & ~(size_t)255;
        if (cudaMalloc(&k->fast_scratch, image + 256 + kMappedOutputMax) == cudaSuccess &&
            cudaMemsetAsync((char*)k->fast_scratch + image, 0, 256, st) == cudaSuccess) {
            k->fast_image_bytes = image;
        } else {
            if (k->fast_scratch) cudaFree(k->fast_scratch);
            k->fast_scratch = nullptr;
            cudaGetLastError();
            fast = false;   // the copy path needs no scratch
        }
    }

    if (timed) cudaEventRecord(k->ev[0], st);
    for (uint32_t i = 0; i < k->n_bufs; ++i) {
        Slot& s = k->slots[i];
        if (s.mapped || !s.dev_stale) continue;      // the device reads the pinned buffer itself / nothing new
        if (fast && i == 1) continue;                // x is consumed from its mapped staging buffer
        e = cudaMemcpyAsync(s.dev, s.staging, s.valid, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) {
            g_fields.binding = i, g_fields.direction = AXC_COPY_HOST_TO_DEVICE;
            return fail(AXC_ERR_STAGING_COPY_FAILED, "staging copy failed for binding #%u (HostToDevice): %s", i, cudaGetErrorString(e));
        }
        s.dev_stale = false;
    }
    if (timed) cudaEventRecord(k->ev[1], st);

    uint32_t seq = 0;
    if (rows > 0) {
        if (n == 0) {
            e = cudaMemsetAsync(sy.dev, 0, rows * 4, st);  // empty sum: +0.0 per row
        } else if (k->strict.load()) {
            e = k->kind == KernelKind::Q4K
                    ? axc::launch_q4k_matvec_seq((const uint8_t*)sq.dev, (const float*)sx.dev, (float*)sy.dev, (uint32_t)rows, n, st)
                    : axc::launch_q4_0_matvec_seq((const uint8_t*)sq.dev, (const float*)sx.dev, (float*)sy.dev, (uint32_t)rows, n, st);
        } else if (fast) {
            seq = ++k->fast_seq;
            if (seq == 0) seq = ++k->fast_seq;   // 0 is what fresh flag words hold
            uint32_t* words = reinterpret_cast<uint32_t*>((char*)k->fast_scratch + k->fast_image_bytes);
            float* y_dev = reinterpret_cast<float*>((char*)k->fast_scratch + k->fast_image_bytes + 256);
            axc::DoneSignal done{words, k->status_dev + 4, seq, (float*)sy.dev};   // sy.dev: the mapped host view
            axc::HostX hx{(const float*)sx.staging_dev, words + 1, words + 2, seq};
            axc::MatvecTuning tune = k->tune;
            tune.x_prepared = k->fast_scratch;
            tune.done = &done;
            tune.host_x = &hx;
            tune.pdl = 0;   // nothing is in flight before it: a plain launch
            e = k->kind == KernelKind::Q4K
                    ? axc::launch_q4k_matvec((const uint8_t*)sq.dev, nullptr, y_dev, (uint32_t)rows, n, k->status_dev, st, tune, k->sm_count, nullptr)
                    : axc::launch_q4_0_matvec((const uint8_t*)sq.dev, nullptr, y_dev, (uint32_t)rows, n, k->status_dev, st, tune, k->sm_count, nullptr);
        } else {
            const axc::MatvecTuning& tune = k->tune;
            e = k->kind == KernelKind::Q4K
                    ? axc::launch_q4k_matvec((const uint8_t*)sq.dev, (const float*)sx.dev, (float*)sy.dev, (uint32_t)rows, n, k->status_dev, st, tune, k->sm_count, nullptr)
                    : axc::launch_q4_0_matvec((const uint8_t*)sq.dev, (const float*)sx.dev, (float*)sy.dev, (uint32_t)rows, n, k->status_dev, st, tune, k->sm_count, nullptr);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(AXC_ERR_QUEUE_SUBMIT_FAILED, "queue submit failed: kernel launch: %s", cudaGetErrorString(e));
        }
    }
    if (timed) cudaEventRecord(k->ev[2], st);

    bool copies_back = false;
    for (uint32_t i = 0; i < k->n_bufs; ++i) {
        if (output_sizes[i] == 0) continue;
        Slot& s = k->slots[i];
        if (s.mapped) continue;   // already in host memory when the kernel completes
        e = cudaMemcpyAsync(s.staging, s.dev, output_sizes[i], cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) {
            g_fields.binding = i, g_fields.direction = AXC_COPY_DEVICE_TO_HOST;
            return fail(AXC_ERR_STAGING_COPY_FAILED, "staging copy failed for binding #%u (DeviceToHost): %s", i, cudaGetErrorString(e));
        }
        copies_back = true;
    }

    const uint64_t timeout_ms = fence_timeout_ms_for(ctx);
    cudaError_t werr = cudaSuccess;
    bool ok;
    if (seq != 0 && !copies_back) {
        ok = wait_flag(k->status_host + 4, seq, timeout_ms, st, &werr);
    } else {
        e = cudaEventRecord(timed ? k->ev[3] : k->ev[4], st);
        if (e != cudaSuccess)
            return fail(AXC_ERR_QUEUE_SUBMIT_FAILED, "queue submit failed: %s", cudaGetErrorString(e));
        ok = wait_event(timed ? k->ev[3] : k->ev[4], timeout_ms, &werr);
    }
    if (!ok) {
        if (werr == cudaErrorNotReady) {
            g_fields.timeout_ns = timeout_ms * 1000000ull;
            return fail(AXC_ERR_FENCE_TIMEOUT, "fence wait timed out after %llu ns", (unsigned long long)g_fields.timeout_ns);
        }
        cudaGetLastError();
        return fail(AXC_ERR_QUEUE_SUBMIT_FAILED, "queue submit failed: %s", cudaGetErrorString(werr));
    }
    if (*(volatile uint32_t*)k->status_host != 0) {
        const uint32_t bits = *k->status_host;
        *k->status_host = 0;
        g_fields.timeout_ns = 0;
        return fail(AXC_ERR_FENCE_TIMEOUT, "fence wait timed out after 0 ns: kernel gave up waiting for its weight stream (status bits 0x%x)", bits);
    }
    for (uint32_t i = 0; i < k->n_bufs; ++i) {
        if (output_sizes[i] == 0) continue;
        if (!outputs[i]) {
            g_fields.binding = i;
            return fail(AXC_ERR_READBACK_FAILED, "readback of binding #%u failed: null output buffer for a non-zero output size", i);
        }
        std::memcpy(outputs[i], k->slots[i].staging, output_sizes[i]);
    }
    if (timed) {
        float a = 0, b = 0, c = 0, t = 0;
        cudaEventElapsedTime(&a, k->ev[0], k->ev[1]);
        cudaEventElapsedTime(&b, k->ev[1], k->ev[2]);
        cudaEventElapsedTime(&c, k->ev[2], k->ev[3]);
        cudaEventElapsedTime(&t, k->ev[0], k->ev[3]);
        stats->h2d_ns = (uint64_t)(a * 1e6f);
        stats->kernel_ns = (uint64_t)(b * 1e6f);
        stats->d2h_ns = (uint64_t)(c * 1e6f);
        stats->total_device_ns = (uint64_t)(t * 1e6f);
        stats->rows_effective = (uint32_t)rows;
        stats->blocks_per_row = n;
    }
    return AXC_OK;
}

int check_dispatch_args(axc_ctx* ctx, axc_kernel* k, const uint32_t* wg, const void* const* inputs,
                        const size_t* input_lens, uint32_t n_inputs, void* const* outputs,
                        const size_t* output_sizes, uint32_t n_outputs, const void* pc,
                        size_t pc_len) {
    if (!ctx || !k || !wg) return fail(AXC_ERR_INVALID_ARGUMENT, "null context, kernel or workgroups");
    if ((n_inputs && (!inputs || !input_lens)) || (n_outputs && !output_sizes))
        return fail(AXC_ERR_INVALID_ARGUMENT, "null inputs / input_lens / output_sizes array");
    if (pc_len && !pc) return fail(AXC_ERR_INVALID_ARGUMENT, "null push constants with non-zero length");
    int rc = validate_counts(k->n_bufs, k->pc_total, wg, n_inputs, n_outputs, pc_len);
    if (rc != AXC_OK) return rc;
    for (uint32_t i = 0; i < n_inputs; ++i)
        if (input_lens[i] && !inputs[i])
            return fail(AXC_ERR_INVALID_ARGUMENT, "input #%u is null with non-zero length", i);
    if (n_outputs && !outputs) {
        for (uint32_t i = 0; i < n_outputs; ++i)
            if (output_sizes[i]) return fail(AXC_ERR_INVALID_ARGUMENT, "null outputs array with a non-zero output size");
    }
    if (ctx->device != k->device)
        return fail(AXC_ERR_INVALID_ARGUMENT, "kernel handle belongs to device %d, context to device %d", k->device, ctx->device);
    return AXC_OK;
}

int sm_count_of_current_device() {
    static std::mutex mu;
    static std::map<int, int> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    std::lock_guard<std::mutex> l(mu);
    auto it = cache.find(dev);
    if (it != cache.end()) return it->second;
    int n = 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
    return n;
}

axc::MatvecTuning to_tuning(const axc_tuning* t) {
    axc::MatvecTuning m;
    if (t) {
        m.ctas_per_sm = t->ctas_per_sm, m.tile_rows = t->tile_rows, m.stages = t->stages;
        m.threads = t->threads, m.evict_first = t->evict_first, m.pdl = t->pdl, m.resident = t->resident;
    }
    return m;
}

int check_dev_ptrs(const void* q, const void* x, const void* y) {
    if (!q || !x || !y) return fail(AXC_ERR_INVALID_ARGUMENT, "null device pointer");
    if (((uintptr_t)q | (uintptr_t)x | (uintptr_t)y) & 15u)
        return fail(AXC_ERR_INVALID_ARGUMENT, "device pointers must be 16-byte aligned");
    return AXC_OK;
}

int launch_result(cudaError_t e) {
    if (e == cudaSuccess) return AXC_OK;
    cudaGetLastError();
    return fail(AXC_ERR_QUEUE_SUBMIT_FAILED, "queue submit failed: kernel launch: %s", cudaGetErrorString(e));
}

}  // namespace

extern "C" {

int axc_cuda_version(void) { return 100; }

int axc_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int axc_cuda_probe(void) {
    const int n = axc_cuda_device_count();
    for (int d = 0; d < n; ++d) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess && major == 10)
            return 1;
    }
    return 0;
}

int axc_cuda_gpu_tests_enabled(void) {
    const char* v = std::getenv("AXC_ENABLE_GPU_TESTS");
    return v && std::strcmp(v, "1") == 0;
}

int axc_cuda_ctx_create(const axc_ctx_opts* opts, axc_ctx** out) {
    clear_error();
    if (!out) return fail(AXC_ERR_INVALID_ARGUMENT, "null out pointer");
    *out = nullptr;
    int dev = opts ? opts->physical_device_index : -1;
    if (dev < 0) {
        dev = 0;
        if (const char* s = std::getenv("AXC_PHYSICAL_DEVICE_INDEX")) {
            char* end = nullptr;
            long v = std::strtol(s, &end, 10);
            if (end && end != s && *end == '\0' && v >= 0) dev = (int)v;
        }
    }
    const int n = axc_cuda_device_count();
    if (n <= 0) return fail(AXC_ERR_NO_SUPPORTED_DEVICE, "no CUDA device with compute capability 10.x");
    if (dev >= n) return fail(AXC_ERR_DEVICE_CREATION_FAILED, "failed to create logical device: device index %d out of range (%d devices)", dev, n);
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return fail(AXC_ERR_DEVICE_CREATION_FAILED, "failed to create logical device: %s", cudaGetErrorString(e));
    if (prop.major != 10) return fail(AXC_ERR_NO_SUPPORTED_DEVICE, "device %d (%s) is sm_%d%d; this backend is built for sm_100a only", dev, prop.name, prop.major, prop.minor);
    std::unique_ptr<axc_ctx> c(new axc_ctx);
    c->device = dev;
    c->sm_count = prop.multiProcessorCount;
    c->name = prop.name;
    c->fence_timeout_ms = opts ? opts->fence_timeout_ms : 0;
    c->table = std::make_shared<CacheTable>();
    DeviceGuard g(dev);
    e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail(AXC_ERR_DEVICE_CREATION_FAILED, "failed to create logical device: cudaStreamCreate: %s", cudaGetErrorString(e));
    *out = c.release();
    return AXC_OK;
}

void axc_cuda_ctx_destroy(axc_ctx* ctx) {
    if (!ctx) return;
    {
        DeviceGuard g(ctx->device);
        if (ctx->stream) {
            cudaStreamSynchronize(ctx->stream);  // vkDeviceWaitIdle of context.rs:575
            cudaStreamDestroy(ctx->stream);
        }
    }
    delete ctx;
}

size_t axc_cuda_ctx_device_name(const axc_ctx* ctx, char* buf, size_t cap) {
    if (!ctx) return 0;
    if (buf && cap) {
        const size_t n = std::min(cap - 1, ctx->name.size());
        std::memcpy(buf, ctx->name.data(), n);
        buf[n] = '\0';
    }
    return ctx->name.size();
}

void axc_cuda_ctx_max_grid(const axc_ctx*, uint32_t out[3]) {
    if (out) std::memcpy(out, kMaxGrid, sizeof kMaxGrid);
}

int axc_cuda_ctx_device_index(const axc_ctx* ctx) { return ctx ? ctx->device : -1; }
int axc_cuda_ctx_sm_count(const axc_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

int axc_cuda_prepare_kernel(axc_ctx* ctx, const char* entry_point, const axc_buf_desc* bufs,
                            uint32_t n_bufs, uint32_t pc_total_bytes, uint64_t spirv_hash,
                            uint64_t plan_hash, axc_kernel** out) {
    clear_error();
    if (!ctx || !entry_point || !out) return fail(AXC_ERR_INVALID_ARGUMENT, "null context, entry point or out pointer");
    *out = nullptr;
    KernelKind kind;
    int rc = classify_kernel(entry_point, bufs, n_bufs, pc_total_bytes, &kind);
    if (rc != AXC_OK) return rc;
    // The entry point is part of what the SPIR-V hash identifies in the reference; fold the
    // kind in so one hash cannot alias two kernels.
    const CacheKey key{spirv_hash ^ (kind == KernelKind::Q4K ? 0ull : 0x9E3779B97F4A7C15ull), plan_hash, pc_total_bytes};
    std::lock_guard<std::mutex> l(ctx->table->mu);
    auto it = ctx->table->live.find(key);
    if (it != ctx->table->live.end()) {
        it->second->refs.fetch_add(1);
        *out = it->second;
        return AXC_OK;
    }
    std::unique_ptr<axc_kernel> k(new axc_kernel);
    k->table = ctx->table;
    k->key = key;
    k->kind = kind;
    k->device = ctx->device;
    k->sm_count = ctx->sm_count;
    k->n_bufs = n_bufs;
    k->pc_total = pc_total_bytes;
    DeviceGuard g(ctx->device);
    // The kernel's error word lives in mapped pinned host memory: it is written only when a
    // bounded wait gives up, and reading it back costs no copy after the kernel.
    cudaError_t e = cudaHostAlloc((void**)&k->status_host, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) {
        std::memset(k->status_host, 0, 64);
        e = cudaHostGetDevicePointer((void**)&k->status_dev, k->status_host, 0);
    }
    for (auto& ev : k->ev)
        if (e == cudaSuccess) e = cudaEventCreate(&ev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        axc_kernel* raw = k.release();
        destroy_kernel(raw);
        return fail(AXC_ERR_PIPELINE_CREATION_FAILED, "failed to create compute pipeline: %s", cudaGetErrorString(e));
    }
    *k->status_host = 0;
    ctx->table->live[key] = k.get();
    *out = k.release();
    return AXC_OK;
}

void axc_cuda_kernel_retain(axc_kernel* k) {
    if (k) k->refs.fetch_add(1);
}

void axc_cuda_kernel_release(axc_kernel* k) {
    if (!k) return;
    std::shared_ptr<CacheTable> table = k->table;
    {
        std::lock_guard<std::mutex> l(table->mu);
        if (k->refs.fetch_sub(1) != 1) return;
        auto it = table->live.find(k->key);
        if (it != table->live.end() && it->second == k) table->live.erase(it);
    }
    destroy_kernel(k);
}

uint32_t axc_cuda_kernel_buffer_sizes(const axc_kernel* k, uint64_t* out, uint32_t cap) {
    if (!k) return 0;
    axc_kernel* m = const_cast<axc_kernel*>(k);
    std::lock_guard<std::mutex> l(m->mu);
    uint32_t n = 0;
    for (const Slot& s : m->slots) {
        if (!s.dev) continue;
        if (out && n < cap) out[n] = s.size;
        ++n;
    }
    return n;
}

void axc_cuda_kernel_cache_key(const axc_kernel* k, uint64_t* spirv_hash, uint64_t* plan_hash,
                               uint32_t* pc_total_bytes) {
    if (!k) return;
    if (spirv_hash) *spirv_hash = k->key.spirv_hash;
    if (plan_hash) *plan_hash = k->key.plan_hash;
    if (pc_total_bytes) *pc_total_bytes = k->key.pc_bytes;
}

void axc_cuda_kernel_set_strict_order(axc_kernel* k, int strict) {
    if (k) k->strict.store(strict ? 1 : 0);
}

void axc_cuda_kernel_set_tuning(axc_kernel* k, const axc_tuning* tuning) {
    if (!k) return;
    std::lock_guard<std::mutex> lock(k->mu);
    k->tune = to_tuning(tuning);
}

int axc_cuda_dispatch(axc_ctx* ctx, axc_kernel* k, const uint32_t workgroups[3],
                      const void* const* inputs, const size_t* input_lens, uint32_t n_inputs,
                      void* const* outputs, const size_t* output_sizes, uint32_t n_outputs,
                      const void* push_constants, size_t pc_len, axc_dispatch_stats* stats) {
    clear_error();
    int rc = check_dispatch_args(ctx, k, workgroups, inputs, input_lens, n_inputs, outputs, output_sizes, n_outputs, push_constants, pc_len);
    if (rc != AXC_OK) return rc;
    std::lock_guard<std::mutex> l(k->mu);
    return dispatch_locked(ctx, k, workgroups, inputs, input_lens, outputs, output_sizes, push_constants, stats);
}

int axc_cuda_dispatch_oneshot(axc_ctx* ctx, const char* entry_point, const axc_buf_desc* bufs,
                              uint32_t n_bufs, uint32_t pc_total_bytes, uint64_t spirv_hash,
                              uint64_t plan_hash, const uint32_t workgroups[3],
                              const void* const* inputs, const size_t* input_lens,
                              uint32_t n_inputs, void* const* outputs, const size_t* output_sizes,
                              uint32_t n_outputs, const void* push_constants, size_t pc_len,
                              axc_dispatch_stats* stats) {
    clear_error();
    if (!ctx || !workgroups) return fail(AXC_ERR_INVALID_ARGUMENT, "null context or workgroups");
    // dispatch.rs:109-132 validates against the plan before preparing the kernel.
    int rc = validate_counts(n_bufs, pc_total_bytes, workgroups, n_inputs, n_outputs, pc_len);
    if (rc != AXC_OK) return rc;
    axc_kernel* k = nullptr;
    rc = axc_cuda_prepare_kernel(ctx, entry_point, bufs, n_bufs, pc_total_bytes, spirv_hash, plan_hash, &k);
    if (rc != AXC_OK) return rc;
    rc = axc_cuda_dispatch(ctx, k, workgroups, inputs, input_lens, n_inputs, outputs, output_sizes, n_outputs, push_constants, pc_len, stats);
    const std::string keep = g_detail;
    const axc_error_fields keep_f = g_fields;
    axc_cuda_kernel_release(k);
    g_detail = keep;
    g_fields = keep_f;
    return rc;
}

int axc_cuda_bench_dispatch(axc_ctx* ctx, axc_kernel* k, const uint32_t workgroups[3],
                            const void* const* inputs, const size_t* input_lens, uint32_t n_inputs,
                            void* const* outputs, const size_t* output_sizes, uint32_t n_outputs,
                            const void* push_constants, size_t pc_len, uint32_t sample_count,
                            uint64_t* samples_ns, uint64_t* median_ns, uint64_t* device_kernel_ns) {
    clear_error();
    if (sample_count == 0 || !samples_ns || !median_ns)
        return fail(AXC_ERR_INVALID_ARGUMENT, "sample_count must be >= 1 and samples/median must be non-null");
    for (uint32_t s = 0; s < sample_count; ++s) {
        axc_dispatch_stats st{};
        const auto t0 = std::chrono::steady_clock::now();
        const int rc = axc_cuda_dispatch(ctx, k, workgroups, inputs, input_lens, n_inputs, outputs, output_sizes, n_outputs, push_constants, pc_len, device_kernel_ns ? &st : nullptr);
        const auto t1 = std::chrono::steady_clock::now();
        if (rc != AXC_OK) return rc;
        samples_ns[s] = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count();
        if (device_kernel_ns) device_kernel_ns[s] = st.kernel_ns;
    }
    std::vector<uint64_t> sorted(samples_ns, samples_ns + sample_count);
    std::sort(sorted.begin(), sorted.end());
    *median_ns = sorted[sorted.size() / 2];  // bench_variant.rs:299-301
    return AXC_OK;
}

const char* axc_cuda_strerror(int status) {
    switch (status) {
        case AXC_OK: return "ok";
        case AXC_ERR_NO_SUPPORTED_DEVICE: return "NoSupportedDevice";
        case AXC_ERR_DEVICE_CREATION_FAILED: return "DeviceCreationFailed";
        case AXC_ERR_PIPELINE_CREATION_FAILED: return "PipelineCreationFailed";
        case AXC_ERR_BUFFER_ALLOCATION_FAILED: return "BufferAllocationFailed";
        case AXC_ERR_QUEUE_SUBMIT_FAILED: return "QueueSubmitFailed";
        case AXC_ERR_FENCE_TIMEOUT: return "FenceTimeout";
        case AXC_ERR_READBACK_FAILED: return "ReadbackFailed";
        case AXC_ERR_BINDING_COUNT_MISMATCH: return "BindingCountMismatch";
        case AXC_ERR_PUSH_CONSTANT_SIZE_MISMATCH: return "PushConstantSizeMismatch";
        case AXC_ERR_WORKGROUP_COUNT_EXCEEDS_LIMIT: return "WorkgroupCountExceedsDeviceLimit";
        case AXC_ERR_STAGING_COPY_FAILED: return "StagingCopyFailed";
        case AXC_ERR_INVALID_ARGUMENT: return "InvalidArgument";
        default: return "Unknown";
    }
}

size_t axc_cuda_last_error_detail(char* buf, size_t cap) {
    if (buf && cap) {
        const size_t n = std::min(cap - 1, g_detail.size());
        std::memcpy(buf, g_detail.data(), n);
        buf[n] = '\0';
    }
    return g_detail.size();
}

void axc_cuda_last_error_fields(axc_error_fields* out) {
    if (out) *out = g_fields;
}

// ---- device layer ----

int axc_cuda_q4k_matvec(const void* q, const float* x, float* y, uint32_t rows,
                        uint32_t n_superblocks, void* stream, uint32_t* status,
                        const axc_tuning* tuning) {
    clear_error();
    if (rows == 0) return AXC_OK;
    int rc = check_dev_ptrs(q, x, y);
    if (rc != AXC_OK) return rc;
    if (n_superblocks == 0)
        return launch_result(cudaMemsetAsync(y, 0, (size_t)rows * 4, (cudaStream_t)stream));
    return launch_result(axc::launch_q4k_matvec((const uint8_t*)q, x, y, rows, n_superblocks, status, (cudaStream_t)stream, to_tuning(tuning), sm_count_of_current_device(), nullptr));
}

int axc_cuda_q4_0_matvec(const void* q, const float* x, float* y, uint32_t rows,
                         uint32_t n_blocks, void* stream, uint32_t* status,
                         const axc_tuning* tuning) {
    clear_error();
    if (rows == 0) return AXC_OK;
    int rc = check_dev_ptrs(q, x, y);
    if (rc != AXC_OK) return rc;
    if (n_blocks == 0)
        return launch_result(cudaMemsetAsync(y, 0, (size_t)rows * 4, (cudaStream_t)stream));
    return launch_result(axc::launch_q4_0_matvec((const uint8_t*)q, x, y, rows, n_blocks, status, (cudaStream_t)stream, to_tuning(tuning), sm_count_of_current_device(), nullptr));
}

int axc_cuda_q4k_matvec_seq(const void* q, const float* x, float* y, uint32_t rows,
                            uint32_t n_superblocks, void* stream) {
    clear_error();
    if (rows == 0) return AXC_OK;
    int rc = check_dev_ptrs(q, x, y);
    if (rc != AXC_OK) return rc;
    return launch_result(axc::launch_q4k_matvec_seq((const uint8_t*)q, x, y, rows, n_superblocks, (cudaStream_t)stream));
}

int axc_cuda_q4_0_matvec_seq(const void* q, const float* x, float* y, uint32_t rows,
                             uint32_t n_blocks, void* stream) {
    clear_error();
    if (rows == 0) return AXC_OK;
    int rc = check_dev_ptrs(q, x, y);
    if (rc != AXC_OK) return rc;
    return launch_result(axc::launch_q4_0_matvec_seq((const uint8_t*)q, x, y, rows, n_blocks, (cudaStream_t)stream));
}

int axc_cuda_q4k_dequant(const void* q, float* w, uint32_t rows, uint32_t n_superblocks,
                         void* stream) {
    clear_error();
    if (rows == 0 || n_superblocks == 0) return AXC_OK;
    int rc = check_dev_ptrs(q, w, w);
    if (rc != AXC_OK) return rc;
    return launch_result(axc::launch_q4k_dequant((const uint8_t*)q, w, rows, n_superblocks, (cudaStream_t)stream));
}

int axc_cuda_q4_0_dequant(const void* q, float* w, uint32_t rows, uint32_t n_blocks, void* stream) {
    clear_error();
    if (rows == 0 || n_blocks == 0) return AXC_OK;
    int rc = check_dev_ptrs(q, w, w);
    if (rc != AXC_OK) return rc;
    return launch_result(axc::launch_q4_0_dequant((const uint8_t*)q, w, rows, n_blocks, (cudaStream_t)stream));
}

int axc_cuda_q4k_matvec_allgather(const void* q, const float* x, uint32_t rows_local,
                                  uint32_t n_superblocks, const axc_gather* g, void* stream,
                                  uint32_t* status, const axc_tuning* tuning) {
    clear_error();
    if (rows_local == 0) return AXC_OK;
    if (!g || !g->y_peer_bases || !g->epoch || g->world == 0 || g->world > 16 || g->rank >= g->world || ((g->y_offset_bytes | g->parity_stride_bytes) & 7u))
        return fail(AXC_ERR_INVALID_ARGUMENT, "incomplete all-gather description");
    if (!q || !x || (((uintptr_t)q | (uintptr_t)x) & 15u))
        return fail(AXC_ERR_INVALID_ARGUMENT, "q and x must be non-null and 16-byte aligned");
    if (n_superblocks == 0 || n_superblocks > 128)
        return fail(AXC_ERR_INVALID_ARGUMENT, "the fused all-gather serves rows of 1..128 superblocks");
    axc::GatherArgs ga{};
    ga.y_peer_bases = g->y_peer_bases, ga.y_offset_bytes = g->y_offset_bytes, ga.epoch_ptr = g->epoch;
    ga.world = g->world, ga.rank = g->rank, ga.row_offset = g->row_offset;
    ga.parity_stride_bytes = g->parity_stride_bytes;
    axc::MatvecTuning t = to_tuning(tuning);
    t.gather = &ga;
    return launch_result(axc::launch_q4k_matvec((const uint8_t*)q, x, nullptr, rows_local, n_superblocks, status, (cudaStream_t)stream, t, sm_count_of_current_device(), nullptr));
}

int axc_cuda_q4k_prefill(const void* q, const uint16_t* a_bf16, float* c, uint32_t m_tokens,
                         uint32_t n_rows, uint32_t n_superblocks, void* stream, uint32_t* status) {
    return axc_cuda_q4k_prefill_form(q, a_bf16, c, m_tokens, n_rows, n_superblocks, stream, status, 0, 0);
}

int axc_cuda_q4k_prefill_form(const void* q, const uint16_t* a_bf16, float* c, uint32_t m_tokens,
                              uint32_t n_rows, uint32_t n_superblocks, void* stream, uint32_t* status, int form,
                              uint32_t flags) {
    clear_error();
    if (form < 0 || form > 2) return fail(AXC_ERR_INVALID_ARGUMENT, "prefill form must be 0 (choose), 1 (single CTA) or 2 (CTA pair)");
    if (m_tokens == 0 || n_rows == 0) return AXC_OK;
    if (n_superblocks == 0) return fail(AXC_ERR_INVALID_ARGUMENT, "prefill needs at least one superblock per row");
    int rc = check_dev_ptrs(q, a_bf16, c);
    if (rc != AXC_OK) return rc;
    if ((uint64_t)n_superblocks * 144u >= (1ull << 32) || (uint64_t)m_tokens * n_rows >= (1ull << 40))
        return fail(AXC_ERR_INVALID_ARGUMENT, "prefill shape out of range");
    cudaError_t e = axc::launch_q4k_prefill((const uint8_t*)q, a_bf16, c, m_tokens, n_rows, n_superblocks, status, (cudaStream_t)stream, form, (flags & AXC_PREFILL_INDEPENDENT) != 0);
    if (e == cudaErrorNotSupported)
        return fail(AXC_ERR_PIPELINE_CREATION_FAILED, "pipeline creation failed: the driver does not provide cuTensorMapEncodeTiled");
    if (e == cudaErrorInvalidValue)
        return fail(AXC_ERR_INVALID_ARGUMENT, "tensor map rejected (pointer alignment or shape)");
    return launch_result(e);
}

int axc_cuda_q4k_matvec_fused(const void* q, const axc_xsrc* xs, float* y, uint32_t rows,
                              uint32_t n_superblocks, const axc_gather* g, void* stream,
                              uint32_t* status, const axc_tuning* tuning) {
    clear_error();
    if (rows == 0) return AXC_OK;
    if (!xs || (!xs->x == !xs->x_pairs) || (xs->x2 && xs->x2_pairs))
        return fail(AXC_ERR_INVALID_ARGUMENT, "x source: exactly one of x / x_pairs, at most one of x2 / x2_pairs");
    if ((xs->x_pairs || xs->x2_pairs) && !xs->epoch)
        return fail(AXC_ERR_INVALID_ARGUMENT, "x source: (value, epoch) vectors need the epoch counter");
    if (!q || (((uintptr_t)q | (uintptr_t)xs->x | (uintptr_t)xs->x2 | (uintptr_t)xs->x_pairs | (uintptr_t)xs->x2_pairs) & 15u))
        return fail(AXC_ERR_INVALID_ARGUMENT, "q and the x sources must be 16-byte aligned (q non-null)");
    if (n_superblocks == 0 || n_superblocks > 128)
        return fail(AXC_ERR_INVALID_ARGUMENT, "the fused matvec serves rows of 1..128 superblocks");
    if (!g && (!y || ((uintptr_t)y & 15u)))
        return fail(AXC_ERR_INVALID_ARGUMENT, "y must be non-null and 16-byte aligned when no all-gather is given");
    axc::GatherArgs ga{};
    axc::MatvecTuning t = to_tuning(tuning);
    if (g) {
        if (!g->y_peer_bases || !g->epoch || g->world == 0 || g->world > 16 || g->rank >= g->world || ((g->y_offset_bytes | g->parity_stride_bytes) & 7u))
            return fail(AXC_ERR_INVALID_ARGUMENT, "incomplete all-gather description");
        ga.y_peer_bases = g->y_peer_bases, ga.y_offset_bytes = g->y_offset_bytes, ga.epoch_ptr = g->epoch;
        ga.world = g->world, ga.rank = g->rank, ga.row_offset = g->row_offset;
        ga.parity_stride_bytes = g->parity_stride_bytes;
        t.gather = &ga;
    }
    axc::XSource src;
    src.x = xs->x, src.x2 = xs->x2, src.x_pairs = xs->x_pairs, src.x2_pairs = xs->x2_pairs;
    src.epoch_ptr = xs->epoch, src.unit_rms = xs->unit_rms ? 1 : 0;
    src.parity_stride_bytes = xs->parity_stride_bytes;
    t.xsrc = &src;
    return launch_result(axc::launch_q4k_matvec((const uint8_t*)q, nullptr, y, rows, n_superblocks, status, (cudaStream_t)stream, t, sm_count_of_current_device(), nullptr));
}

size_t axc_cuda_q4k_prepared_x_bytes(uint32_t n_superblocks) { return axc::q4_prepared_x_bytes(n_superblocks * 4u); }

static int check_xsrc(const axc_xsrc* xs) {
    if (!xs || (!xs->x == !xs->x_pairs) || (xs->x2 && xs->x2_pairs))
        return fail(AXC_ERR_INVALID_ARGUMENT, "x source: exactly one of x / x_pairs, at most one of x2 / x2_pairs");
    if ((xs->x_pairs || xs->x2_pairs) && !xs->epoch)
        return fail(AXC_ERR_INVALID_ARGUMENT, "x source: (value, epoch) vectors need the epoch counter");
    if (((uintptr_t)xs->x | (uintptr_t)xs->x2 | (uintptr_t)xs->x_pairs | (uintptr_t)xs->x2_pairs) & 15u)
        return fail(AXC_ERR_INVALID_ARGUMENT, "x sources must be 16-byte aligned");
    return AXC_OK;
}

int axc_cuda_q4k_prepare_x(const axc_xsrc* xs, void* image, float* plain_out, uint32_t n_superblocks,
                           void* stream, uint32_t* status, uint32_t flags) {
    clear_error();
    if (n_superblocks == 0) return AXC_OK;
    int rc = check_xsrc(xs);
    if (rc != AXC_OK) return rc;
    if (!image || ((uintptr_t)image & 15u) || ((uintptr_t)plain_out & 15u))
        return fail(AXC_ERR_INVALID_ARGUMENT, "image must be non-null; image and plain_out 16-byte aligned");
    if (n_superblocks > 128) return fail(AXC_ERR_INVALID_ARGUMENT, "a prepared x serves rows of 1..128 superblocks");
    if ((flags & AXC_FINISH_OVERLAP_PREVIOUS) && (xs->x || xs->x2))
        return fail(AXC_ERR_INVALID_ARGUMENT, "only (value, epoch) sources may overlap the launch before");
    axc::XSource src;
    src.x = xs->x, src.x2 = xs->x2, src.x_pairs = xs->x_pairs, src.x2_pairs = xs->x2_pairs, src.epoch_ptr = xs->epoch;
    src.parity_stride_bytes = xs->parity_stride_bytes;
    return launch_result(axc::launch_q4_prepare_x(src, image, plain_out, n_superblocks * 4u, status, (cudaStream_t)stream,
                                                  (flags & AXC_FINISH_OVERLAP_PREVIOUS) != 0));
}

int axc_cuda_q4k_matvec_prepared(const void* q, const void* image, uint32_t unit_rms, float* y, uint32_t rows,
                                 uint32_t n_superblocks, const axc_gather* g, void* stream, uint32_t* status,
                                 const axc_tuning* tuning) {
    clear_error();
    if (rows == 0) return AXC_OK;
    if (!q || !image || (((uintptr_t)q | (uintptr_t)image) & 15u))
        return fail(AXC_ERR_INVALID_ARGUMENT, "q and the prepared x must be non-null and 16-byte aligned");
    if (n_superblocks == 0 || n_superblocks > 128)
        return fail(AXC_ERR_INVALID_ARGUMENT, "a prepared x serves rows of 1..128 superblocks");
    if (!g && (!y || ((uintptr_t)y & 15u)))
        return fail(AXC_ERR_INVALID_ARGUMENT, "y must be non-null and 16-byte aligned when no all-gather is given");
    axc::GatherArgs ga{};
    axc::MatvecTuning t = to_tuning(tuning);
    if (g) {
        if (!g->y_peer_bases || !g->epoch || g->world == 0 || g->world > 16 || g->rank >= g->world || ((g->y_offset_bytes | g->parity_stride_bytes) & 7u))
            return fail(AXC_ERR_INVALID_ARGUMENT, "incomplete all-gather description");
        ga.y_peer_bases = g->y_peer_bases, ga.y_offset_bytes = g->y_offset_bytes, ga.epoch_ptr = g->epoch;
        ga.world = g->world, ga.rank = g->rank, ga.row_offset = g->row_offset;
        ga.parity_stride_bytes = g->parity_stride_bytes;
        t.gather = &ga;
    }
    t.x_prepared = image, t.x_prepared_rms = unit_rms ? 1 : 0;
    return launch_result(axc::launch_q4k_matvec((const uint8_t*)q, nullptr, y, rows, n_superblocks, status, (cudaStream_t)stream, t, sm_count_of_current_device(), nullptr));
}

int axc_cuda_gather_next_epoch(uint32_t* epoch, void* stream) {
    clear_error();
    if (!epoch) return fail(AXC_ERR_INVALID_ARGUMENT, "null epoch counter");
    return launch_result(axc::launch_gather_next_epoch(epoch, (cudaStream_t)stream));
}

int axc_cuda_gather_finish(const uint64_t* pairs, const uint32_t* epoch, float* out, uint32_t n,
                           void* stream, uint32_t* status, uint32_t flags, uint64_t parity_stride_bytes,
                           const axc_gather_sync* sync) {
    clear_error();
    if (n == 0 && !sync) return AXC_OK;
    if (!epoch || (n && (!pairs || !out)) || ((uintptr_t)pairs & 7u) || (parity_stride_bytes & 7u))
        return fail(AXC_ERR_INVALID_ARGUMENT, "null or misaligned pair storage / epoch / output");
    axc::GatherSync gs{};
    if (sync) {
        if (!sync->done_peer_bases || !sync->done_local || !sync->arrive_counter || !sync->epoch ||
            sync->world == 0 || sync->world > 16 || sync->rank >= sync->world)
            return fail(AXC_ERR_INVALID_ARGUMENT, "incomplete end-of-step handshake description");
        if (flags & AXC_FINISH_OVERLAP_PREVIOUS)
            return fail(AXC_ERR_INVALID_ARGUMENT, "the end-of-step handshake advances the epoch: it cannot overlap the launch before it");
        gs.done_peer_bases = sync->done_peer_bases, gs.done_local = sync->done_local;
        gs.arrive_counter = sync->arrive_counter, gs.epoch_rw = sync->epoch, gs.world = sync->world, gs.rank = sync->rank;
    }
    return launch_result(axc::launch_gather_finish(pairs, epoch, out, n, status, (cudaStream_t)stream,
                                                   (flags & AXC_FINISH_OVERLAP_PREVIOUS) != 0, parity_stride_bytes,
                                                   sync ? &gs : nullptr, (flags & AXC_FINISH_LET_NEXT_START) != 0));
}

int axc_cuda_gather_reduce_finish(const uint64_t* pairs, const uint32_t* epoch, float* out, uint32_t n,
                                  uint32_t n_parts, uint64_t part_stride_bytes, void* stream, uint32_t* status,
                                  uint32_t flags, uint64_t parity_stride_bytes) {
    clear_error();
    if (n == 0) return AXC_OK;
    if (!pairs || !epoch || !out || ((uintptr_t)pairs & 7u) || ((part_stride_bytes | parity_stride_bytes) & 7u))
        return fail(AXC_ERR_INVALID_ARGUMENT, "null or misaligned pair storage / epoch / output");
    if (n_parts == 0 || n_parts > 16) return fail(AXC_ERR_INVALID_ARGUMENT, "1..16 parts");
    return launch_result(axc::launch_gather_reduce_finish(pairs, epoch, out, n, n_parts, part_stride_bytes, status,
                                                          (cudaStream_t)stream, (flags & AXC_FINISH_OVERLAP_PREVIOUS) != 0,
                                                          parity_stride_bytes));
}

int axc_cuda_q4k_matvec_plan(uint32_t rows, uint32_t n_superblocks, const axc_tuning* tuning,
                             int32_t sm_count, int32_t out[5]) {
    clear_error();
    if (!out) return fail(AXC_ERR_INVALID_ARGUMENT, "null out array");
    axc::MatvecTuning t = to_tuning(tuning);
    t.dry_run = 1;
    axc::LaunchInfo info;
    cudaError_t e = axc::launch_q4k_matvec(nullptr, nullptr, nullptr, rows, n_superblocks, nullptr, nullptr, t, sm_count > 0 ? sm_count : 148, &info);
    if (e != cudaSuccess) return fail(AXC_ERR_INVALID_ARGUMENT, "no launch geometry for rows=%u n=%u", rows, n_superblocks);
    out[0] = info.grid, out[1] = info.block, out[2] = (int32_t)info.smem, out[3] = info.tile_rows, out[4] = info.stages;
    return AXC_OK;
}

}  // extern "C"
