// C++ host-side mirror of axc-runtime's public surface over the CUDA C ABI (axc_cuda.h).
//
// The reference's callers (axc-driver's benches and tests, bench_variant, grid_search) use the
// concrete Rust methods of `axc_runtime::VulkanContext` (crates/axc-runtime/src/lib.rs:57-62).
// A Rust backend module would wrap libaxc_cuda.so with exactly these types; this header is the
// same surface for C++ hosts, with the same names, argument meaning and error behaviour:
//
//   VulkanContextOptions / VulkanContext      crates/axc-runtime/src/context.rs:76-109,160-547
//   KernelHandle / KernelCacheKey             crates/axc-runtime/src/kernel_handle.rs:44-51,123-151
//   DispatchRequest                           crates/axc-runtime/src/dispatch.rs:33-50
//   DispatchError (25 variants) / CopyDirection   crates/axc-runtime/src/error.rs:14-198
//   ParamBindingPlan and its slots            crates/axc-hir/src/param.rs:66-126
//   probe_vulkan_available, gpu_tests_enabled, captured_icd_path   crates/axc-runtime/src/icd.rs:22-80
//   KernelMetadata, load_kernel_metadata, CURRENT_SCHEMA_VERSION   crates/axc-runtime/src/metadata.rs:35,45-122
//
// Rust's `Result<T, DispatchError>` becomes `axc::Result<T>` (a value or an error, never an
// exception).  Header-only; link with libaxc_cuda.so.  There is no CPU fallback behind it.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <variant>
#include <vector>

#include "axc_cuda.h"

namespace axc {

enum class CopyDirection { HostToDevice = 0, DeviceToHost = 1 };   // error.rs:14-20

// error.rs:27-195.  All 25 variants exist so that code written against the reference's enum keeps
// its shape; the CUDA backend produces the ones axc_cuda.h lists.
enum class ErrorKind {
    VulkanEntryFailed, NoVulkanInstance, NoSupportedDevice, NoComputeQueue, DeviceCreationFailed,
    ShaderModuleCreationFailed, DescriptorSetLayoutFailed, DescriptorPoolFailed, PipelineLayoutFailed,
    PipelineCreationFailed, BufferAllocationFailed, MemoryMapFailed, NoCompatibleMemoryType,
    CommandBufferRecordFailed, QueueSubmitFailed, FenceTimeout, ReadbackFailed, BindingCountMismatch,
    PushConstantSizeMismatch, WorkgroupCountExceedsDeviceLimit, MetadataIoError, MetadataParseError,
    MetadataSchemaMismatch, PipelineCacheLoadFailed, StagingCopyFailed,
    InvalidArgument   // a null / malformed argument at the C boundary; no Rust counterpart
};
constexpr int kDispatchErrorVariantCount = 25;   // the count error.rs pins (AT-801)

struct DispatchError {
    ErrorKind kind = ErrorKind::QueueSubmitFailed;
    std::string message;            // the reference's Display text
    uint32_t binding = 0;           // BufferAllocationFailed, ReadbackFailed, StagingCopyFailed
    uint64_t size = 0;              // BufferAllocationFailed
    uint64_t expected = 0, provided = 0;   // BindingCountMismatch, PushConstantSizeMismatch
    uint64_t timeout_ns = 0;        // FenceTimeout
    uint32_t requested[3] = {0, 0, 0}, max[3] = {0, 0, 0};   // WorkgroupCountExceedsDeviceLimit
    CopyDirection direction = CopyDirection::HostToDevice;   // StagingCopyFailed
};

template <class T>
class Result {
public:
    Result(T v) : v_(std::move(v)) {}
    Result(DispatchError e) : v_(std::move(e)) {}
    bool is_ok() const { return v_.index() == 0; }
    bool is_err() const { return !is_ok(); }
    T& unwrap() {
        if (!is_ok()) std::abort();   // Rust's unwrap() panics
        return std::get<0>(v_);
    }
    const DispatchError& unwrap_err() const {
        if (is_ok()) std::abort();
        return std::get<1>(v_);
    }
private:
    std::variant<T, DispatchError> v_;
};

namespace detail {
inline DispatchError last_error(int status) {
    DispatchError e;
    const size_t n = axc_cuda_last_error_detail(nullptr, 0);
    std::string msg(n + 1, '\0');
    axc_cuda_last_error_detail(msg.data(), n + 1);
    msg.resize(n);
    e.message = msg.empty() ? std::string(axc_cuda_strerror(status)) : msg;
    axc_error_fields f;
    axc_cuda_last_error_fields(&f);
    e.binding = f.binding, e.size = f.size, e.expected = f.expected, e.provided = f.provided;
    e.timeout_ns = f.timeout_ns;
    e.direction = f.direction == AXC_COPY_DEVICE_TO_HOST ? CopyDirection::DeviceToHost : CopyDirection::HostToDevice;
    for (int i = 0; i < 3; ++i) e.requested[i] = f.requested[i], e.max[i] = f.max[i];
    switch (status) {
        case AXC_ERR_NO_SUPPORTED_DEVICE: e.kind = ErrorKind::NoSupportedDevice; break;
        case AXC_ERR_DEVICE_CREATION_FAILED: e.kind = ErrorKind::DeviceCreationFailed; break;
        case AXC_ERR_PIPELINE_CREATION_FAILED: e.kind = ErrorKind::PipelineCreationFailed; break;
        case AXC_ERR_BUFFER_ALLOCATION_FAILED: e.kind = ErrorKind::BufferAllocationFailed; break;
        case AXC_ERR_QUEUE_SUBMIT_FAILED: e.kind = ErrorKind::QueueSubmitFailed; break;
        case AXC_ERR_FENCE_TIMEOUT: e.kind = ErrorKind::FenceTimeout; break;
        case AXC_ERR_READBACK_FAILED: e.kind = ErrorKind::ReadbackFailed; break;
        case AXC_ERR_BINDING_COUNT_MISMATCH: e.kind = ErrorKind::BindingCountMismatch; break;
        case AXC_ERR_PUSH_CONSTANT_SIZE_MISMATCH: e.kind = ErrorKind::PushConstantSizeMismatch; break;
        case AXC_ERR_WORKGROUP_COUNT_EXCEEDS_LIMIT: e.kind = ErrorKind::WorkgroupCountExceedsDeviceLimit; break;
        case AXC_ERR_STAGING_COPY_FAILED: e.kind = ErrorKind::StagingCopyFailed; break;
        case AXC_ERR_INVALID_ARGUMENT: e.kind = ErrorKind::InvalidArgument; break;
        default: e.kind = ErrorKind::QueueSubmitFailed; break;
    }
    return e;
}
inline uint64_t fnv1a64(const void* p, size_t n, uint64_t h = 1469598103934665603ull) {
    const unsigned char* b = static_cast<const unsigned char*>(p);
    for (size_t i = 0; i < n; ++i) h = (h ^ b[i]) * 1099511628211ull;
    return h;
}
}  // namespace detail

// ---- binding plan (crates/axc-hir/src/param.rs, buffer.rs, ty.rs) ----
enum class ScalarTy { U8, F32, U32, Other };
enum class BufferAccess { ReadOnly, ReadWrite, WriteOnly };
struct BufferTy { ScalarTy elem; BufferAccess access; };
struct BufferBindingSlot { std::string name; BufferTy ty; uint32_t position; uint32_t buffer_position; };
struct ScalarPushConstantSlot { std::string name; ScalarTy ty; uint32_t offset; uint32_t member_index; uint32_t position; };
struct ParamBindingPlan {
    std::vector<BufferBindingSlot> buffers;
    std::vector<ScalarPushConstantSlot> scalars;
    uint32_t push_constant_total_bytes = 0;
    // Digest of the plan's fields (the reference hashes the serde_json text with xxh3_64; only
    // equality of keys matters, kernel_handle.rs:216-246).
    uint64_t hash64() const {
        uint64_t h = detail::fnv1a64(&push_constant_total_bytes, 4);
        for (const auto& b : buffers) {
            h = detail::fnv1a64(b.name.data(), b.name.size(), h);
            const uint32_t v[4] = {(uint32_t)b.ty.elem, (uint32_t)b.ty.access, b.position, b.buffer_position};
            h = detail::fnv1a64(v, sizeof v, h);
        }
        for (const auto& s : scalars) {
            h = detail::fnv1a64(s.name.data(), s.name.size(), h);
            const uint32_t v[4] = {(uint32_t)s.ty, s.offset, s.member_index, s.position};
            h = detail::fnv1a64(v, sizeof v, h);
        }
        return h;
    }
};

// The plan `compute_binding_plan` yields for both Q4 kernels (examples/q4km_dequant_matvec.axc:7-12,
// examples/q4_0_dequant_matvec.axc:7-12): q, x, y at bindings 0..2, one u32 push constant.
inline ParamBindingPlan q4_matvec_binding_plan(const std::string& kernel = "q4km_dequant_matvec") {
    ParamBindingPlan p;
    p.buffers = {{"q", {ScalarTy::U8, BufferAccess::ReadOnly}, 0, 0},
                 {"x", {ScalarTy::F32, BufferAccess::ReadOnly}, 1, 1},
                 {"y", {ScalarTy::F32, BufferAccess::ReadWrite}, 2, 2}};
    p.scalars = {{kernel == "q4km_dequant_matvec" ? "n_superblocks" : "n_blocks", ScalarTy::U32, 0, 0, 3}};
    p.push_constant_total_bytes = 4;
    return p;
}

struct KernelCacheKey {   // kernel_handle.rs:44-51
    uint64_t spirv_hash = 0, binding_plan_hash = 0;
    uint32_t push_constant_bytes = 0;
    bool operator==(const KernelCacheKey& o) const {
        return spirv_hash == o.spirv_hash && binding_plan_hash == o.binding_plan_hash &&
               push_constant_bytes == o.push_constant_bytes;
    }
};

// kernel_handle.rs:123-151: Clone = one more reference to the same prepared kernel, Drop = release;
// a handle may outlive the context that prepared it.
class KernelHandle {
public:
    KernelHandle() = default;
    KernelHandle(axc_kernel* k, size_t words) : k_(k), words_(words) {}
    KernelHandle(const KernelHandle& o) : k_(o.k_), words_(o.words_) { if (k_) axc_cuda_kernel_retain(k_); }
    KernelHandle(KernelHandle&& o) noexcept : k_(o.k_), words_(o.words_) { o.k_ = nullptr; }
    KernelHandle& operator=(KernelHandle o) { std::swap(k_, o.k_); std::swap(words_, o.words_); return *this; }
    ~KernelHandle() { if (k_) axc_cuda_kernel_release(k_); }
    size_t spirv_word_count() const { return words_; }
    KernelCacheKey cache_key() const {
        KernelCacheKey key;
        axc_cuda_kernel_cache_key(k_, &key.spirv_hash, &key.binding_plan_hash, &key.push_constant_bytes);
        return key;
    }
    std::vector<uint64_t> buffer_sizes() const {
        uint64_t tmp[16];
        const uint32_t n = axc_cuda_kernel_buffer_sizes(k_, tmp, 16);
        return std::vector<uint64_t>(tmp, tmp + (n < 16 ? n : 16));
    }
    axc_kernel* raw() const { return k_; }
private:
    axc_kernel* k_ = nullptr;
    size_t words_ = 0;
};

struct VulkanContextOptions {   // context.rs:76-109
    std::optional<std::string> pipeline_cache_path;    // accepted and ignored (kernels are compiled ahead of time)
    std::optional<size_t> physical_device_index;       // CUDA ordinal
    std::optional<uint64_t> fence_timeout_ms;
    static VulkanContextOptions from_env() {
        VulkanContextOptions o;
        if (const char* s = std::getenv("AXC_PHYSICAL_DEVICE_INDEX")) o.physical_device_index = std::strtoull(s, nullptr, 10);
        if (const char* s = std::getenv("AXC_FENCE_TIMEOUT_MS")) o.fence_timeout_ms = std::strtoull(s, nullptr, 10);
        return o;
    }
};

struct DispatchRequest {   // dispatch.rs:33-50
    const std::vector<uint32_t>* spirv = nullptr;
    const ParamBindingPlan* binding_plan = nullptr;
    uint32_t workgroups[3] = {1, 1, 1};
    std::vector<std::pair<const void*, size_t>> inputs;
    std::vector<size_t> output_sizes;
    std::vector<uint8_t> push_constants;
    std::string entry_point;
};

class VulkanContext {   // the reference's name; the device behind it is a CUDA GPU
public:
    VulkanContext(const VulkanContext&) = delete;
    VulkanContext& operator=(const VulkanContext&) = delete;
    VulkanContext(VulkanContext&& o) noexcept : ctx_(o.ctx_) { o.ctx_ = nullptr; }
    ~VulkanContext() { if (ctx_) axc_cuda_ctx_destroy(ctx_); }   // waits for the device to go idle

    static Result<VulkanContext> new_() { return new_with_options(VulkanContextOptions::from_env()); }
    static Result<VulkanContext> new_with_options(const VulkanContextOptions& o) {
        axc_ctx_opts c{};
        c.physical_device_index = o.physical_device_index ? (int32_t)*o.physical_device_index : -1;
        c.fence_timeout_ms = o.fence_timeout_ms.value_or(0);
        c.pipeline_cache_path = o.pipeline_cache_path ? o.pipeline_cache_path->c_str() : nullptr;
        axc_ctx* ctx = nullptr;
        const int rc = axc_cuda_ctx_create(&c, &ctx);
        if (rc != AXC_OK) return detail::last_error(rc);
        return VulkanContext(ctx);
    }
    std::string physical_device_name() const {
        const size_t n = axc_cuda_ctx_device_name(ctx_, nullptr, 0);
        std::string s(n + 1, '\0');
        axc_cuda_ctx_device_name(ctx_, s.data(), n + 1);
        s.resize(n);
        return s;
    }
    void max_compute_work_group_count(uint32_t out[3]) const { axc_cuda_ctx_max_grid(ctx_, out); }

    static std::vector<axc_buf_desc> buf_descs(const ParamBindingPlan& plan) {
        std::vector<axc_buf_desc> d(plan.buffers.size());
        for (size_t i = 0; i < d.size(); ++i) {
            const auto& b = plan.buffers[i];
            d[i].elem_ty = b.ty.elem == ScalarTy::U8 ? AXC_TY_U8 : b.ty.elem == ScalarTy::F32 ? AXC_TY_F32
                         : b.ty.elem == ScalarTy::U32 ? AXC_TY_U32 : AXC_TY_OTHER;
            d[i].access = b.ty.access == BufferAccess::ReadOnly ? AXC_ACCESS_READ_ONLY
                        : b.ty.access == BufferAccess::ReadWrite ? AXC_ACCESS_READ_WRITE : AXC_ACCESS_WRITE_ONLY;
            d[i].buffer_position = b.buffer_position, d[i].position = b.position;
        }
        return d;
    }

    // context.rs:392-486.  `spirv` only feeds the cache key: the kernels are compiled ahead of
    // time and selected by `entry_point`.
    Result<KernelHandle> prepare_kernel(const std::vector<uint32_t>& spirv, const ParamBindingPlan& plan,
                                        uint32_t push_constant_total_bytes, const std::string& entry_point) {
        std::vector<axc_buf_desc> d = buf_descs(plan);
        axc_kernel* k = nullptr;
        const int rc = axc_cuda_prepare_kernel(ctx_, entry_point.c_str(), d.data(), (uint32_t)d.size(),
                                               push_constant_total_bytes,
                                               detail::fnv1a64(spirv.data(), spirv.size() * 4), plan.hash64(), &k);
        if (rc != AXC_OK) return detail::last_error(rc);
        return KernelHandle(k, spirv.size());
    }

    // context.rs:498-547: inputs are borrowed for the call and copied; one freshly allocated
    // output per binding, empty where the size is 0; an empty input keeps the device contents.
    Result<std::vector<std::vector<uint8_t>>> dispatch_handle(
        const KernelHandle& h, const uint32_t workgroups[3], const std::vector<std::pair<const void*, size_t>>& inputs,
        const std::vector<size_t>& output_sizes, const std::vector<uint8_t>& push_constants) {
        std::vector<const void*> in_ptrs(inputs.size());
        std::vector<size_t> in_lens(inputs.size());
        for (size_t i = 0; i < inputs.size(); ++i) in_ptrs[i] = inputs[i].first, in_lens[i] = inputs[i].second;
        std::vector<std::vector<uint8_t>> outs(output_sizes.size());
        std::vector<void*> out_ptrs(output_sizes.size());
        for (size_t i = 0; i < outs.size(); ++i) {
            outs[i].resize(output_sizes[i]);
            out_ptrs[i] = outs[i].empty() ? nullptr : outs[i].data();
        }
        const int rc = axc_cuda_dispatch(ctx_, h.raw(), workgroups, in_ptrs.data(), in_lens.data(), (uint32_t)inputs.size(),
                                         out_ptrs.data(), output_sizes.data(), (uint32_t)output_sizes.size(),
                                         push_constants.data(), push_constants.size(), nullptr);
        if (rc != AXC_OK) return detail::last_error(rc);
        return outs;
    }

    // dispatch.rs:109-132: validate (counts, push-constant size, workgroup limits, in that order,
    // before anything is created), prepare, dispatch once, drop the handle.
    Result<std::vector<std::vector<uint8_t>>> dispatch(const DispatchRequest& req) {
        std::vector<axc_buf_desc> d = buf_descs(*req.binding_plan);
        std::vector<const void*> in_ptrs(req.inputs.size());
        std::vector<size_t> in_lens(req.inputs.size());
        for (size_t i = 0; i < req.inputs.size(); ++i) in_ptrs[i] = req.inputs[i].first, in_lens[i] = req.inputs[i].second;
        std::vector<std::vector<uint8_t>> outs(req.output_sizes.size());
        std::vector<void*> out_ptrs(req.output_sizes.size());
        for (size_t i = 0; i < outs.size(); ++i) {
            outs[i].resize(req.output_sizes[i]);
            out_ptrs[i] = outs[i].empty() ? nullptr : outs[i].data();
        }
        const int rc = axc_cuda_dispatch_oneshot(
            ctx_, req.entry_point.c_str(), d.data(), (uint32_t)d.size(), req.binding_plan->push_constant_total_bytes,
            detail::fnv1a64(req.spirv->data(), req.spirv->size() * 4), req.binding_plan->hash64(), req.workgroups,
            in_ptrs.data(), in_lens.data(), (uint32_t)in_ptrs.size(), out_ptrs.data(), req.output_sizes.data(),
            (uint32_t)out_ptrs.size(), req.push_constants.data(), req.push_constants.size(), nullptr);
        if (rc != AXC_OK) return detail::last_error(rc);
        return outs;
    }

    axc_ctx* raw() const { return ctx_; }
private:
    explicit VulkanContext(axc_ctx* c) : ctx_(c) {}
    axc_ctx* ctx_ = nullptr;
};
using CudaContext = VulkanContext;
using CudaContextOptions = VulkanContextOptions;

// ---- metadata sidecar (crates/axc-runtime/src/metadata.rs) ----
// `<output>.axc.meta.json`, schema v1: {schema_version, kernel_name, workgroup_size[3], binding_plan
// {buffers[{name, ty{elem, access}, position, buffer_position}], scalars[{name, ty, offset,
// member_index, position}], push_constant_total_bytes}, push_constant_total_bytes, entry_point};
// enums are serde's external tags ("U8", "F32", "U32", "ReadOnly", ...); source spans are not
// serialised.  load_kernel_metadata reads, parses, then checks the version, in the reference's
// order: MetadataIoError, MetadataParseError, MetadataSchemaMismatch{got, supported} (carried in
// `expected` = supported and `provided` = got).
constexpr uint32_t CURRENT_SCHEMA_VERSION = 1;   // metadata.rs:35

struct KernelMetadata {   // metadata.rs:45-71
    uint32_t schema_version = CURRENT_SCHEMA_VERSION;
    std::string kernel_name;
    uint32_t workgroup_size[3] = {1, 1, 1};
    ParamBindingPlan binding_plan;
    uint32_t push_constant_total_bytes = 0;
    std::string entry_point;
    // metadata.rs:77-92: the version is the current one, the push-constant size the plan's
    static KernelMetadata new_(std::string kernel_name, const uint32_t (&wg)[3], ParamBindingPlan plan,
                               std::string entry_point) {
        KernelMetadata m;
        m.kernel_name = std::move(kernel_name), m.entry_point = std::move(entry_point);
        for (int i = 0; i < 3; ++i) m.workgroup_size[i] = wg[i];
        m.push_constant_total_bytes = plan.push_constant_total_bytes;
        m.binding_plan = std::move(plan);
        return m;
    }
};

namespace detail {
// A JSON value: just enough of a reader for the sidecar (objects, arrays, strings, numbers,
// true / false / null; \uXXXX escapes below 0x80 only, which is all serde_json emits for ASCII names).
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
    const Json* get(const char* key) const {
        for (const auto& kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
};
struct JsonReader {
    const char* p;
    const char* end;
    std::string err;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\r' || *p == '\t')) ++p; }
    bool fail(const char* what) { if (err.empty()) err = what; return false; }
    bool string(std::string& out) {
        if (p >= end || *p != '"') return fail("expected a string");
        ++p;
        while (p < end && *p != '"') {
            char c = *p++;
            if (c == '\\') {
                if (p >= end) return fail("unterminated escape");
                const char e = *p++;
                switch (e) {
                    case 'n': c = '\n'; break; case 't': c = '\t'; break; case 'r': c = '\r'; break;
                    case 'b': c = '\b'; break; case 'f': c = '\f'; break;
                    case '"': case '\\': case '/': c = e; break;
                    case 'u': {
                        if (end - p < 4) return fail("short \\u escape");
                        const unsigned v = (unsigned)std::strtoul(std::string(p, p + 4).c_str(), nullptr, 16);
                        p += 4;
                        if (v >= 0x80) return fail("non-ASCII \\u escape");
                        c = (char)v;
                        break;
                    }
                    default: return fail("bad escape");
                }
            }
            out.push_back(c);
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
    bool value(Json& v, int depth = 0) {
        if (depth > 32) return fail("nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end of input");
        if (*p == '{') {
            v.kind = Json::Obj;
            ++p, ws();
            if (p < end && *p == '}') { ++p; return true; }
            for (;;) {
                ws();
                std::string key;
                if (!string(key)) return false;
                ws();
                if (p >= end || *p != ':') return fail("expected ':'");
                ++p;
                Json child;
                if (!value(child, depth + 1)) return false;
                v.obj.emplace_back(std::move(key), std::move(child));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (*p == '[') {
            v.kind = Json::Arr;
            ++p, ws();
            if (p < end && *p == ']') { ++p; return true; }
            for (;;) {
                Json child;
                if (!value(child, depth + 1)) return false;
                v.arr.push_back(std::move(child));
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (*p == '"') { v.kind = Json::Str; return string(v.str); }
        if (end - p >= 4 && std::strncmp(p, "true", 4) == 0) { v.kind = Json::Bool, v.b = true, p += 4; return true; }
        if (end - p >= 5 && std::strncmp(p, "false", 5) == 0) { v.kind = Json::Bool, p += 5; return true; }
        if (end - p >= 4 && std::strncmp(p, "null", 4) == 0) { p += 4; return true; }
        char* stop = nullptr;
        const std::string tail(p, (size_t)(end - p) < 64 ? (size_t)(end - p) : 64);
        v.num = std::strtod(tail.c_str(), &stop);
        if (stop == tail.c_str()) return fail("unexpected character");
        v.kind = Json::Num;
        p += stop - tail.c_str();
        return true;
    }
};
inline bool json_u32(const Json* j, uint32_t& out) {
    if (!j || j->kind != Json::Num || j->num < 0 || j->num > 4294967295.0 || j->num != (double)(uint64_t)j->num) return false;
    out = (uint32_t)j->num;
    return true;
}
inline bool json_str(const Json* j, std::string& out) {
    if (!j || j->kind != Json::Str) return false;
    out = j->str;
    return true;
}
inline bool scalar_ty_from(const std::string& s, ScalarTy& t) {
    if (s == "U8") t = ScalarTy::U8; else if (s == "F32") t = ScalarTy::F32; else if (s == "U32") t = ScalarTy::U32;
    else t = ScalarTy::Other;   // the other axc-hir scalar types exist; none of this backend's kernels binds them
    return true;
}
inline DispatchError metadata_error(ErrorKind k, std::string msg) {
    DispatchError e;
    e.kind = k, e.message = std::move(msg);
    return e;
}
}  // namespace detail

// metadata.rs:107-122.
inline Result<KernelMetadata> load_kernel_metadata(const std::string& path) {
    using namespace detail;
    std::FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return metadata_error(ErrorKind::MetadataIoError, "metadata I/O error: cannot open " + path);
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, n);
    const bool read_ok = !std::ferror(f);
    std::fclose(f);
    if (!read_ok) return metadata_error(ErrorKind::MetadataIoError, "metadata I/O error: read failed: " + path);

    JsonReader rd{text.data(), text.data() + text.size(), {}};
    Json root;
    bool ok = rd.value(root);
    if (ok) { rd.ws(); if (rd.p != rd.end) ok = rd.fail("trailing characters"); }
    auto parse_error = [&](const std::string& what) {
        return metadata_error(ErrorKind::MetadataParseError, "metadata parse error: " + what);
    };
    if (!ok || root.kind != Json::Obj) return parse_error(ok ? "top level is not an object" : rd.err);
    KernelMetadata m;
    if (!json_u32(root.get("schema_version"), m.schema_version)) return parse_error("missing field `schema_version`");
    if (!json_str(root.get("kernel_name"), m.kernel_name)) return parse_error("missing field `kernel_name`");
    if (!json_str(root.get("entry_point"), m.entry_point)) return parse_error("missing field `entry_point`");
    if (!json_u32(root.get("push_constant_total_bytes"), m.push_constant_total_bytes))
        return parse_error("missing field `push_constant_total_bytes`");
    const Json* wg = root.get("workgroup_size");
    if (!wg || wg->kind != Json::Arr || wg->arr.size() != 3) return parse_error("`workgroup_size` must be an array of 3");
    for (int i = 0; i < 3; ++i)
        if (!json_u32(&wg->arr[i], m.workgroup_size[i])) return parse_error("`workgroup_size` entries must be u32");
    const Json* plan = root.get("binding_plan");
    if (!plan || plan->kind != Json::Obj) return parse_error("missing field `binding_plan`");
    const Json* bufs = plan->get("buffers");
    const Json* scal = plan->get("scalars");
    if (!bufs || bufs->kind != Json::Arr || !scal || scal->kind != Json::Arr ||
        !json_u32(plan->get("push_constant_total_bytes"), m.binding_plan.push_constant_total_bytes))
        return parse_error("`binding_plan` needs buffers, scalars and push_constant_total_bytes");
    for (const Json& b : bufs->arr) {
        BufferBindingSlot s{};
        std::string elem, access;
        const Json* ty = b.get("ty");
        if (b.kind != Json::Obj || !json_str(b.get("name"), s.name) || !ty || !json_str(ty->get("elem"), elem) ||
            !json_str(ty->get("access"), access) || !json_u32(b.get("position"), s.position) ||
            !json_u32(b.get("buffer_position"), s.buffer_position))
            return parse_error("malformed buffer binding slot");
        scalar_ty_from(elem, s.ty.elem);
        if (access == "ReadOnly") s.ty.access = BufferAccess::ReadOnly;
        else if (access == "ReadWrite") s.ty.access = BufferAccess::ReadWrite;
        else if (access == "WriteOnly") s.ty.access = BufferAccess::WriteOnly;
        else return parse_error("unknown variant `" + access + "` of BufferAccess");
        m.binding_plan.buffers.push_back(std::move(s));
    }
    for (const Json& c : scal->arr) {
        ScalarPushConstantSlot s{};
        std::string ty;
        if (c.kind != Json::Obj || !json_str(c.get("name"), s.name) || !json_str(c.get("ty"), ty) ||
            !json_u32(c.get("offset"), s.offset) || !json_u32(c.get("member_index"), s.member_index) ||
            !json_u32(c.get("position"), s.position))
            return parse_error("malformed scalar push-constant slot");
        scalar_ty_from(ty, s.ty);
        m.binding_plan.scalars.push_back(std::move(s));
    }
    if (m.schema_version != CURRENT_SCHEMA_VERSION) {
        DispatchError e = metadata_error(ErrorKind::MetadataSchemaMismatch,
                                         "metadata schema version mismatch: got " + std::to_string(m.schema_version) +
                                             ", supported " + std::to_string(CURRENT_SCHEMA_VERSION));
        e.provided = m.schema_version, e.expected = CURRENT_SCHEMA_VERSION;
        return e;
    }
    return m;
}

inline bool probe_vulkan_available() { return axc_cuda_probe() == 1; }   // icd.rs:22-38
inline bool gpu_tests_enabled() {                                         // icd.rs:40-48
    const char* s = std::getenv("AXC_ENABLE_GPU_TESTS");
    return s && std::strcmp(s, "1") == 0;
}
inline std::string captured_icd_path() { return std::string(); }          // no installable client driver for CUDA

}  // namespace axc
