// Tests of the C++ host mirror (include/axc_runtime.hpp), written the way the reference's own
// runtime tests are (crates/axc-runtime/tests/: AT-506a/517/518 typed errors before any device
// work, AT-805 handle reuse, AT-827 handle outlives context, AT-1324 parity on the LCG fixture).
//   runtime_test            host-only part: runs anywhere (no GPU: bring-up must fail with
//                           NoSupportedDevice, never a crash, never a CPU fallback)
//   runtime_test --gpu E F  the device part; E = expected value, F = fixture file (both made by
//                           the caller with the CPU oracle)
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "axc_runtime.hpp"

#define CHECK(cond)                                                                   \
    do {                                                                              \
        if (!(cond)) {                                                                \
            std::fprintf(stderr, "CHECK failed at line %d: %s\n", __LINE__, #cond);   \
            return 1;                                                                 \
        }                                                                             \
    } while (0)

// q (n * 144 bytes) followed by x (n * 256 floats): the reference's LCG fixture, written by the
// caller (tests/test_cpp_mirror.py generates it with the CPU oracle).
static bool read_fixture(const char* path, uint32_t n, std::vector<uint8_t>& q, std::vector<float>& x) {
    std::FILE* f = std::fopen(path, "rb");
    if (!f) return false;
    q.resize((size_t)n * 144), x.resize((size_t)n * 256);
    const bool ok = std::fread(q.data(), 1, q.size(), f) == q.size() && std::fread(x.data(), 4, x.size(), f) == x.size();
    std::fclose(f);
    return ok;
}

static bool write_text(const char* path, const char* text) {
    std::FILE* f = std::fopen(path, "wb");
    if (!f) return false;
    const bool ok = std::fputs(text, f) >= 0;
    std::fclose(f);
    return ok;
}

// metadata.rs tests: round trip of a v1 sidecar, other versions rejected with got / supported,
// malformed text and a missing file are typed errors.
static int metadata_cases(const char* dir) {
    using namespace axc;
    const std::string base = std::string(dir) + "/axc_meta_test";
    const char* good =
        "{\n  \"schema_version\": 1,\n  \"kernel_name\": \"q4km_dequant_matvec\",\n  \"workgroup_size\": [64, 1, 1],\n"
        "  \"binding_plan\": {\"buffers\": ["
        "{\"name\": \"q\", \"ty\": {\"elem\": \"U8\", \"access\": \"ReadOnly\"}, \"position\": 0, \"buffer_position\": 0},"
        "{\"name\": \"x\", \"ty\": {\"elem\": \"F32\", \"access\": \"ReadOnly\"}, \"position\": 1, \"buffer_position\": 1},"
        "{\"name\": \"y\", \"ty\": {\"elem\": \"F32\", \"access\": \"ReadWrite\"}, \"position\": 2, \"buffer_position\": 2}],"
        " \"scalars\": [{\"name\": \"n_superblocks\", \"ty\": \"U32\", \"offset\": 0, \"member_index\": 0, \"position\": 3}],"
        " \"push_constant_total_bytes\": 4},\n  \"push_constant_total_bytes\": 4,\n  \"entry_point\": \"q4km_dequant_matvec\"\n}\n";
    CHECK(write_text((base + ".json").c_str(), good));
    auto r = load_kernel_metadata(base + ".json");
    CHECK(r.is_ok());
    const KernelMetadata& m = r.unwrap();
    CHECK(m.schema_version == CURRENT_SCHEMA_VERSION && m.kernel_name == "q4km_dequant_matvec" && m.entry_point == m.kernel_name);
    CHECK(m.workgroup_size[0] == 64 && m.workgroup_size[1] == 1 && m.workgroup_size[2] == 1 && m.push_constant_total_bytes == 4);
    CHECK(m.binding_plan.hash64() == q4_matvec_binding_plan().hash64());   // the plan both Q4 kernels compile to
    const uint32_t wg[3] = {64, 1, 1};
    const KernelMetadata made = KernelMetadata::new_("k", wg, q4_matvec_binding_plan(), "k");
    CHECK(made.schema_version == 1 && made.push_constant_total_bytes == 4);

    std::string v2 = good;
    v2.replace(v2.find("\"schema_version\": 1"), 19, "\"schema_version\": 2");
    CHECK(write_text((base + "_v2.json").c_str(), v2.c_str()));
    auto r2 = load_kernel_metadata(base + "_v2.json");
    CHECK(r2.is_err() && r2.unwrap_err().kind == ErrorKind::MetadataSchemaMismatch);
    CHECK(r2.unwrap_err().provided == 2 && r2.unwrap_err().expected == 1);

    CHECK(write_text((base + "_bad.json").c_str(), "{\"schema_version\": 1, \"kernel_name\": "));
    auto r3 = load_kernel_metadata(base + "_bad.json");
    CHECK(r3.is_err() && r3.unwrap_err().kind == ErrorKind::MetadataParseError);
    std::string noentry = good;
    noentry.replace(noentry.find("\"entry_point\""), 13, "\"entry_pointx\"");
    CHECK(write_text((base + "_noentry.json").c_str(), noentry.c_str()));
    auto r4 = load_kernel_metadata(base + "_noentry.json");
    CHECK(r4.is_err() && r4.unwrap_err().kind == ErrorKind::MetadataParseError);
    auto r5 = load_kernel_metadata(base + "_does_not_exist.json");
    CHECK(r5.is_err() && r5.unwrap_err().kind == ErrorKind::MetadataIoError);
    for (const char* suffix : {".json", "_v2.json", "_bad.json", "_noentry.json"}) std::remove((base + suffix).c_str());
    return 0;
}

static int host_only() {
    using namespace axc;
    {
        const char* tmp = std::getenv("TMPDIR");
        if (metadata_cases(tmp && *tmp ? tmp : "/tmp") != 0) return 1;
    }
    CHECK(kDispatchErrorVariantCount == 25);
    const ParamBindingPlan plan = q4_matvec_binding_plan();
    CHECK(plan.buffers.size() == 3 && plan.scalars.size() == 1 && plan.push_constant_total_bytes == 4);
    CHECK(plan.buffers[0].ty.elem == ScalarTy::U8 && plan.buffers[2].ty.access == BufferAccess::ReadWrite);
    CHECK(plan.hash64() == q4_matvec_binding_plan().hash64());
    CHECK(plan.hash64() != q4_matvec_binding_plan("q4_0_dequant_matvec").hash64());
    CHECK(captured_icd_path().empty());
    if (!probe_vulkan_available()) {
        auto r = VulkanContext::new_with_options(VulkanContextOptions{});
        CHECK(r.is_err());
        CHECK(r.unwrap_err().kind == ErrorKind::NoSupportedDevice);   // typed failure, no CPU fallback
        std::printf("host-only ok (no device: bring-up fails with NoSupportedDevice)\n");
    } else {
        std::printf("host-only ok (a device is present)\n");
    }
    return 0;
}

static int with_gpu(double expected, const char* fixture_path) {
    using namespace axc;
    CHECK(probe_vulkan_available());
    auto cr = VulkanContext::new_with_options(VulkanContextOptions{});
    CHECK(cr.is_ok());
    VulkanContext ctx = std::move(cr.unwrap());
    CHECK(ctx.physical_device_name().find("B200") != std::string::npos);
    uint32_t lim[3];
    ctx.max_compute_work_group_count(lim);
    CHECK(lim[0] == 2147483647u && lim[1] == 65535u && lim[2] == 65535u);

    const ParamBindingPlan plan = q4_matvec_binding_plan();
    const std::vector<uint32_t> spirv = {0x07230203u, 0x00010300u, 0, 1, 0};
    const uint32_t n = 128;
    std::vector<uint8_t> q;
    std::vector<float> x;
    CHECK(read_fixture(fixture_path, n, q, x));
    const std::vector<uint8_t> pc = {(uint8_t)n, 0, 0, 0};
    const uint32_t wg[3] = {1, 1, 1};
    const float zero = 0.0f;

    // typed errors before any device work, in the reference's order (dispatch.rs:60-92)
    {
        DispatchRequest req;
        req.spirv = &spirv, req.binding_plan = &plan, req.entry_point = "q4km_dequant_matvec";
        req.inputs = {{q.data(), q.size()}, {x.data(), x.size() * 4}};   // one input short
        req.output_sizes = {0, 0, 4}, req.push_constants = pc;
        auto r = ctx.dispatch(req);
        CHECK(r.is_err() && r.unwrap_err().kind == ErrorKind::BindingCountMismatch);
        CHECK(r.unwrap_err().expected == 3 && r.unwrap_err().provided == 2);
        req.inputs.push_back({&zero, 4});
        req.push_constants = {1, 0, 0};
        r = ctx.dispatch(req);
        CHECK(r.is_err() && r.unwrap_err().kind == ErrorKind::PushConstantSizeMismatch);
        req.push_constants = pc;
        req.workgroups[1] = 70000;
        r = ctx.dispatch(req);
        CHECK(r.is_err() && r.unwrap_err().kind == ErrorKind::WorkgroupCountExceedsDeviceLimit);
        CHECK(r.unwrap_err().requested[1] == 70000 && r.unwrap_err().max[1] == 65535);
        req.workgroups[1] = 1;
        req.entry_point = "saxpy";
        r = ctx.dispatch(req);
        CHECK(r.is_err() && r.unwrap_err().kind == ErrorKind::PipelineCreationFailed);
        CHECK(r.unwrap_err().message.find("unsupported kernel for CUDA backend") != std::string::npos);
        // one-shot dispatch of the reference's own shape (AT-1324): one output, n = 128
        req.entry_point = "q4km_dequant_matvec";
        r = ctx.dispatch(req);
        CHECK(r.is_ok());
        float y;
        std::memcpy(&y, r.unwrap()[2].data(), 4);
        CHECK(r.unwrap()[0].empty() && r.unwrap()[1].empty() && r.unwrap()[2].size() == 4);
        CHECK(std::fabs((double)y - expected) <= 1e-5 * std::fabs(expected));
    }

    // prepare once, dispatch many (AT-805 / AT-816); same key -> same prepared kernel
    auto hr = ctx.prepare_kernel(spirv, plan, 4, "q4km_dequant_matvec");
    CHECK(hr.is_ok());
    KernelHandle h = hr.unwrap();
    auto h2 = ctx.prepare_kernel(spirv, plan, 4, "q4km_dequant_matvec");
    CHECK(h2.is_ok() && h2.unwrap().raw() == h.raw() && h2.unwrap().cache_key() == h.cache_key());
    CHECK(h.spirv_word_count() == spirv.size() && h.cache_key().push_constant_bytes == 4);
    auto out = ctx.dispatch_handle(h, wg, {{q.data(), q.size()}, {x.data(), x.size() * 4}, {&zero, 4}}, {0, 0, 4}, pc);
    CHECK(out.is_ok());
    float y1;
    std::memcpy(&y1, out.unwrap()[2].data(), 4);
    CHECK(std::fabs((double)y1 - expected) <= 1e-5 * std::fabs(expected));
    const auto sizes = h.buffer_sizes();
    CHECK(sizes.size() == 3 && sizes[0] == 32768 && sizes[1] == 131072 && sizes[2] == 4);   // round_up_pow2
    // empty inputs keep the device contents (resident weights)
    out = ctx.dispatch_handle(h, wg, {{nullptr, 0}, {nullptr, 0}, {nullptr, 0}}, {0, 0, 4}, pc);
    CHECK(out.is_ok());
    float y2;
    std::memcpy(&y2, out.unwrap()[2].data(), 4);
    CHECK(y2 == y1);

    // rows from the grid: 64 copies of the fixture row, resident after the first call; the calls with an
    // empty q take the single-launch path (x read from host memory by the kernel, completion polled):
    // every row must give the fixture's value, call after call, also after x changes
    {
        const uint32_t rows = 64;
        std::vector<uint8_t> q64((size_t)rows * q.size());
        for (uint32_t r = 0; r < rows; ++r) std::memcpy(q64.data() + (size_t)r * q.size(), q.data(), q.size());
        const uint32_t wg64[3] = {rows, 1, 1};
        auto hr64 = ctx.prepare_kernel({0x07230203u, 64u}, plan, 4, "q4km_dequant_matvec");
        CHECK(hr64.is_ok());
        KernelHandle h64 = hr64.unwrap();
        auto o64 = ctx.dispatch_handle(h64, wg64, {{q64.data(), q64.size()}, {x.data(), x.size() * 4}, {nullptr, 0}},
                                       {0, 0, (size_t)rows * 4}, pc);
        CHECK(o64.is_ok());
        std::vector<float> x2(x);
        for (int it = 0; it < 6; ++it) {
            const float scale = it % 2 ? 0.5f : 1.0f;
            for (size_t i = 0; i < x.size(); ++i) x2[i] = x[i] * scale;
            o64 = ctx.dispatch_handle(h64, wg64, {{nullptr, 0}, {x2.data(), x2.size() * 4}, {nullptr, 0}},
                                      {0, 0, (size_t)rows * 4}, pc);
            CHECK(o64.is_ok() && o64.unwrap()[2].size() == (size_t)rows * 4);
            for (uint32_t r = 0; r < rows; ++r) {
                float yr;
                std::memcpy(&yr, o64.unwrap()[2].data() + 4 * r, 4);
                CHECK(std::fabs((double)yr - expected * scale) <= 1e-5 * std::fabs(expected * scale));
            }
        }
    }

    // a clone keeps the kernel usable after the context is gone (AT-827): release must not crash
    KernelHandle survivor = h;
    {
        VulkanContext moved = std::move(ctx);
    }
    CHECK(survivor.cache_key() == h.cache_key());
    std::printf("gpu ok: y = %.6f (expected %.6f)\n", y1, expected);
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 4 && std::strcmp(argv[1], "--gpu") == 0) return with_gpu(std::atof(argv[2]), argv[3]);
    return host_only();
}
