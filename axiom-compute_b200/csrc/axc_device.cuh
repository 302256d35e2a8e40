// Device-side helpers shared by the sm_100a kernels: block-format constants, the bit-exact
// scale/min unpack, bulk-async-copy (TMA, untiled) and mbarrier wrappers with bounded waits.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace axc {

constexpr int Q4K_SB_BYTES = 144;   // d(f16) dmin(f16) scales[12] qs[128]
constexpr int Q4K_SB_ELEMS = 256;
constexpr int Q4_0_BLK_BYTES = 18;  // d(f16) qs[16]
constexpr int Q4_0_BLK_ELEMS = 32;

// Error bits a kernel may set in its status word (host turns them into typed errors).
constexpr uint32_t ERR_BULK_WAIT_TIMEOUT = 1u;  // an mbarrier wait gave up
constexpr uint32_t ERR_BAD_ARGUMENT = 2u;
constexpr uint32_t ERR_PEER_WAIT_TIMEOUT = 4u;  // a peer's all-gather flag never arrived
constexpr uint32_t ERR_EPOCH_AHEAD = 8u;        // an all-gather word from a later step: storage reused too early

// Spin limit for every mbarrier wait.  try_wait itself blocks for a hardware-defined slice,
// so this is far beyond any legitimate HBM latency yet ends within a fraction of a second.
constexpr uint32_t MBAR_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits16) {
    return __half2float(__ushort_as_half((unsigned short)bits16));
}

// Q4_K scale/min unpack for the sub-block pair (2c, 2c+1) of one superblock, from the three
// little-endian words of the 12-byte scales field (s0 = bytes 0..3, s1 = 4..7, s2 = 8..11).
// Returns sc pair and m pair packed as (value of 2c) | (value of 2c+1) << 8.  Same bits as
// get_scale_min_k4 in the reference (crates/axc-driver/tests/common_helpers.rs:365-381):
//   j <  4: sc = s[j] & 63,                          m = s[j+4] & 63
//   j >= 4: sc = (s[j+4] & 15) | ((s[j-4] >> 6) << 4), m = (s[j+4] >> 4) | ((s[j] >> 6) << 4)
__device__ __forceinline__ void q4k_unpack_pair(uint32_t s0, uint32_t s1, uint32_t s2, int c,
                                                uint32_t& sc_pair, uint32_t& m_pair) {
    const int sh = (c & 1) * 16;
    const uint32_t a = (s0 >> sh) & 0xFFFFu;
    const uint32_t b = (s1 >> sh) & 0xFFFFu;
    const uint32_t e = (s2 >> sh) & 0xFFFFu;
    const bool big = c >= 2;
    sc_pair = big ? ((e & 0x0F0Fu) | ((a >> 2) & 0x3030u)) : (a & 0x3F3Fu);
    m_pair = big ? (((e >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u)) : (b & 0x3F3Fu);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Makes freshly initialised mbarriers visible to the async (TMA) proxy.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

// Bounded wait on phase `parity`.  Returns false (after setting *err) if the limit ran out;
// the caller then skips the work that depended on the data and falls through to the exit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* err) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < MBAR_SPIN_LIMIT; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    if (err) atomicOr(err, ERR_BULK_WAIT_TIMEOUT);
    return false;
}

// Untiled bulk copy global -> shared (TMA engine).  dst, src and bytes are multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Same, with an L2 evict-first policy: weights are streamed once per call.
__device__ __forceinline__ void bulk_g2s_stream(void* dst_smem, const void* src_gmem,
                                                uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Packed fp32x2 FMA (two independent fp32 FMAs per instruction on sm_100): acc += a * b.
__device__ __forceinline__ void ffma2(uint64_t& acc, uint64_t a, uint64_t b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}

__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// 2^k as a float for k in [-126, 127].
__device__ __forceinline__ float exp2i(int k) { return __int_as_float((k + 127) << 23); }

}  // namespace axc
