// Batched Q4_K_M prefill: C[m][n] = sum_k A[m][k] * bf16(W[n][k]), A bf16, fp32 accumulate.
//
// The M > 1 case is a dense contraction, so it runs on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory).  One CTA per 128 weight rows and up to 512
// tokens; the weight rows are the MMA's M dimension (128 TMEM lanes), the tokens its N dimension
// (two instructions of N = 256 -> all 512 TMEM columns), so every superblock is dequantised once.
//
//   warp 0   one thread: TMA loads of the token tile (bf16, 128-byte swizzle) per 64-wide k block
//   warp 1   one thread: issues tcgen05.mma (8 per k block) and the commits that free the stages
//   warp 2   one thread: TMA loads of the raw Q4_K_M superblocks (128 rows x 144 B per superblock
//            column); the whole warp allocates and frees tensor memory
//   warps 3..10  dequantise raw superblocks to bf16 (bit-exact fp32 dequant, round to nearest
//            even) into the K-major 128-byte-swizzled operand tile, then run the epilogue
//            (tcgen05.ld of the accumulators, coalesced stores of C)
//
// Two forms.  Single: one CTA per tile, `tcgen05.mma.cta_group::1`.  Pair (default): two CTAs of
// a cluster work as one 256-row tile with `tcgen05.mma.cta_group::2`: each CTA dequantises its own
// 128 rows and holds half of every 256-token block, so per SM the token loads and the B-operand
// reads are halved (with one CTA the shared-memory port, not the tensor pipe, is the limit).  The
// leader CTA issues the MMAs for both; the peer tells the leader's barriers (remote mbarrier
// arrives) when its tiles are ready, and `tcgen05.commit` with cluster multicast frees the stages
// in both CTAs.  TMA loads are CTA-local in both forms (no multicast loads).
//
// Every wait on an mbarrier is bounded; a wait that runs out sets an error bit and an abort flag,
// all roles fall through to the common exit, outstanding copies are waited for and tensor memory
// is freed.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <mutex>

#include "axc_device.cuh"
#include "axc_kernels.h"

namespace axc {
namespace {

constexpr uint32_t PF_ROWS = 128;                 // weight rows per CTA = MMA M
constexpr uint32_t PF_TOK = 256;                  // tokens per MMA = MMA N
constexpr uint32_t PF_TOK_MAX = 512;              // tokens per CTA (all of tensor memory)
constexpr uint32_t PF_RAW_STAGES = 2;
// Token stages + operand-tile stages share 176 KB: single 2 x 64 KB + 3 x 16 KB; pair 3 x 32 KB +
// 5 x 16 KB (the pair's stage hand-offs cross between two SMs and need the deeper operand ring).
constexpr uint32_t PF_MAX_A_STAGES = 4, PF_MAX_W_STAGES = 5;
constexpr uint32_t PF_W_BYTES = PF_ROWS * 128;                // 128 rows x 64 bf16
constexpr uint32_t PF_RAW_BYTES = PF_ROWS * Q4K_SB_BYTES;     // 18432
constexpr uint32_t PF_OFF_RAW = 180224;
constexpr uint32_t PF_OFF_BAR = PF_OFF_RAW + PF_RAW_STAGES * PF_RAW_BYTES;     // 217088
constexpr uint32_t PF_SMEM = PF_OFF_BAR + 256 + 1024;                          // + alignment slack
constexpr uint32_t PF_DEQ_WARPS = 8;
constexpr uint32_t PF_THREADS = (3 + PF_DEQ_WARPS) * 32;

// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both operands K-major,
// N = 256 (field N >> 3 at bit 17), M = 128 (field M >> 4 at bit 24).
constexpr uint32_t PF_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((PF_TOK >> 3) << 17) | ((PF_ROWS >> 4) << 24);
// the pair form: M = 256 over the two CTAs
constexpr uint32_t PF_IDESC_PAIR = (1u << 4) | (1u << 7) | (1u << 10) | ((PF_TOK >> 3) << 17) | ((256u >> 4) << 24);

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) with the
// 128-byte swizzle: start address / 16, leading offset 1 (unused with a swizzle), stride between
// 8-row groups 1024 B / 16, descriptor version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t sw128_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(PF_IDESC), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(PF_IDESC_PAIR), "r"(accumulate)
        : "memory");
}

// Arrives (once the MMAs issued so far have completed) on the barrier at this shared-memory
// offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"((uint16_t)3)
        : "memory");
}

// Arrive on the barrier at the same offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t cta) {
    asm volatile(
        "{\n\t.reg .b32 r;\n\t"
        "mapa.shared::cluster.u32 r, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [r];\n\t}" ::"r"(smem_u32(bar)),
        "r"(cta)
        : "memory");
}

// Bounded wait that also acquires what other CTAs of the cluster released before arriving.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, uint32_t* err) {
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

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

struct PfBars {
    uint64_t a_full[PF_MAX_A_STAGES], a_empty[PF_MAX_A_STAGES];
    uint64_t w_full[PF_MAX_W_STAGES], w_empty[PF_MAX_W_STAGES];
    uint64_t raw_full[PF_RAW_STAGES], raw_empty[PF_RAW_STAGES];
    uint64_t acc_full;
    uint32_t tmem_base;
    volatile uint32_t abort;
};

template <bool PAIR>
__global__ void __launch_bounds__(PF_THREADS, 1)
q4k_prefill_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                   float* __restrict__ c, uint32_t m_total, uint32_t n_rows, uint32_t n_sb, uint32_t* status,
                   uint32_t independent) {
    // Programmatic dependent launch: the next launch may be scheduled onto SMs this grid leaves
    // idle.  Unless the caller declared this call independent of the one before it (inputs not
    // produced, C not read by it), nothing is read before that call is done, and the next launch is
    // let through only after that wait: a launch scheduled behind an ordered one may read its
    // inputs at once and must find every earlier launch of the stream complete.
    if (!independent) asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t raw_addr = smem_u32(smem_dyn);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;   // the swizzled tiles need 1024-byte alignment
    uint8_t* sm = smem_dyn + (base - raw_addr);
    PfBars* bars = reinterpret_cast<PfBars*>(sm + PF_OFF_BAR);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n0 = blockIdx.x * PF_ROWS;
    const uint32_t m0 = blockIdx.y * PF_TOK_MAX;
    const uint32_t m_count = min(PF_TOK_MAX, m_total - m0);
    const uint32_t halves = (m_count + PF_TOK - 1) / PF_TOK;
    const uint32_t n_kb = n_sb * 4;
    // Pair form: CTA `rank` of the cluster holds tokens [rank * 128, rank * 128 + 128) of every
    // 256-token block; rank 0 (the leader) issues the MMAs.
    constexpr uint32_t A_STAGES = PAIR ? 3u : 2u;
    constexpr uint32_t PF_W_STAGES = PAIR ? 5u : 3u;
    constexpr uint32_t PF_OFF_W = PAIR ? 3u * 32768u : 2u * 65536u;
    static_assert(PF_OFF_W + PF_W_STAGES * PF_W_BYTES == PF_OFF_RAW, "token and operand stages fill the region below the raw tiles");
    constexpr uint32_t A_HALF_BYTES = PAIR ? 128u * 128u : PF_TOK * 128u;   // one block's share per CTA
    constexpr uint32_t A_BYTES = 2u * A_HALF_BYTES;
    uint32_t rank = 0;
    if constexpr (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const bool leader = rank == 0;

    if (tid == 0) {
        // pair: the leader's "full" barriers also count the peer (its relay thread / its dequant warps)
        const uint32_t both = PAIR && leader ? 2u : 1u;
        for (uint32_t s = 0; s < A_STAGES; ++s) mbar_init(&bars->a_full[s], both), mbar_init(&bars->a_empty[s], 1);
        for (uint32_t s = 0; s < PF_W_STAGES; ++s)
            mbar_init(&bars->w_full[s], PF_DEQ_WARPS * both), mbar_init(&bars->w_empty[s], 1);
        for (uint32_t s = 0; s < PF_RAW_STAGES; ++s)
            mbar_init(&bars->raw_full[s], 1), mbar_init(&bars->raw_empty[s], PF_DEQ_WARPS);
        mbar_init(&bars->acc_full, 1);
        bars->abort = 0;
        mbar_init_fence();
    }
    if (warp == 2) {  // tensor memory: all 512 columns (this kernel runs one CTA per SM)
        if constexpr (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(&bars->tmem_base)),
                         "r"(512u)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                             smem_u32(&bars->tmem_base)),
                         "r"(512u)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();   // both CTAs' barriers exist before anyone arrives remotely
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ---------------- token tiles: [tokens][64 k] bf16 per k block ----------------
        if (lane == 0) {
            uint32_t issued = 0;
            for (uint32_t kb = 0; kb < n_kb && !bars->abort; ++kb, ++issued) {
                const uint32_t s = kb % A_STAGES, ph = (kb / A_STAGES) & 1u;
                if (!mbar_wait(&bars->a_empty[s], ph ^ 1u, status)) {
                    bars->abort = 1;
                    break;
                }
                mbar_expect_tx(&bars->a_full[s], halves * A_HALF_BYTES);
                for (uint32_t h = 0; h < halves; ++h)
                    tma_load_2d(base + s * A_BYTES + h * A_HALF_BYTES, &tm_a, (int32_t)(kb * 64u),
                                (int32_t)(m0 + h * PF_TOK + (PAIR ? rank * 128u : 0u)), &bars->a_full[s]);
            }
            // nothing may still be in flight towards this CTA's shared memory at exit
            for (uint32_t j = issued > A_STAGES ? issued - A_STAGES : 0; j < issued; ++j)
                (void)mbar_wait(&bars->a_full[j % A_STAGES], (j / A_STAGES) & 1u, status);
        }
    } else if (warp == 1) {
        // ---------------- MMA issue (pair: the leader issues for both; the peer relays) ----------------
        if (lane == 0 && (!PAIR || leader)) {
            bool ok = true;
            for (uint32_t kb = 0; kb < n_kb && ok && !bars->abort; ++kb) {
                const uint32_t sa = kb % A_STAGES, pa = (kb / A_STAGES) & 1u;
                const uint32_t sw = kb % PF_W_STAGES, pw = (kb / PF_W_STAGES) & 1u;
                if constexpr (PAIR)
                    ok = mbar_wait_cluster(&bars->a_full[sa], pa, status) && mbar_wait_cluster(&bars->w_full[sw], pw, status);
                else
                    ok = mbar_wait(&bars->a_full[sa], pa, status) && mbar_wait(&bars->w_full[sw], pw, status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t wd = sw128_desc(base + PF_OFF_W + sw * PF_W_BYTES);
                for (uint32_t h = 0; h < halves; ++h) {
                    const uint64_t ad = sw128_desc(base + sa * A_BYTES + h * A_HALF_BYTES);
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; ++kk) {  // 16 bf16 = 32 bytes = 2 descriptor units per step
                        if constexpr (PAIR) umma_bf16_pair(tmem + h * PF_TOK, wd + 2u * kk, ad + 2u * kk, (kb | kk) != 0u);
                        else umma_bf16(tmem + h * PF_TOK, wd + 2u * kk, ad + 2u * kk, (kb | kk) != 0u);
                    }
                }
                if constexpr (PAIR) {
                    umma_commit_pair(&bars->a_empty[sa]);   // frees the stages in both CTAs
                    umma_commit_pair(&bars->w_empty[sw]);
                } else {
                    umma_commit(&bars->a_empty[sa]);   // both fire when the MMAs above have read their operands
                    umma_commit(&bars->w_empty[sw]);
                }
            }
            if (!ok) bars->abort = 1;
            if constexpr (PAIR) umma_commit_pair(&bars->acc_full);
            else umma_commit(&bars->acc_full);     // accumulators complete (or nothing outstanding)
        } else if (PAIR && lane == 0) {
            // peer: tell the leader when this CTA's share of the token tile has landed
            for (uint32_t kb = 0; kb < n_kb && !bars->abort; ++kb) {
                const uint32_t sa = kb % A_STAGES, pa = (kb / A_STAGES) & 1u;
                if (!mbar_wait(&bars->a_full[sa], pa, status)) {
                    bars->abort = 1;
                    break;
                }
                mbar_arrive_remote(&bars->a_full[sa], 0u);
            }
        }
    } else if (warp == 2) {
        // ---------------- raw superblocks: 128 rows x 144 bytes per superblock column ----------------
        if (lane == 0) {
            uint32_t issued = 0;
            for (uint32_t sb = 0; sb < n_sb && !bars->abort; ++sb, ++issued) {
                const uint32_t s = sb % PF_RAW_STAGES, ph = (sb / PF_RAW_STAGES) & 1u;
                if (!mbar_wait(&bars->raw_empty[s], ph ^ 1u, status)) {
                    bars->abort = 1;
                    break;
                }
                mbar_expect_tx(&bars->raw_full[s], PF_RAW_BYTES);
                tma_load_2d(base + PF_OFF_RAW + s * PF_RAW_BYTES, &tm_w, (int32_t)(sb * Q4K_SB_BYTES), (int32_t)n0,
                            &bars->raw_full[s]);
            }
            for (uint32_t j = issued > PF_RAW_STAGES ? issued - PF_RAW_STAGES : 0; j < issued; ++j)
                (void)mbar_wait(&bars->raw_full[j % PF_RAW_STAGES], (j / PF_RAW_STAGES) & 1u, status);
        }
    } else {
        // ---------------- dequantise: thread = (row, 16-byte half of the chunk's nibbles) ----------------
        const uint32_t dt = tid - 96u;            // 0..255
        const uint32_t row = dt & 127u, seg = dt >> 7;
        const uint32_t dw = warp - 3u;
        bool ok = true;
        for (uint32_t sb = 0; sb < n_sb && ok; ++sb) {
            const uint32_t sr = sb % PF_RAW_STAGES, pr = (sb / PF_RAW_STAGES) & 1u;
            // every outcome of a wait is made warp-uniform: the code below has warp-wide barriers and loads
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(&bars->raw_full[sr], pr, status) && !bars->abort);
            if (!ok) break;
            const uint8_t* blk = sm + PF_OFF_RAW + sr * PF_RAW_BYTES + row * Q4K_SB_BYTES;
            const uint4 hdr = *reinterpret_cast<const uint4*>(blk);   // d, dmin, 12 scale bytes
            const float d = f16_bits_to_f32(hdr.x & 0xFFFFu), dmin = f16_bits_to_f32(hdr.x >> 16);
#pragma unroll
            for (uint32_t cc = 0; cc < 4; ++cc) {
                const uint32_t kb = sb * 4u + cc;
                const uint32_t sw = kb % PF_W_STAGES, pw = (kb / PF_W_STAGES) & 1u;
                uint32_t sc_pair, m_pair;
                q4k_unpack_pair(hdr.y, hdr.z, hdr.w, (int)cc, sc_pair, m_pair);
                // same operations and rounding points as the reference: d1 = d * sc, m1 = dmin * m,
                // w = d1 * nibble - m1 (no contraction), then bf16 round-to-nearest-even
                const float d1 = __fmul_rn(d, (float)(sc_pair & 0xFFu)), m1 = __fmul_rn(dmin, (float)(m_pair & 0xFFu));
                const float d2 = __fmul_rn(d, (float)(sc_pair >> 8)), m2 = __fmul_rn(dmin, (float)(m_pair >> 8));
                const uint4 qs = *reinterpret_cast<const uint4*>(blk + 16 + cc * 32 + seg * 16);
                const uint32_t qw[4] = {qs.x, qs.y, qs.z, qs.w};
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                        const uint32_t b0 = (qw[j] >> (16 * b)) & 0xFFu, b1 = (qw[j] >> (16 * b + 8)) & 0xFFu;
                        lo[2 * j + b] = pack_bf16x2(__fsub_rn(__fmul_rn(d1, (float)(b0 & 15u)), m1),
                                                    __fsub_rn(__fmul_rn(d1, (float)(b1 & 15u)), m1));
                        hi[2 * j + b] = pack_bf16x2(__fsub_rn(__fmul_rn(d2, (float)(b0 >> 4)), m2),
                                                    __fsub_rn(__fmul_rn(d2, (float)(b1 >> 4)), m2));
                    }
                }
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(&bars->w_empty[sw], pw ^ 1u, status) && !bars->abort);
                if (!ok) break;
                // row `row` of the tile is 128 bytes; its 16-byte chunk j sits at chunk j ^ (row & 7)
                uint8_t* wrow = sm + PF_OFF_W + sw * PF_W_BYTES + row * 128u;
                const uint32_t x7 = row & 7u;
                *reinterpret_cast<uint4*>(wrow + (((2u * seg) ^ x7) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4*>(wrow + (((2u * seg + 1u) ^ x7) << 4)) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                *reinterpret_cast<uint4*>(wrow + (((4u + 2u * seg) ^ x7) << 4)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(wrow + (((5u + 2u * seg) ^ x7) << 4)) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> async proxy (MMA)
                __syncwarp();
                if (lane == 0) {
                    if (PAIR && !leader) mbar_arrive_remote(&bars->w_full[sw], 0u);   // the leader's MMA thread waits
                    else mbar_arrive(&bars->w_full[sw]);
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->raw_empty[sr]);
        }
        if (!ok) bars->abort = 1;

        // ---------------- epilogue: TMEM lane = weight row, column = token ----------------
        ok = __all_sync(0xFFFFFFFFu, mbar_wait(&bars->acc_full, 0u, status) && !bars->abort);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (independent) asm volatile("griddepcontrol.wait;" ::: "memory");   // stream order for the stores of C
        if (ok) {
            const uint32_t quad = warp & 3u;             // the TMEM lanes this warp may read
            const uint32_t col_half = dw / 4u;           // warps 3..6: tokens 0..255, warps 7..10: 256..511
            const uint32_t n = n0 + quad * 32u + lane;
            if (col_half < halves) {
                for (uint32_t cb = 0; cb < PF_TOK; cb += 32u) {
                    const uint32_t mrel = col_half * PF_TOK + cb;
                    if (mrel >= m_count) break;          // warp-uniform
                    uint32_t v[32];
                    const uint32_t taddr = tmem + ((quad * 32u) << 16) + mrel;
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (n < n_rows) {
#pragma unroll
                        for (uint32_t j = 0; j < 32u; ++j)
                            if (mrel + j < m_count)
                                c[(size_t)(m0 + mrel + j) * n_rows + n] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();   // no remote arrive or multicast commit may still target a CTA that left
    if (warp == 2) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }();
    return fn;
}

}  // namespace

cudaError_t launch_q4k_prefill(const uint8_t* q, const uint16_t* a_bf16, float* c, uint32_t m_tokens,
                               uint32_t n_rows, uint32_t n_sb, uint32_t* status, cudaStream_t stream, int form,
                               bool independent) {
    if (m_tokens == 0 || n_rows == 0 || n_sb == 0) return cudaSuccess;
    auto encode = encode_fn();
    if (!encode) return cudaErrorNotSupported;
    const uint32_t tiles = (n_rows + PF_ROWS - 1) / PF_ROWS;
    const bool pair = form != 1 && tiles >= 2;   // form: 0 = choose, 1 = single CTA, 2 = CTA pair
    const uint64_t k = (uint64_t)n_sb * Q4K_SB_ELEMS;
    CUtensorMap tm_a, tm_w;
    {   // tokens: [m_tokens][k] bf16, box = 64 k x 256 (pair: 128) tokens, 128-byte swizzle; rows past
        // the end read as zero
        cuuint64_t dims[2] = {k, m_tokens};
        cuuint64_t strides[1] = {k * 2};
        cuuint32_t box[2] = {64, pair ? 128u : PF_TOK};
        cuuint32_t estr[2] = {1, 1};
        if (encode(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(a_bf16), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    {   // raw weights: [n_rows][n_sb * 144] bytes, box = one superblock x 128 rows
        cuuint64_t dims[2] = {(uint64_t)n_sb * Q4K_SB_BYTES, n_rows};
        cuuint64_t strides[1] = {(uint64_t)n_sb * Q4K_SB_BYTES};
        cuuint32_t box[2] = {Q4K_SB_BYTES, PF_ROWS};
        cuuint32_t estr[2] = {1, 1};
        if (encode(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(q), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    auto kern = pair ? q4k_prefill_kernel<true> : q4k_prefill_kernel<false>;
    {   // raise the dynamic shared-memory limit once per device and kernel form, not on every call
        static std::mutex mu;
        static bool done[64][2] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !done[dev][pair ? 1 : 0]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) done[dev][pair ? 1 : 0] = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    // pair: an even number of CTAs; a trailing CTA without rows of its own still holds its share of the tokens
    cfg.gridDim = dim3(pair ? (tiles + 1u) & ~1u : tiles, (m_tokens + PF_TOK_MAX - 1) / PF_TOK_MAX);
    cfg.blockDim = dim3(PF_THREADS);
    cfg.dynamicSmemBytes = PF_SMEM, cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2, attr[1].val.clusterDim.y = 1, attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr, cfg.numAttrs = pair ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, tm_a, tm_w, c, m_tokens, n_rows, n_sb, status, independent ? 1u : 0u);
}

}  // namespace axc
