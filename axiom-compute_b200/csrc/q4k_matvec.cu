// Q4_K_M dequantise + matrix-vector kernels for sm_100a.
//
// Replaces the reference's single-invocation SPIR-V kernel
// (examples/q4km_dequant_matvec.axc:1-117), generalised from one output to `rows` outputs:
// row r is one reference call on the 144-byte superblocks q[r*n_sb .. (r+1)*n_sb) against the
// shared activation vector x.
//
//  * q4k_matvec_segmented_kernel -- rows longer than 128 superblocks (K > 32768): the row is
//    cut into K segments of 64 superblocks, each staged through shared memory with one bulk
//    async copy per row, and y is accumulated over the segments.  Same arithmetic as the
//    streaming kernel in q4_stream.cu (which serves every shorter row and explains it).
//  * q4k_matvec_seq_kernel -- one thread per row in the reference's exact operation order
//    (separately rounded multiplies and adds); its y is bit-identical to the CPU reference.
//  * q4k_dequant_kernel -- writes the dequantised weights, bit-identical to the reference's
//    d1*nibble - m1f (crates/axc-driver/tests/common_helpers.rs:442-454).
#include "axc_device.cuh"
#include "axc_kernels.h"

namespace axc {

struct Q4kSegParams {
    const uint8_t* q;
    const float* x;
    float* y;
    uint32_t* status;
    uint32_t rows;
    uint32_t n_sb;           // superblocks per row
    uint32_t seg_sb;         // superblocks per K segment (multiple of 8)
    uint32_t n_seg;          // K segments per row
    uint32_t warps_per_row;  // seg_sb / 8
    uint32_t rows_per_pass;  // warps per CTA / warps_per_row
    uint32_t tile_rows;      // rows per stage = PASSES * rows_per_pass
    uint32_t stages;
    uint32_t stage_bytes;    // tile_rows * seg_sb * 144
    uint32_t evict_first;
};

// Dot of one 64-weight chunk with the thread's pre-scaled activations.  `ptr` addresses the
// superblock in shared memory.  Returns this thread's contribution to the row sum.
struct ChunkCtx {
    uint64_t xq[8][4];  // pre-scaled activation pairs, see prologue
    float x_lo_sum, x_hi_sum;
    float rs_a, rs_b;   // 2^(149 - C) split in two representable factors
    int c;
};

__device__ __forceinline__ float q4k_chunk_dot(const uint8_t* ptr, const ChunkCtx& t) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(ptr);
    const uint4 qa = *reinterpret_cast<const uint4*>(ptr + 16 + t.c * 32);
    const uint4 qb = *reinterpret_cast<const uint4*>(ptr + 32 + t.c * 32);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};

    uint64_t acc_lo0 = 0, acc_lo1 = 0, acc_hi0 = 0, acc_hi1 = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t v = w[j];
        const uint32_t u = v >> 8;
        // A nibble n at bit position s, taken as float bits, is exactly n * 2^(s-149).
        ffma2(acc_lo0, pack_u32x2(v & 0x0000000Fu, v & 0x00000F00u), t.xq[j][0]);
        ffma2(acc_lo1, pack_u32x2(v & 0x000F0000u, u & 0x000F0000u), t.xq[j][1]);
        ffma2(acc_hi0, pack_u32x2(v & 0x000000F0u, v & 0x0000F000u), t.xq[j][2]);
        ffma2(acc_hi1, pack_u32x2(v & 0x00F00000u, u & 0x00F00000u), t.xq[j][3]);
    }
    float a0, a1, a2, a3;
    unpack_f32x2(acc_lo0, a0, a1);
    unpack_f32x2(acc_lo1, a2, a3);
    const float s_lo = (((a0 + a1) + (a2 + a3)) * t.rs_a) * t.rs_b;
    unpack_f32x2(acc_hi0, a0, a1);
    unpack_f32x2(acc_hi1, a2, a3);
    const float s_hi = (((a0 + a1) + (a2 + a3)) * t.rs_a) * t.rs_b;

    uint32_t sc_pair, m_pair;
    q4k_unpack_pair(hdr.y, hdr.z, hdr.w, t.c, sc_pair, m_pair);
    const float d = f16_bits_to_f32(hdr.x & 0xFFFFu);
    const float dmin = f16_bits_to_f32(hdr.x >> 16);
    const float d1 = d * (float)(sc_pair & 0xFFu);
    const float d2 = d * (float)(sc_pair >> 8);
    const float m1 = dmin * (float)(m_pair & 0xFFu);
    const float m2 = dmin * (float)(m_pair >> 8);
    float p = d1 * s_lo;
    p = fmaf(-m1, t.x_lo_sum, p);
    p = fmaf(d2, s_hi, p);
    p = fmaf(-m2, t.x_hi_sum, p);
    return p;
}

template <int PASSES>
__global__ void __launch_bounds__(512, 1) q4k_matvec_segmented_kernel(const Q4kSegParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    const uint32_t n_warps = blockDim.x >> 5;

    uint8_t* ring = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * p.stage_bytes);
    float* red = reinterpret_cast<float*>(bars + p.stages);  // [2][n_warps][PASSES]

    // Rows owned by this CTA: an even split, so no CTA has more than one extra row.
    const uint32_t r0 = (uint32_t)(((uint64_t)p.rows * blockIdx.x) / gridDim.x);
    const uint32_t r1 = (uint32_t)(((uint64_t)p.rows * (blockIdx.x + 1)) / gridDim.x);
    const uint32_t my_rows = r1 - r0;
    if (my_rows == 0) return;
    const uint32_t n_tiles = (my_rows + p.tile_rows - 1) / p.tile_rows;
    const uint32_t total_iters = n_tiles * p.n_seg;
    const size_t row_bytes = (size_t)p.n_sb * Q4K_SB_BYTES;
    // Row stride inside a stage: whole rows when there is a single K segment (one bulk copy per
    // tile), else the fixed segment capacity (one bulk copy per row).
    const uint32_t smem_row_stride = (p.n_seg == 1 ? p.n_sb : p.seg_sb) * Q4K_SB_BYTES;

    if (tid == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) mbar_init(&bars[s], 1);
        mbar_init_fence();
    }
    __syncthreads();

    uint64_t policy = 0;
    if (p.evict_first) policy = l2_evict_first_policy();

    // Producer: warp 0 issues the copies for iteration `it` (tile it % n_tiles of segment
    // it / n_tiles) into stage it % stages.
    auto issue = [&](uint32_t it) {
        if (warp != 0 || it >= total_iters) return;
        const uint32_t seg = it / n_tiles, tile = it - seg * n_tiles;
        const uint32_t s = it % p.stages;
        const uint32_t row_begin = r0 + tile * p.tile_rows;
        const uint32_t nrows = min(p.tile_rows, r1 - row_begin);
        uint8_t* dst = ring + (size_t)s * p.stage_bytes;
        if (p.n_seg == 1) {
            if (lane == 0) {
                const uint32_t bytes = nrows * (uint32_t)row_bytes;
                const uint8_t* src = p.q + (size_t)row_begin * row_bytes;
                mbar_expect_tx(&bars[s], bytes);
                if (p.evict_first) bulk_g2s_stream(dst, src, bytes, &bars[s], policy);
                else bulk_g2s(dst, src, bytes, &bars[s]);
            }
        } else {
            const uint32_t seg_len = min(p.seg_sb, p.n_sb - seg * p.seg_sb);
            const uint32_t bytes = seg_len * Q4K_SB_BYTES;
            if (lane == 0) mbar_expect_tx(&bars[s], bytes * nrows);
            __syncwarp();
            for (uint32_t r = lane; r < nrows; r += 32) {
                const uint8_t* src = p.q + (size_t)(row_begin + r) * row_bytes +
                                     (size_t)seg * p.seg_sb * Q4K_SB_BYTES;
                bulk_g2s(dst + (size_t)r * smem_row_stride, src, bytes, &bars[s]);
            }
        }
    };

    // Start the weight stream before touching x: the first `stages` tiles are in flight
    // while the activations are loaded and pre-scaled.
    for (uint32_t it = 0; it < p.stages; ++it) issue(it);

    const uint32_t row_in_pass = warp / p.warps_per_row;
    const uint32_t sb_in_seg = (warp % p.warps_per_row) * 8 + (lane >> 2);
    ChunkCtx ctx;
    ctx.c = lane & 3;
    bool failed = false;

    for (uint32_t seg = 0; seg < p.n_seg; ++seg) {
        const uint32_t sb = seg * p.seg_sb + sb_in_seg;
        const bool active = sb < p.n_sb && row_in_pass < p.rows_per_pass;

        // ---- per-segment prologue: activations of this thread's chunk, pre-scaled ----
        {
            float xv[64];
            if (active) {
                const float4* xp =
                    reinterpret_cast<const float4*>(p.x + (size_t)sb * Q4K_SB_ELEMS + ctx.c * 64);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 v = __ldg(xp + i);
                    xv[4 * i] = v.x, xv[4 * i + 1] = v.y, xv[4 * i + 2] = v.z, xv[4 * i + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) xv[i] = 0.0f;
            }
            float amax = 0.0f, sl = 0.0f, sh = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                sl += xv[i];
                sh += xv[32 + i];
            }
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const float a = fabsf(xv[i]);
                if (a < __int_as_float(0x7F800000) && a > amax) amax = a;  // finite only
            }
            ctx.x_lo_sum = sl;
            ctx.x_hi_sum = sh;
            int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127;
            if (e < -126) e = -126;
            // Products n*x*2^(C-149) sit near 2^-61 for the largest |x|: far from both overflow
            // and the subnormal range whatever the magnitude of the activations.
            const int C = 88 - e;        // in [-39, 214]
            const int C1 = C >> 1;       // both halves are representable powers of two
            const int C2 = C - C1;
            const int R = 149 - C;       // = 61 + e, in [-65, 188]
            const int R1 = R >> 1;
            ctx.rs_a = exp2i(R1);
            ctx.rs_b = exp2i(R - R1);
            const float f1 = exp2i(C1);
            const float g0 = exp2i(C2), g4 = exp2i(C2 - 4), g8 = exp2i(C2 - 8),
                        g12 = exp2i(C2 - 12), g16 = exp2i(C2 - 16), g20 = exp2i(C2 - 20);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                ctx.xq[j][0] = pack_f32x2(xv[4 * j] * f1 * g0, xv[4 * j + 1] * f1 * g8);
                ctx.xq[j][1] = pack_f32x2(xv[4 * j + 2] * f1 * g16, xv[4 * j + 3] * f1 * g16);
                ctx.xq[j][2] = pack_f32x2(xv[32 + 4 * j] * f1 * g4, xv[32 + 4 * j + 1] * f1 * g12);
                ctx.xq[j][3] =
                    pack_f32x2(xv[32 + 4 * j + 2] * f1 * g20, xv[32 + 4 * j + 3] * f1 * g20);
            }
        }

        for (uint32_t tile = 0; tile < n_tiles; ++tile) {
            const uint32_t it = seg * n_tiles + tile;
            const uint32_t s = it % p.stages;
            const uint32_t parity = (it / p.stages) & 1u;
            const uint32_t row_begin = r0 + tile * p.tile_rows;
            const uint32_t nrows = min(p.tile_rows, r1 - row_begin);
            const uint8_t* stage = ring + (size_t)s * p.stage_bytes;

            if (!failed && !mbar_wait(&bars[s], parity, p.status)) failed = true;

            float part[PASSES];
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) {
                const uint32_t r = ps * p.rows_per_pass + row_in_pass;
                float v = 0.0f;
                if (active && r < nrows && !failed)
                    v = q4k_chunk_dot(stage + (size_t)r * smem_row_stride +
                                          (size_t)sb_in_seg * Q4K_SB_BYTES, ctx);
                part[ps] = v;
            }
            // Warp reduction (a warp always lies inside one row).
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) {
                float v = part[ps];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                part[ps] = v;
            }
            float* red_cur = red + (size_t)(it & 1u) * n_warps * PASSES;
            if (lane == 0) {
#pragma unroll
                for (int ps = 0; ps < PASSES; ++ps) red_cur[warp * PASSES + ps] = part[ps];
            }
            __syncthreads();  // stage fully consumed; partials visible
            // Refill this stage for iteration it + stages, then finish the rows of this tile.
            issue(it + p.stages);
            if (tid < nrows) {
                const uint32_t ps = tid / p.rows_per_pass, rp = tid - ps * p.rows_per_pass;
                float sum = 0.0f;
                for (uint32_t wv = 0; wv < p.warps_per_row; ++wv)
                    sum += red_cur[(rp * p.warps_per_row + wv) * PASSES + ps];
                float* yp = p.y + row_begin + tid;
                *yp = (seg == 0) ? sum : (*yp + sum);
            }
        }
    }
}

// ---- reference-order kernel: bit-identical y (common_helpers.rs:411-461) ----
__global__ void q4k_matvec_seq_kernel(const uint8_t* __restrict__ q, const float* __restrict__ x,
                                      float* __restrict__ y, uint32_t rows, uint32_t n_sb) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const uint8_t* row = q + (size_t)r * n_sb * Q4K_SB_BYTES;
    float sum = 0.0f;
    for (uint32_t sb = 0; sb < n_sb; ++sb) {
        const uint4 hdr = *reinterpret_cast<const uint4*>(row + (size_t)sb * Q4K_SB_BYTES);
        const float d = f16_bits_to_f32(hdr.x & 0xFFFFu);
        const float dmin = f16_bits_to_f32(hdr.x >> 16);
        for (int c = 0; c < 4; ++c) {
            uint32_t sc_pair, m_pair;
            q4k_unpack_pair(hdr.y, hdr.z, hdr.w, c, sc_pair, m_pair);
            const float d1 = __fmul_rn(d, (float)(sc_pair & 0xFFu));
            const float m1 = __fmul_rn(dmin, (float)(m_pair & 0xFFu));
            const float d2 = __fmul_rn(d, (float)(sc_pair >> 8));
            const float m2 = __fmul_rn(dmin, (float)(m_pair >> 8));
            const uint8_t* qs = row + (size_t)sb * Q4K_SB_BYTES + 16 + c * 32;
            const float* xs = x + (size_t)sb * Q4K_SB_ELEMS + c * 64;
            for (int l4 = 0; l4 < 8; ++l4) {
                const uint32_t v = *reinterpret_cast<const uint32_t*>(qs + 4 * l4);
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const uint32_t byte = (v >> (8 * b)) & 0xFFu;
                    const int l = 4 * l4 + b;
                    const float lo_f = __fsub_rn(__fmul_rn(d1, (float)(byte & 0xFu)), m1);
                    const float hi_f = __fsub_rn(__fmul_rn(d2, (float)(byte >> 4)), m2);
                    sum = __fadd_rn(sum, __fmul_rn(lo_f, xs[l]));
                    sum = __fadd_rn(sum, __fmul_rn(hi_f, xs[32 + l]));
                }
            }
        }
    }
    y[r] = sum;
}

// ---- bit-exact dequantised weights: one thread per (row, superblock, chunk, 4-byte word) ----
__global__ void q4k_dequant_kernel(const uint8_t* __restrict__ q, float* __restrict__ w,
                                   uint64_t n_words /* rows * n_sb * 32 */) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
        const uint64_t sbi = i >> 5;          // global superblock index
        const uint32_t word = (uint32_t)i & 31u;
        const uint32_t c = word >> 3, l4 = word & 7u;
        const uint8_t* sbp = q + sbi * Q4K_SB_BYTES;
        const uint4 hdr = *reinterpret_cast<const uint4*>(sbp);
        uint32_t sc_pair, m_pair;
        q4k_unpack_pair(hdr.y, hdr.z, hdr.w, (int)c, sc_pair, m_pair);
        const float d = f16_bits_to_f32(hdr.x & 0xFFFFu);
        const float dmin = f16_bits_to_f32(hdr.x >> 16);
        const float d1 = __fmul_rn(d, (float)(sc_pair & 0xFFu));
        const float m1 = __fmul_rn(dmin, (float)(m_pair & 0xFFu));
        const float d2 = __fmul_rn(d, (float)(sc_pair >> 8));
        const float m2 = __fmul_rn(dmin, (float)(m_pair >> 8));
        const uint32_t v = *reinterpret_cast<const uint32_t*>(sbp + 16 + c * 32 + l4 * 4);
        float4 lo, hi;
        lo.x = __fsub_rn(__fmul_rn(d1, (float)(v & 0xFu)), m1);
        hi.x = __fsub_rn(__fmul_rn(d2, (float)((v >> 4) & 0xFu)), m2);
        lo.y = __fsub_rn(__fmul_rn(d1, (float)((v >> 8) & 0xFu)), m1);
        hi.y = __fsub_rn(__fmul_rn(d2, (float)((v >> 12) & 0xFu)), m2);
        lo.z = __fsub_rn(__fmul_rn(d1, (float)((v >> 16) & 0xFu)), m1);
        hi.z = __fsub_rn(__fmul_rn(d2, (float)((v >> 20) & 0xFu)), m2);
        lo.w = __fsub_rn(__fmul_rn(d1, (float)((v >> 24) & 0xFu)), m1);
        hi.w = __fsub_rn(__fmul_rn(d2, (float)(v >> 28)), m2);
        float* out = w + sbi * Q4K_SB_ELEMS + c * 64 + l4 * 4;
        *reinterpret_cast<float4*>(out) = lo;
        *reinterpret_cast<float4*>(out + 32) = hi;
    }
}

// ---------------------------------------------------------------------------------------------

static int round_up8(uint32_t v) { return (int)((v + 7u) & ~7u); }

cudaError_t launch_q4k_matvec_segmented(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                        uint32_t n_sb, uint32_t* status, cudaStream_t stream,
                                        const MatvecTuning& tune, int sm_count, LaunchInfo* info) {
    if (rows == 0 || n_sb == 0) return cudaSuccess;  // caller handles the n = 0 case
    constexpr int kMaxSeg = 128;                     // 16 warps cover 128 superblocks (K = 32768)
    Q4kSegParams p{};
    p.q = q, p.x = x, p.y = y, p.status = status, p.rows = rows, p.n_sb = n_sb;
    const int seg = n_sb <= (uint32_t)kMaxSeg ? round_up8(n_sb) : 64;
    p.seg_sb = (uint32_t)seg;
    p.n_seg = (n_sb + seg - 1) / seg;
    p.warps_per_row = seg / 8;

    // Threads per CTA: fill ~8 warps (or ~16 when one CTA per SM) with whole rows.
    // Two resident CTAs of <= 8 warps each (registers allow 16 warps per SM); rows too long
    // for 8 warps get one 16-warp CTA per SM.
    int ctas_per_sm = tune.ctas_per_sm > 0 ? tune.ctas_per_sm : 2;
    if (p.warps_per_row > 8) ctas_per_sm = 1;
    if (ctas_per_sm > 2) ctas_per_sm = 2;
    int target_warps = ctas_per_sm >= 2 ? 8 : 16;
    int rows_per_pass = target_warps / (int)p.warps_per_row;
    if (rows_per_pass < 1) rows_per_pass = 1;
    int warps = rows_per_pass * (int)p.warps_per_row;
    if (warps > 16) return cudaErrorInvalidConfiguration;
    p.rows_per_pass = (uint32_t)rows_per_pass;

    const size_t seg_bytes = (size_t)seg * Q4K_SB_BYTES;
    const size_t smem_budget = (size_t)(227 * 1024) / ctas_per_sm - 2048;
    int passes = 2;
    if (tune.tile_rows > 0) passes = tune.tile_rows / rows_per_pass;
    if (passes < 1) passes = 1;
    if (passes > 2 && passes < 4) passes = 2;
    if (passes > 4) passes = 4;
    while (passes > 1 && (size_t)passes * rows_per_pass * seg_bytes * 2 > smem_budget) passes >>= 1;
    p.tile_rows = (uint32_t)(passes * rows_per_pass);
    p.stage_bytes = (uint32_t)(p.tile_rows * seg_bytes);
    int stages = tune.stages > 0 ? tune.stages : (int)(smem_budget / p.stage_bytes);
    if (stages < 1) stages = 1;
    if (stages > 32) stages = 32;
    size_t smem = (size_t)stages * p.stage_bytes + (size_t)stages * 8 + (size_t)2 * warps * passes * 4;
    while (stages > 1 && smem > smem_budget) {
        --stages;
        smem = (size_t)stages * p.stage_bytes + (size_t)stages * 8 + (size_t)2 * warps * passes * 4;
    }
    if (smem > (size_t)227 * 1024) return cudaErrorInvalidConfiguration;
    p.stages = (uint32_t)stages;
    p.evict_first = tune.evict_first > 0 ? 1u : 0u;

    // Grid: one CTA per resident slot, but never more CTAs than tiles of work.
    uint32_t grid = (uint32_t)(sm_count * ctas_per_sm);
    const uint32_t max_useful = (rows + (uint32_t)rows_per_pass - 1) / (uint32_t)rows_per_pass;
    if (grid > max_useful) grid = max_useful;
    if (grid < 1) grid = 1;

    void (*kern)(Q4kSegParams) = nullptr;
    switch (passes) {
        case 1: kern = q4k_matvec_segmented_kernel<1>; break;
        case 2: kern = q4k_matvec_segmented_kernel<2>; break;
        default: kern = q4k_matvec_segmented_kernel<4>; break;
    }
    if (!tune.dry_run) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    if (info) {
        info->grid = (int)grid, info->block = warps * 32, info->smem = smem;
        info->tile_rows = (int)p.tile_rows, info->stages = stages, info->seg = seg;
        info->n_seg = (int)p.n_seg;
    }
    if (tune.dry_run) return cudaSuccess;
    kern<<<grid, warps * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_q4k_matvec_seq(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                  uint32_t n_sb, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const int block = 64;
    q4k_matvec_seq_kernel<<<(rows + block - 1) / block, block, 0, stream>>>(q, x, y, rows, n_sb);
    return cudaGetLastError();
}

cudaError_t launch_q4k_dequant(const uint8_t* q, float* w, uint32_t rows, uint32_t n_sb,
                               cudaStream_t stream) {
    const uint64_t n_words = (uint64_t)rows * n_sb * 32;
    if (n_words == 0) return cudaSuccess;
    const int block = 256;
    uint64_t blocks = (n_words + block - 1) / block;
    if (blocks > 148ull * 32) blocks = 148ull * 32;
    q4k_dequant_kernel<<<(unsigned)blocks, block, 0, stream>>>(q, w, n_words);
    return cudaGetLastError();
}

}  // namespace axc
