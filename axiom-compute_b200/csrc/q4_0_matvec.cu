// Q4_0 dequantise + matrix-vector kernels for sm_100a.
//
// Replaces the reference's single-invocation SPIR-V kernel
// (examples/q4_0_dequant_matvec.axc:1-51), generalised to `rows` outputs: row r is one
// reference call on the 18-byte blocks q[r*n_blocks .. (r+1)*n_blocks) against the shared x.
//
//  * q4_0_matvec_stream_kernel -- fast path for an even number of blocks per row (K a multiple
//    of 64) up to 1024 blocks.  The CTA's rows are one contiguous byte range; it is streamed
//    through a shared-memory ring with untiled bulk async copies of the enclosing 16-byte
//    aligned range (18-byte blocks are only 2-byte aligned).  A thread owns one block *pair*
//    position (36 bytes, 4-byte aligned, 64 weights) and keeps its 64 activations in
//    registers, pre-scaled so that masked nibbles feed packed fp32x2 FMAs directly (the
//    Q4_K_M kernel explains the trick).  Per block: d * (sum(q_i x_i) - 8 * sum(x_i)).
//  * q4_0_matvec_rowwarp_kernel -- any n_blocks: a warp per row, plain loads.
//  * q4_0_matvec_seq_kernel -- the reference's exact operation order, bit-identical y
//    (crates/axc-driver/benches/common.rs:224-258).
//  * q4_0_dequant_kernel -- bit-exact weights ((nibble - 8) * d).
#include "axc_device.cuh"
#include "axc_kernels.h"

namespace axc {

struct Q40StreamParams {
    const uint8_t* q;
    const float* x;
    float* y;
    uint32_t* status;
    uint32_t rows;
    uint32_t n_blocks;       // blocks per row (even)
    uint32_t warps_per_row;  // ceil(n_blocks / 64)
    uint32_t rows_per_pass;
    uint32_t tile_rows;
    uint32_t stages;
    uint32_t stage_bytes;    // tile_rows * n_blocks * 18 rounded up to 16, + 16
    uint32_t evict_first;
};

struct PairCtx {
    uint64_t xq[8][4];  // [word 0..3 of block 0, word 0..3 of block 1][pair]
    float xsum0, xsum1;  // 8 * sum of the 32 activations of block 0 / 1
    float rs_a, rs_b;
};

__device__ __forceinline__ void q40_words_dot(const uint32_t* w, const uint64_t (*xq)[4],
                                              uint64_t& acc0, uint64_t& acc1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t v = w[j];
        const uint32_t u = v >> 8;
        ffma2(acc0, pack_u32x2(v & 0x0000000Fu, v & 0x00000F00u), xq[j][0]);
        ffma2(acc1, pack_u32x2(v & 0x000F0000u, u & 0x000F0000u), xq[j][1]);
        ffma2(acc0, pack_u32x2(v & 0x000000F0u, v & 0x0000F000u), xq[j][2]);
        ffma2(acc1, pack_u32x2(v & 0x00F00000u, u & 0x00F00000u), xq[j][3]);
    }
}

// `ptr` (4-byte aligned) addresses a block pair in shared memory.
__device__ __forceinline__ float q40_pair_dot(const uint8_t* ptr, const PairCtx& t) {
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(ptr);
    uint32_t W[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) W[i] = wp[i];
    // block 0: scale = low half of W0, nibble bytes straddle words by 16 bits
    const uint32_t q0[4] = {__funnelshift_r(W[0], W[1], 16), __funnelshift_r(W[1], W[2], 16),
                            __funnelshift_r(W[2], W[3], 16), __funnelshift_r(W[3], W[4], 16)};
    const uint32_t q1[4] = {W[5], W[6], W[7], W[8]};
    uint64_t a0 = 0, a1 = 0, b0 = 0, b1 = 0;
    q40_words_dot(q0, t.xq, a0, a1);
    q40_words_dot(q1, t.xq + 4, b0, b1);
    float f0, f1, f2, f3;
    unpack_f32x2(a0, f0, f1);
    unpack_f32x2(a1, f2, f3);
    const float s0 = (((f0 + f1) + (f2 + f3)) * t.rs_a) * t.rs_b;
    unpack_f32x2(b0, f0, f1);
    unpack_f32x2(b1, f2, f3);
    const float s1 = (((f0 + f1) + (f2 + f3)) * t.rs_a) * t.rs_b;
    const float d0 = f16_bits_to_f32(W[0] & 0xFFFFu);
    const float d1 = f16_bits_to_f32(W[4] >> 16);
    return fmaf(d1, s1 - t.xsum1, d0 * (s0 - t.xsum0));
}

template <int PASSES>
__global__ void __launch_bounds__(512, 1) q4_0_matvec_stream_kernel(const Q40StreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    const uint32_t n_warps = blockDim.x >> 5;

    uint8_t* ring = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * p.stage_bytes);
    float* red = reinterpret_cast<float*>(bars + p.stages);

    const uint32_t r0 = (uint32_t)(((uint64_t)p.rows * blockIdx.x) / gridDim.x);
    const uint32_t r1 = (uint32_t)(((uint64_t)p.rows * (blockIdx.x + 1)) / gridDim.x);
    const uint32_t my_rows = r1 - r0;
    if (my_rows == 0) return;
    const uint32_t n_tiles = (my_rows + p.tile_rows - 1) / p.tile_rows;
    const size_t row_bytes = (size_t)p.n_blocks * Q4_0_BLK_BYTES;

    if (tid == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) mbar_init(&bars[s], 1);
        mbar_init_fence();
    }
    __syncthreads();

    uint64_t policy = 0;
    if (p.evict_first) policy = l2_evict_first_policy();

    auto issue = [&](uint32_t it) {
        if (tid != 0 || it >= n_tiles) return;
        const uint32_t s = it % p.stages;
        const uint32_t row_begin = r0 + it * p.tile_rows;
        const uint32_t nrows = min(p.tile_rows, r1 - row_begin);
        const size_t start = (size_t)row_begin * row_bytes;
        const size_t a_start = start & ~(size_t)15;
        const size_t a_end = (start + (size_t)nrows * row_bytes + 15) & ~(size_t)15;
        const uint32_t bytes = (uint32_t)(a_end - a_start);
        uint8_t* dst = ring + (size_t)s * p.stage_bytes;
        mbar_expect_tx(&bars[s], bytes);
        // The enclosing aligned range stays inside the 16-byte granules that hold valid bytes,
        // so it never leaves the pages of the weight buffer.
        if (p.evict_first) bulk_g2s_stream(dst, p.q + a_start, bytes, &bars[s], policy);
        else bulk_g2s(dst, p.q + a_start, bytes, &bars[s]);
    };
    for (uint32_t it = 0; it < p.stages; ++it) issue(it);

    const uint32_t row_in_pass = warp / p.warps_per_row;
    const uint32_t pair = (warp % p.warps_per_row) * 32 + lane;  // block pair within the row
    const bool active = pair * 2 < p.n_blocks;
    PairCtx ctx;
    {
        float xv[64];
        if (active) {
            const float4* xp = reinterpret_cast<const float4*>(p.x + (size_t)pair * 64);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float4 v = __ldg(xp + i);
                xv[4 * i] = v.x, xv[4 * i + 1] = v.y, xv[4 * i + 2] = v.z, xv[4 * i + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 64; ++i) xv[i] = 0.0f;
        }
        float amax = 0.0f, s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            s0 += xv[i];
            s1 += xv[32 + i];
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            const float a = fabsf(xv[i]);
            if (a < __int_as_float(0x7F800000) && a > amax) amax = a;
        }
        ctx.xsum0 = 8.0f * s0;
        ctx.xsum1 = 8.0f * s1;
        int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127;
        if (e < -126) e = -126;
        const int C = 88 - e, C1 = C >> 1, C2 = C - C1;
        const int R = 149 - C, R1 = R >> 1;
        ctx.rs_a = exp2i(R1);
        ctx.rs_b = exp2i(R - R1);
        const float f1 = exp2i(C1);
        const float g0 = exp2i(C2), g4 = exp2i(C2 - 4), g8 = exp2i(C2 - 8), g12 = exp2i(C2 - 12),
                    g16 = exp2i(C2 - 16), g20 = exp2i(C2 - 20);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* lo = xv + 32 * b + 4 * j;        // low nibbles: elements k
                const float* hi = xv + 32 * b + 16 + 4 * j;   // high nibbles: elements k + 16
                ctx.xq[4 * b + j][0] = pack_f32x2(lo[0] * f1 * g0, lo[1] * f1 * g8);
                ctx.xq[4 * b + j][1] = pack_f32x2(lo[2] * f1 * g16, lo[3] * f1 * g16);
                ctx.xq[4 * b + j][2] = pack_f32x2(hi[0] * f1 * g4, hi[1] * f1 * g12);
                ctx.xq[4 * b + j][3] = pack_f32x2(hi[2] * f1 * g20, hi[3] * f1 * g20);
            }
        }
    }

    bool failed = false;
    for (uint32_t it = 0; it < n_tiles; ++it) {
        const uint32_t s = it % p.stages;
        const uint32_t parity = (it / p.stages) & 1u;
        const uint32_t row_begin = r0 + it * p.tile_rows;
        const uint32_t nrows = min(p.tile_rows, r1 - row_begin);
        const uint32_t delta = (uint32_t)(((size_t)row_begin * row_bytes) & 15);
        const uint8_t* stage = ring + (size_t)s * p.stage_bytes + delta;

        if (!failed && !mbar_wait(&bars[s], parity, p.status)) failed = true;

        float part[PASSES];
#pragma unroll
        for (int ps = 0; ps < PASSES; ++ps) {
            const uint32_t r = ps * p.rows_per_pass + row_in_pass;
            float v = 0.0f;
            if (active && r < nrows && !failed)
                v = q40_pair_dot(stage + (size_t)r * row_bytes + (size_t)pair * 36, ctx);
            part[ps] = v;
        }
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
        __syncthreads();
        issue(it + p.stages);
        if (tid < nrows) {
            const uint32_t ps = tid / p.rows_per_pass, rp = tid - ps * p.rows_per_pass;
            float sum = 0.0f;
            for (uint32_t wv = 0; wv < p.warps_per_row; ++wv)
                sum += red_cur[(rp * p.warps_per_row + wv) * PASSES + ps];
            p.y[row_begin + tid] = sum;
        }
    }
}

// Any n_blocks: one warp per row, lanes stride over blocks, 2-byte loads.
__global__ void q4_0_matvec_rowwarp_kernel(const uint8_t* __restrict__ q,
                                           const float* __restrict__ x, float* __restrict__ y,
                                           uint32_t rows, uint32_t n_blocks) {
    const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint8_t* rp = q + (size_t)row * n_blocks * Q4_0_BLK_BYTES;
    float acc = 0.0f;
    for (uint32_t b = lane; b < n_blocks; b += 32) {
        const uint16_t* hp = reinterpret_cast<const uint16_t*>(rp + (size_t)b * Q4_0_BLK_BYTES);
        const float d = f16_bits_to_f32(hp[0]);
        const float* xs = x + (size_t)b * Q4_0_BLK_ELEMS;
        float s = 0.0f;
#pragma unroll
        for (int k2 = 0; k2 < 8; ++k2) {
            const uint32_t two = hp[1 + k2];
            s = fmaf((float)(two & 0xFu) - 8.0f, xs[2 * k2], s);
            s = fmaf((float)((two >> 4) & 0xFu) - 8.0f, xs[2 * k2 + 16], s);
            s = fmaf((float)((two >> 8) & 0xFu) - 8.0f, xs[2 * k2 + 1], s);
            s = fmaf((float)(two >> 12) - 8.0f, xs[2 * k2 + 17], s);
        }
        acc = fmaf(d, s, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    if (lane == 0) y[row] = acc;
}

__global__ void q4_0_matvec_seq_kernel(const uint8_t* __restrict__ q, const float* __restrict__ x,
                                       float* __restrict__ y, uint32_t rows, uint32_t n_blocks) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const uint8_t* row = q + (size_t)r * n_blocks * Q4_0_BLK_BYTES;
    float acc = 0.0f;
    for (uint32_t b = 0; b < n_blocks; ++b) {
        const uint8_t* bp = row + (size_t)b * Q4_0_BLK_BYTES;
        const float scale = f16_bits_to_f32((uint32_t)bp[0] | ((uint32_t)bp[1] << 8));
        const float* xs = x + (size_t)b * Q4_0_BLK_ELEMS;
        for (int k = 0; k < 16; ++k) {
            const uint32_t packed = bp[2 + k];
            const float w_lo = __fmul_rn(__fsub_rn((float)(packed & 0xFu), 8.0f), scale);
            acc = __fadd_rn(acc, __fmul_rn(w_lo, xs[k]));
            const float w_hi = __fmul_rn(__fsub_rn((float)(packed >> 4), 8.0f), scale);
            acc = __fadd_rn(acc, __fmul_rn(w_hi, xs[k + 16]));
        }
    }
    y[r] = acc;
}

// One thread per (block, byte pair): bit-exact (nibble - 8) * d.
__global__ void q4_0_dequant_kernel(const uint8_t* __restrict__ q, float* __restrict__ w,
                                    uint64_t n_items /* total blocks * 8 */) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_items; i += stride) {
        const uint64_t blk = i >> 3;
        const uint32_t k2 = (uint32_t)i & 7u;
        const uint16_t* hp = reinterpret_cast<const uint16_t*>(q + blk * Q4_0_BLK_BYTES);
        const float d = f16_bits_to_f32(hp[0]);
        const uint32_t two = hp[1 + k2];
        float* out = w + blk * Q4_0_BLK_ELEMS;
        out[2 * k2] = __fmul_rn(__fsub_rn((float)(two & 0xFu), 8.0f), d);
        out[2 * k2 + 16] = __fmul_rn(__fsub_rn((float)((two >> 4) & 0xFu), 8.0f), d);
        out[2 * k2 + 1] = __fmul_rn(__fsub_rn((float)((two >> 8) & 0xFu), 8.0f), d);
        out[2 * k2 + 17] = __fmul_rn(__fsub_rn((float)(two >> 12), 8.0f), d);
    }
}

// ---------------------------------------------------------------------------------------------

cudaError_t launch_q4_0_matvec(const uint8_t* q, const float* x, float* y, uint32_t rows,
                               uint32_t n_blocks, uint32_t* status, cudaStream_t stream,
                               const MatvecTuning& tune, int sm_count, LaunchInfo* info) {
    if (rows == 0 || n_blocks == 0) return cudaSuccess;
    if ((n_blocks & 1u) || n_blocks > 1024u) {
        const int block = 256;  // 8 rows per CTA
        const uint32_t grid = (rows + 7) / 8;
        if (info) info->grid = (int)grid, info->block = block, info->smem = 0;
        q4_0_matvec_rowwarp_kernel<<<grid, block, 0, stream>>>(q, x, y, rows, n_blocks);
        return cudaGetLastError();
    }
    Q40StreamParams p{};
    p.q = q, p.x = x, p.y = y, p.status = status, p.rows = rows, p.n_blocks = n_blocks;
    p.warps_per_row = (n_blocks + 63) / 64;
    // Two resident CTAs of <= 8 warps each (registers allow 16 warps per SM); rows too long
    // for 8 warps get one 16-warp CTA per SM.
    int ctas_per_sm = tune.ctas_per_sm > 0 ? tune.ctas_per_sm : 2;
    if (p.warps_per_row > 8) ctas_per_sm = 1;
    if (ctas_per_sm > 2) ctas_per_sm = 2;
    int target_warps = ctas_per_sm >= 2 ? 8 : 16;
    int rows_per_pass = target_warps / (int)p.warps_per_row;
    if (rows_per_pass < 1) rows_per_pass = 1;
    const int warps = rows_per_pass * (int)p.warps_per_row;
    if (warps > 16) return cudaErrorInvalidConfiguration;
    p.rows_per_pass = (uint32_t)rows_per_pass;
    const size_t row_bytes = (size_t)n_blocks * Q4_0_BLK_BYTES;
    const size_t smem_budget = (size_t)(227 * 1024) / ctas_per_sm - 2048;
    int passes = 2;
    if (tune.tile_rows > 0) passes = tune.tile_rows / rows_per_pass;
    if (passes < 1) passes = 1;
    if (passes > 2 && passes < 4) passes = 2;
    if (passes > 4) passes = 4;
    auto stage_bytes_for = [&](int ps) {
        return (((size_t)ps * rows_per_pass * row_bytes + 15) & ~(size_t)15) + 32;
    };
    while (passes > 1 && stage_bytes_for(passes) * 2 > smem_budget) passes >>= 1;
    p.tile_rows = (uint32_t)(passes * rows_per_pass);
    p.stage_bytes = (uint32_t)stage_bytes_for(passes);
    int stages = tune.stages > 0 ? tune.stages : (int)(smem_budget / p.stage_bytes);
    if (stages < 1) stages = 1;
    if (stages > 32) stages = 32;
    auto smem_for = [&](int st) {
        return (size_t)st * p.stage_bytes + (size_t)st * 8 + (size_t)2 * warps * passes * 4;
    };
    while (stages > 1 && smem_for(stages) > smem_budget) --stages;
    const size_t smem = smem_for(stages);
    if (smem > (size_t)227 * 1024) return cudaErrorInvalidConfiguration;
    p.stages = (uint32_t)stages;
    p.evict_first = tune.evict_first > 0 ? 1u : 0u;
    uint32_t grid = (uint32_t)(sm_count * ctas_per_sm);
    const uint32_t max_useful = (rows + (uint32_t)rows_per_pass - 1) / (uint32_t)rows_per_pass;
    if (grid > max_useful) grid = max_useful;
    if (grid < 1) grid = 1;
    void (*kern)(Q40StreamParams) = nullptr;
    switch (passes) {
        case 1: kern = q4_0_matvec_stream_kernel<1>; break;
        case 2: kern = q4_0_matvec_stream_kernel<2>; break;
        default: kern = q4_0_matvec_stream_kernel<4>; break;
    }
    if (!tune.dry_run) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    if (info) {
        info->grid = (int)grid, info->block = warps * 32, info->smem = smem;
        info->tile_rows = (int)p.tile_rows, info->stages = stages, info->seg = (int)n_blocks;
        info->n_seg = 1;
    }
    if (tune.dry_run) return cudaSuccess;
    kern<<<grid, warps * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_q4_0_matvec_seq(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                   uint32_t n_blocks, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const int block = 64;
    q4_0_matvec_seq_kernel<<<(rows + block - 1) / block, block, 0, stream>>>(q, x, y, rows, n_blocks);
    return cudaGetLastError();
}

cudaError_t launch_q4_0_dequant(const uint8_t* q, float* w, uint32_t rows, uint32_t n_blocks,
                                cudaStream_t stream) {
    const uint64_t n_items = (uint64_t)rows * n_blocks * 8;
    if (n_items == 0) return cudaSuccess;
    const int block = 256;
    uint64_t blocks = (n_items + block - 1) / block;
    if (blocks > 148ull * 32) blocks = 148ull * 32;
    q4_0_dequant_kernel<<<(unsigned)blocks, block, 0, stream>>>(q, w, n_items);
    return cudaGetLastError();
}

}  // namespace axc
