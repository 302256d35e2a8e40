// Q4_0 dequantise + matrix-vector: fallback, reference-order and dequantisation kernels.
//
// The fast path for rows of an even number of blocks up to 1024 is the streaming kernel in
// q4_stream.cu.  Here:
//  * q4_0_matvec_rowwarp_kernel -- any n_blocks: a warp per row, plain loads.
//  * q4_0_matvec_seq_kernel -- the reference's exact operation order, bit-identical y
//    (crates/axc-driver/benches/common.rs:224-258).
//  * q4_0_dequant_kernel -- bit-exact weights ((nibble - 8) * d).
#include "axc_device.cuh"
#include "axc_kernels.h"

namespace axc {

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

cudaError_t launch_q4_0_matvec_rowwarp(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                       uint32_t n_blocks, cudaStream_t stream, LaunchInfo* info) {
    const int block = 256;  // 8 rows per CTA
    const uint32_t grid = (rows + 7) / 8;
    if (info) info->grid = (int)grid, info->block = block, info->smem = 0;
    q4_0_matvec_rowwarp_kernel<<<grid, block, 0, stream>>>(q, x, y, rows, n_blocks);
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
