// Q4_K_M dequantise + matrix-vector, streaming kernel for sm_100a (rows of up to 128
// superblocks, i.e. K <= 32768; longer rows take the K-segmented kernel in q4k_matvec.cu).
//
// Replaces examples/q4km_dequant_matvec.axc:1-117 for `rows` outputs at once.
//
// Data movement.  A CTA owns a contiguous range of rows, i.e. one contiguous byte range of q.
// Thread 0 starts untiled bulk async copies (TMA engine) of that range into a shared-memory
// ring, one mbarrier per stage, before anything else happens; when the ring is as large as the
// CTA's share (the 14336 x 4096 case: 48-49 rows = 112 KB per CTA, two CTAs per SM) the whole
// matrix is in flight from the first cycles of the kernel and no stage is ever refilled.
// Otherwise stages are recycled: every warp arrives on the stage's "empty" mbarrier when it has
// read it, and the warp that observes the phase complete re-arms and refills it.  There is no
// CTA-wide barrier in the loop; warps run ahead independently.
//
// Arithmetic.  A thread owns one 64-weight chunk position (superblock s, chunk c: 32 bytes of
// nibbles, sub-blocks 2c and 2c+1) for the life of the CTA and keeps the 64 activations it
// needs in registers as 32 fp32 pairs, each pre-multiplied by a power of two.  The 32 bytes are
// read as four 64-bit words; `word & 0x0000000F0000000F` (two LOP3, result already a register
// pair) isolates the same nibble of two 32-bit halves, and those bits, read as fp32, are
// exactly nibble * 2^(pos-149).  The pair goes straight into a packed fma.rn.f32x2 against the
// matching activation pair: one LOP3 and half an FMA instruction per weight, no int-to-float
// conversion, no register moves, products exact.  Per sub-block the algebraically equal form
// d*sc*sum(q_i x_i) - dmin*m*sum(x_i) is used, so weights are never materialised here (the
// bit-exact dequantised values come from q4k_dequant_kernel, which shares q4k_unpack_pair).
// Row sums: transposed warp-shuffle reduction, per-warp partials in shared memory, one fixed-
// order combine per CTA at the end (deterministic).
//
// With programmatic dependent launch the next call's CTAs may be scheduled while this call
// drains; `griddepcontrol.wait` comes before x is read, the weight stream started or y written.
#include "axc_device.cuh"
#include "axc_kernels.h"

#ifdef AXC_TRACE
__device__ unsigned long long g_axc_trace[2048 * 24];
#define TRACE(slot) do { if (tid == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_axc_trace[blockIdx.x * 24 + (slot)] = t_; } } while (0)
extern "C" int axc_debug_copy_trace(unsigned long long* dst, int n) {
    return (int)cudaMemcpyFromSymbol(dst, g_axc_trace, sizeof(unsigned long long) * n);
}
#else
#define TRACE(slot) do { } while (0)
#endif

namespace axc {

struct Q4kStreamParams {
    const uint8_t* q;
    const float* x;
    float* y;
    uint32_t* status;
    uint32_t rows;
    uint32_t n_sb;
    uint32_t warps_per_row;  // ceil(n_sb / 8)
    uint32_t rows_per_pass;  // warps per CTA / warps_per_row
    uint32_t tile_rows;      // PASSES * rows_per_pass
    uint32_t stages;
    uint32_t stage_bytes;    // tile_rows * n_sb * 144
    uint32_t ring_bytes;     // stages * stage_bytes, or the CTA's exact share when all resident
    uint32_t part_entries;   // capacity of the partial-sum array (>= rows per CTA * warps_per_row)
    uint32_t evict_first;
    uint32_t prefetch_first; // start the weight stream before griddepcontrol.wait
    uint32_t x_pitch;        // positions (4 per superblock) rounded up to 8
    uint32_t rows_base;      // rows / grid
    uint32_t rows_rem;       // rows % grid: the first rows_rem CTAs take one row more
    uint32_t tiles_lo, tiles_hi;  // tiles of a CTA with rows_base / rows_base + 1 rows
    uint32_t xs_offset;      // byte offset of the staged activations in shared memory
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Per-thread constants: the chunk's 64 activations as pre-scaled pairs, and the header decode
// selectors for chunk c.
struct LaneCtx {
    uint64_t xl[4][4];  // [64-bit word k][byte b]: low-nibble columns (8k+b, 8k+4+b)
    uint64_t xh[4][4];  // high-nibble columns (32+8k+b, 32+8k+4+b)
    float x_lo_sum, x_hi_sum;
    float rs_a, rs_b;   // 2^(149 - C) as two representable factors
    uint32_t sh0, sh_m, sh2, mask_a, mask_b;  // scale/min unpack selectors
    bool big;
};

__device__ __forceinline__ float q4k_chunk_dot64(const uint8_t* sb_ptr, uint32_t qs_off,
                                                 const LaneCtx& t) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(sb_ptr);
    const ulonglong2 qa = *reinterpret_cast<const ulonglong2*>(sb_ptr + qs_off);
    const ulonglong2 qb = *reinterpret_cast<const ulonglong2*>(sb_ptr + qs_off + 16);
    const uint64_t w[4] = {qa.x, qa.y, qb.x, qb.y};

    uint64_t al0 = 0, al1 = 0, ah0 = 0, ah1 = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint64_t v = w[k];
        const uint64_t u = v >> 8;  // byte 3 of each half down to bits 16..23
        ffma2(al0, v & 0x0000000F0000000FULL, t.xl[k][0]);
        ffma2(ah0, v & 0x000000F0000000F0ULL, t.xh[k][0]);
        ffma2(al1, v & 0x00000F0000000F00ULL, t.xl[k][1]);
        ffma2(ah1, v & 0x0000F0000000F000ULL, t.xh[k][1]);
        ffma2(al0, v & 0x000F0000000F0000ULL, t.xl[k][2]);
        ffma2(ah0, v & 0x00F0000000F00000ULL, t.xh[k][2]);
        ffma2(al1, u & 0x000F0000000F0000ULL, t.xl[k][3]);
        ffma2(ah1, u & 0x00F0000000F00000ULL, t.xh[k][3]);
    }
    float a0, a1, a2, a3;
    unpack_f32x2(al0, a0, a1);
    unpack_f32x2(al1, a2, a3);
    const float s_lo = (a0 + a1) + (a2 + a3);  // sum(q_i x_i) * 2^(C-149), sub-block 2c
    unpack_f32x2(ah0, a0, a1);
    unpack_f32x2(ah1, a2, a3);
    const float s_hi = (a0 + a1) + (a2 + a3);  // sub-block 2c+1

    // get_scale_min_k4 for sub-blocks 2c, 2c+1 with per-lane selectors (same bits as
    // q4k_unpack_pair; crates/axc-driver/tests/common_helpers.rs:365-381).
    const uint32_t wa_sc = t.big ? hdr.w : hdr.y;
    const uint32_t wa_m = t.big ? hdr.w : hdr.z;
    const uint32_t sc_pair = ((wa_sc >> t.sh0) & t.mask_a) | ((hdr.y >> t.sh2) & t.mask_b);
    const uint32_t m_pair = ((wa_m >> t.sh_m) & t.mask_a) | ((hdr.z >> t.sh2) & t.mask_b);
    const float d = f16_bits_to_f32(hdr.x & 0xFFFFu);
    const float dmin = f16_bits_to_f32(hdr.x >> 16);
    // d * (sc0 * S_lo + sc1 * S_hi) - dmin * (m0 * sum_lo(x) + m1 * sum_hi(x))
    float t1 = (float)(sc_pair & 0xFFu) * s_lo;
    t1 = fmaf((float)(sc_pair >> 8), s_hi, t1);
    float t2 = (float)(m_pair & 0xFFu) * t.x_lo_sum;
    t2 = fmaf((float)(m_pair >> 8), t.x_hi_sum, t2);
    t1 = (t1 * t.rs_a) * t.rs_b;  // back to true scale (two exact power-of-two steps)
    return fmaf(-dmin, t2, d * t1);
}

// Sum each of the PASSES per-lane values over the warp; afterwards lane (8 * i) holds the total
// of value i (PASSES = 4), lanes 0 / 16 (PASSES = 2) or lane 0 (PASSES = 1).
template <int PASSES>
__device__ __forceinline__ float warp_reduce_transposed(const float (&v)[PASSES], uint32_t lane) {
    constexpr uint32_t FULL = 0xFFFFFFFFu;
    float r;
    if constexpr (PASSES == 4) {
        const bool hi16 = lane & 16u;
        const float k0 = hi16 ? v[2] : v[0], k1 = hi16 ? v[3] : v[1];
        const float s0 = hi16 ? v[0] : v[2], s1 = hi16 ? v[1] : v[3];
        const float b0 = k0 + __shfl_xor_sync(FULL, s0, 16);
        const float b1 = k1 + __shfl_xor_sync(FULL, s1, 16);
        const bool hi8 = lane & 8u;
        r = (hi8 ? b1 : b0) + __shfl_xor_sync(FULL, hi8 ? b0 : b1, 8);
    } else if constexpr (PASSES == 2) {
        const bool hi16 = lane & 16u;
        r = (hi16 ? v[1] : v[0]) + __shfl_xor_sync(FULL, hi16 ? v[0] : v[1], 16);
        r += __shfl_xor_sync(FULL, r, 8);
    } else {
        r = v[0] + __shfl_xor_sync(FULL, v[0], 16);
        r += __shfl_xor_sync(FULL, r, 8);
    }
    r += __shfl_xor_sync(FULL, r, 4);
    r += __shfl_xor_sync(FULL, r, 2);
    r += __shfl_xor_sync(FULL, r, 1);
    return r;
}

template <int PASSES>
__global__ void __launch_bounds__(512, 1) q4k_matvec_stream_kernel(const Q4kStreamParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    const uint32_t n_warps = blockDim.x >> 5;

    uint8_t* ring = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.ring_bytes);
    uint64_t* empty = full + p.stages;
    uint32_t* claim = reinterpret_cast<uint32_t*>(empty + p.stages);
    float* part = reinterpret_cast<float*>(claim + p.stages);
    float4* xs = reinterpret_cast<float4*>(smem + p.xs_offset);  // [16][x_pitch] float4

    // Let the next grid in the stream begin its own prologue as early as the hardware allows.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    TRACE(0);

    // Rows owned by this CTA: an even split computed on the host (no CTA has more than one
    // extra row).
    const uint32_t bid = blockIdx.x;
    const uint32_t r0 = bid * p.rows_base + min(bid, p.rows_rem);
    const uint32_t my_rows = p.rows_base + (bid < p.rows_rem ? 1u : 0u);
    const uint32_t r1 = r0 + my_rows;
    if (my_rows == 0) return;
    const uint32_t n_tiles = bid < p.rows_rem ? p.tiles_hi : p.tiles_lo;
    const uint32_t row_bytes = p.n_sb * Q4K_SB_BYTES;

    const uint32_t row_in_pass = warp / p.warps_per_row;
    const uint32_t warp_in_row = warp - row_in_pass * p.warps_per_row;
    const uint32_t sb = warp_in_row * 8 + (lane >> 2);
    const uint32_t c = lane & 3;
    const bool active = sb < p.n_sb;
    const uint32_t sb_off = sb * Q4K_SB_BYTES;
    const uint32_t qs_off = 16 + c * 32;

    uint64_t policy = 0;
    if (p.evict_first) policy = l2_evict_first_policy();

    auto issue = [&](uint32_t tile, uint32_t s) {  // one thread: arm stage s, start tile's copy
        const uint32_t row_begin = r0 + tile * p.tile_rows;
        const uint32_t nrows = min(p.tile_rows, r1 - row_begin);
        const uint32_t bytes = nrows * row_bytes;
        const uint8_t* src = p.q + (size_t)row_begin * row_bytes;
        uint8_t* dst = ring + (size_t)s * p.stage_bytes;
        mbar_expect_tx(&full[s], bytes);
        if (p.evict_first) bulk_g2s_stream(dst, src, bytes, &full[s], policy);
        else bulk_g2s(dst, src, bytes, &full[s]);
    };

    if (tid == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], n_warps);
            claim[s] = s;  // tile currently assigned to the stage
        }
        mbar_init_fence();
    }
    __syncthreads();  // barriers are initialised for everyone

    auto start_stream = [&]() {  // issuing a bulk copy takes tens of nanoseconds and never blocks
        if (tid == 0) {
            const uint32_t first = min(p.stages, n_tiles);
            for (uint32_t t = 0; t < first; ++t) issue(t, t);
        }
    };

    // Weights never depend on an earlier kernel.  When this CTA was scheduled early (programmatic
    // dependent launch, previous grid still running) the first ring-full of weights is fetched
    // while it waits for that grid.
    if (p.prefetch_first) start_stream();

    // x may be the output of the previous kernel in the stream; y may still be read by it.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    TRACE(1);

    // Stage x through shared memory: coalesced 16-byte loads (each lane reading its own 256-byte
    // chunk straight from global memory would touch 32 cache lines per instruction and serialise
    // in L1 for microseconds), stored transposed as xs[k][position] with an XOR swizzle so that
    // both these stores and the per-thread reads below are free of bank conflicts.
    {
        const uint32_t n_vec = p.n_sb * 64;  // float4 elements of x
        const float4* xg = reinterpret_cast<const float4*>(p.x);
        for (uint32_t g = tid; g < n_vec; g += blockDim.x) {
            const float4 v = __ldg(xg + g);
            const uint32_t k = g & 15u, pos = g >> 4;
            xs[k * p.x_pitch + (pos ^ (k & 7u))] = v;
        }
    }
    if (!p.prefetch_first) start_stream();
    __syncthreads();
    TRACE(2);

    float xv[64];
    if (active) {
        const uint32_t pos = sb * 4 + c;
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float4 v = xs[k * p.x_pitch + (pos ^ (k & 7u))];
            xv[4 * k] = v.x, xv[4 * k + 1] = v.y, xv[4 * k + 2] = v.z, xv[4 * k + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) xv[i] = 0.0f;
    }

    LaneCtx ctx;
    {
        const uint32_t h16 = (c & 1u) * 16u;
        ctx.big = c >= 2;
        ctx.sh0 = h16;
        ctx.sh_m = ctx.big ? h16 + 4 : h16;
        ctx.sh2 = h16 + 2;
        ctx.mask_a = ctx.big ? 0x0F0Fu : 0x3F3Fu;
        ctx.mask_b = ctx.big ? 0x3030u : 0u;

        float amax = 0.0f, sl = 0.0f, sh = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            sl += xv[i];
            sh += xv[32 + i];
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(xv[i]));  // NaN operands are ignored
        // An infinite |x| makes the row non-finite whatever the scaling: take the largest finite
        // exponent so that the power-of-two factors below stay representable.
        amax = fminf(amax, __int_as_float(0x7F7FFFFF));
        ctx.x_lo_sum = sl;
        ctx.x_hi_sum = sh;
        int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127;
        if (e < -126) e = -126;
        // nibble * 2^(pos-149) times x * 2^(C-pos) = nibble * x * 2^(C-149): about 2^-61 for the
        // largest |x| of the chunk, far from overflow and from the subnormal range whatever the
        // magnitude of the activations.  Both scalings are by exact powers of two.
        const int C = 88 - e;   // [-39, 214]
        const int C1 = C >> 1, C2 = C - C1;
        const int R = 149 - C;  // [-65, 188]
        const int R1 = R >> 1;
        ctx.rs_a = exp2i(R1);
        ctx.rs_b = exp2i(R - R1);
        const float f1 = exp2i(C1);
        const float gl[4] = {exp2i(C2), exp2i(C2 - 8), exp2i(C2 - 16), exp2i(C2 - 16)};
        const float gh[4] = {exp2i(C2 - 4), exp2i(C2 - 12), exp2i(C2 - 20), exp2i(C2 - 20)};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                ctx.xl[k][b] = pack_f32x2(xv[8 * k + b] * f1 * gl[b], xv[8 * k + 4 + b] * f1 * gl[b]);
                ctx.xh[k][b] = pack_f32x2(xv[32 + 8 * k + b] * f1 * gh[b],
                                          xv[32 + 8 * k + 4 + b] * f1 * gh[b]);
            }
        }
    }

    TRACE(3);
    // Inactive lanes (superblock index past the row) read superblock 0 and are zeroed below.
    const uint8_t* lane_base = ring + (active ? sb_off : 0u) + row_in_pass * row_bytes;
    const uint32_t pass_stride = p.rows_per_pass * row_bytes;
    const uint32_t wpr = p.warps_per_row;
    float* part_ptr = part + row_in_pass * wpr + warp_in_row;
    const uint32_t part_pass_stride = p.rows_per_pass * wpr;
    const uint32_t part_tile_stride = p.tile_rows * wpr;
    constexpr uint32_t kWriterStep = PASSES == 4 ? 8u : 16u;
    const uint32_t writer_ps = lane / kWriterStep;  // which of the PASSES totals this lane ends up with
    const bool is_writer = (lane & (kWriterStep - 1)) == 0 && writer_ps < (uint32_t)PASSES;
    const uint32_t writer_row = writer_ps * p.rows_per_pass + row_in_pass;

    uint32_t s = 0, parity = 0, rows_left = my_rows;
    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        if (!mbar_wait(&full[s], parity, p.status)) break;  // status word set; y stays partial
        if (tile < 14) TRACE(4 + tile);
        const uint8_t* sp = lane_base + s * p.stage_bytes;

        float v[PASSES];
        if (rows_left >= p.tile_rows) {
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) v[ps] = q4k_chunk_dot64(sp + ps * pass_stride, qs_off, ctx);
        } else {
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps)
                v[ps] = ps * p.rows_per_pass + row_in_pass < rows_left
                            ? q4k_chunk_dot64(sp + ps * pass_stride, qs_off, ctx)
                            : 0.0f;
        }
        if (!active) {
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) v[ps] = 0.0f;
        }
        const float total = warp_reduce_transposed<PASSES>(v, lane);
        if (is_writer && writer_row < rows_left) part_ptr[writer_ps * part_pass_stride] = total;

        if (tile + p.stages < n_tiles) {  // the stage will be needed again
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[s]);
                // Whoever sees all warps done with the stage (at least the last one to arrive)
                // competes for the refill; the compare-and-swap lets exactly one thread through.
                if (mbar_test(&empty[s], parity) &&
                    atomicCAS(&claim[s], tile, tile + p.stages) == tile)
                    issue(tile + p.stages, s);
            }
        }
        part_ptr += part_tile_stride;
        rows_left = rows_left > p.tile_rows ? rows_left - p.tile_rows : 0u;
        if (++s == p.stages) s = 0, parity ^= 1u;
    }

    TRACE(18);
    __syncthreads();
    TRACE(19);
    for (uint32_t r = tid; r < my_rows; r += blockDim.x) {
        float sum = part[r * p.warps_per_row];
        for (uint32_t wv = 1; wv < p.warps_per_row; ++wv) sum += part[r * p.warps_per_row + wv];
        p.y[r0 + r] = sum;
    }
}

// ---------------------------------------------------------------------------------------------

cudaError_t launch_q4k_matvec_segmented(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                        uint32_t n_sb, uint32_t* status, cudaStream_t stream,
                                        const MatvecTuning& tune, int sm_count, LaunchInfo* info);

cudaError_t launch_q4k_matvec(const uint8_t* q, const float* x, float* y, uint32_t rows,
                              uint32_t n_sb, uint32_t* status, cudaStream_t stream,
                              const MatvecTuning& tune, int sm_count, LaunchInfo* info) {
    if (rows == 0 || n_sb == 0) return cudaSuccess;
    if (n_sb > 128) return launch_q4k_matvec_segmented(q, x, y, rows, n_sb, status, stream, tune, sm_count, info);

    Q4kStreamParams p{};
    p.q = q, p.x = x, p.y = y, p.status = status, p.rows = rows, p.n_sb = n_sb;
    p.warps_per_row = (n_sb + 7) / 8;
    // CTA shape: whole rows per pass, about `threads` threads.  `ctas_per_sm` sizes the grid,
    // `resident` the shared-memory budget (CTAs of this and of the next kernel that should fit
    // on an SM together; about 118 registers per thread allow 16 warps per SM in total).
    int threads = tune.threads > 0 ? tune.threads : 256;
    if (p.warps_per_row > 8) threads = 512;
    int rows_per_pass = (threads / 32) / (int)p.warps_per_row;
    if (rows_per_pass < 1) rows_per_pass = 1;
    const int warps = rows_per_pass * (int)p.warps_per_row;
    p.rows_per_pass = (uint32_t)rows_per_pass;
    const int max_resident = 16 / warps > 0 ? 16 / warps : 1;
    int ctas_per_sm = tune.ctas_per_sm > 0 ? tune.ctas_per_sm : max_resident;
    if (ctas_per_sm > 16) ctas_per_sm = 16;
    int resident = tune.resident > 0 ? tune.resident : (ctas_per_sm < max_resident ? ctas_per_sm : max_resident);
    if (resident > max_resident) resident = max_resident;

    uint32_t grid = (uint32_t)(sm_count * ctas_per_sm);
    const uint32_t max_useful = (rows + (uint32_t)rows_per_pass - 1) / (uint32_t)rows_per_pass;
    if (grid > max_useful) grid = max_useful;
    // Keep the per-CTA partial-sum array small: more CTAs (several waves) for very tall matrices.
    const uint32_t max_part_entries = 4096;
    const uint32_t max_rows_per_cta = max_part_entries / p.warps_per_row;
    if ((rows + grid - 1) / grid > max_rows_per_cta) grid = (rows + max_rows_per_cta - 1) / max_rows_per_cta;
    if (grid < 1) grid = 1;
    const uint32_t rows_per_cta = (rows + grid - 1) / grid;
    p.part_entries = rows_per_cta * p.warps_per_row;

    const size_t row_bytes = (size_t)n_sb * Q4K_SB_BYTES;
    const size_t smem_cap = (size_t)(227 * 1024) / resident - 1024;  // 1 KB per CTA is reserved
    p.x_pitch = (n_sb * 4 + 7) & ~7u;
    const size_t xs_bytes = (size_t)16 * p.x_pitch * 16;
    const size_t fixed = (((size_t)p.part_entries * 4 + 64 + 15) & ~(size_t)15) + xs_bytes;
    int passes = 2;
    if (tune.tile_rows > 0) passes = tune.tile_rows / rows_per_pass;
    if (passes >= 4) passes = 4;
    else if (passes >= 2) passes = 2;
    else passes = 1;
    // Ring size: `st` stages of `ps` passes; when every tile of the CTA has its own stage the
    // last (partial) tile only needs its own rows, so the ring is exactly the CTA's share.
    auto tiles_for = [&](int ps) {
        return (int)((rows_per_cta + (uint32_t)(ps * rows_per_pass) - 1) / (uint32_t)(ps * rows_per_pass));
    };
    auto smem_for = [&](int ps, int st) {
        const size_t stage = (size_t)ps * rows_per_pass * row_bytes;
        const size_t ring = st >= tiles_for(ps) ? (size_t)rows_per_cta * row_bytes : (size_t)st * stage;
        return ((ring + (size_t)st * 20 + 15) & ~(size_t)15) + fixed;
    };
    while (passes > 1 && smem_for(passes, 2) > smem_cap) passes >>= 1;
    if (smem_for(passes, 1) > smem_cap) return cudaErrorInvalidConfiguration;
    p.tile_rows = (uint32_t)(passes * rows_per_pass);
    p.stage_bytes = (uint32_t)(p.tile_rows * row_bytes);
    const int tiles_per_cta = tiles_for(passes);
    int stages = tune.stages > 0 ? tune.stages : tiles_per_cta;  // whole share resident if it fits
    if (stages > tiles_per_cta) stages = tiles_per_cta;
    if (stages > 64) stages = 64;
    while (stages > 1 && smem_for(passes, stages) > smem_cap) --stages;
    const size_t smem = smem_for(passes, stages);
    p.stages = (uint32_t)stages;
    p.ring_bytes = (uint32_t)(stages >= tiles_per_cta ? (size_t)rows_per_cta * row_bytes
                                                      : (size_t)stages * p.stage_bytes);
    p.xs_offset = (uint32_t)(smem - xs_bytes);
    p.rows_base = rows / grid, p.rows_rem = rows % grid;
    p.tiles_lo = (p.rows_base + p.tile_rows - 1) / p.tile_rows;
    p.tiles_hi = (p.rows_base + 1 + p.tile_rows - 1) / p.tile_rows;
    p.evict_first = tune.evict_first > 0 ? 1u : 0u;
    p.prefetch_first = tune.pdl == 2 || tune.pdl < 0 ? 1u : 0u;

    void (*kern)(Q4kStreamParams) = nullptr;
    switch (passes) {
        case 1: kern = q4k_matvec_stream_kernel<1>; break;
        case 2: kern = q4k_matvec_stream_kernel<2>; break;
        default: kern = q4k_matvec_stream_kernel<4>; break;
    }
    if (info) {
        info->grid = (int)grid, info->block = warps * 32, info->smem = smem;
        info->tile_rows = (int)p.tile_rows, info->stages = stages, info->seg = (int)n_sb;
        info->n_seg = 1;
    }
    if (tune.dry_run) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;

    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3((unsigned)warps * 32);
    cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tune.pdl != 0 ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

}  // namespace axc
