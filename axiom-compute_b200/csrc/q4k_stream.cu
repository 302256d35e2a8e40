// Q4_K_M dequantise + matrix-vector, streaming kernel for sm_100a (rows of up to 128
// superblocks, i.e. K <= 32768; longer rows take the K-segmented kernel in q4k_matvec.cu).
//
// Replaces examples/q4km_dequant_matvec.axc:1-117 for `rows` outputs at once.
//
// Data movement.  A CTA owns a contiguous range of rows, i.e. one contiguous byte range of q,
// and pulls it through a shared-memory ring with untiled bulk async copies (TMA engine), one
// mbarrier per stage.  Issuing a bulk copy costs tens of nanoseconds and never blocks, so one
// thread requests the whole ring up front.  Stages are recycled without any CTA-wide barrier:
// every warp arrives on the stage's "empty" mbarrier when it has read it, and the warp that
// observes the phase complete re-arms and refills it.  With programmatic dependent launch the
// next call's CTAs are scheduled while this call drains and fetch their first ring-full of
// weights before `griddepcontrol.wait`; x is read and y written only after it.
//
// Arithmetic.  The 4-bit weights stay integers.  Per CTA the activations are quantised ONCE to
// 23-bit signed fixed point relative to the largest |x| of each 64-column chunk (a power-of-two
// scale: an error of at most 2^-23 of the chunk maximum per element, below what an fp32
// accumulation of the row keeps), and the three low bytes of that integer are used as base-256
// digits (two unsigned, the top one signed), transposed so that one 32-bit word holds one digit
// of four neighbouring columns.  A thread owns one chunk position (superblock s, chunk c: 32
// bytes of nibbles, sub-blocks 2c and 2c+1) for the life of the CTA and keeps its 48 digit
// words in registers.  Per 32-bit word of nibbles: `w & 0x0F0F0F0F` is the four low nibbles as
// bytes, `w & 0xF0F0F0F0` the four high ones times 16 (the 1/16 is folded into the scale), and
// six dp4a (u8 x u8/s8, exact int32 accumulation) multiply them with the digit words: two
// logic instructions and six integer-dot instructions per eight weights, nothing converted per
// weight.  Per sub-block the exact integer sum is rescaled once and combined as
// d*sc*sum(q_i x_i) - dmin*m*sum(x_i), so weights are never materialised here (the bit-exact
// dequantised values come from q4k_dequant_kernel, which shares q4k_unpack_pair).  Row sums:
// transposed warp-shuffle reduction, per-warp partials in shared memory, one fixed-order combine
// per CTA at the end (deterministic).
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
    uint32_t x_pitch;        // chunk positions (4 per superblock) rounded up to 8
    uint32_t xs_offset;      // byte offset of the digit words  uint4[16][x_pitch]
    uint32_t xm_offset;      // byte offset of the chunk metadata float4[x_pitch]
    uint32_t rows_base;      // rows / grid
    uint32_t rows_rem;       // rows % grid: the first rows_rem CTAs take one row more
    uint32_t tiles_lo, tiles_hi;  // tiles of a CTA with rows_base / rows_base + 1 rows
    uint32_t x_pos_end;      // chunk positions rounded up to a whole warp's worth (8)
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

// acc += sum_i a.u8[i] * b.s8[i]   (exact)
__device__ __forceinline__ void dp4a_us(int& acc, uint32_t a, uint32_t b) {
    asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(acc) : "r"(a), "r"(b));
}
// acc += sum_i a.u8[i] * b.u8[i]   (exact)
__device__ __forceinline__ void dp4a_uu(uint32_t& acc, uint32_t a, uint32_t b) {
    asm("dp4a.u32.u32 %0, %1, %2, %0;" : "+r"(acc) : "r"(a), "r"(b));
}

constexpr int X_FRAC_BITS = 21;  // |x| < 2^(e+1)  ->  |x * 2^(21-e)| < 2^22: top byte in [-64, 63]

// Per-thread constants for the life of the CTA.
struct LaneCtx {
    uint32_t al[8][3];  // low-nibble columns 4w..4w+3 of the chunk: digit words j = 0..2
    uint32_t ah[8][3];  // high-nibble columns 32+4w..32+4w+3
    float x_lo_sum, x_hi_sum;  // sum of the 32 activations of sub-block 2c / 2c+1
    float ps_a, ps_b;          // 2^(e - 21) as two representable factors
    uint32_t sh0, sh_m, sh2, mask_a, mask_b;  // scale/min unpack selectors for chunk c
    bool big;
};

// Dot of one 64-weight chunk (32 nibble bytes at sb_ptr + qs_off) with the thread's digit words.
// Returns this thread's contribution to the row sum.
__device__ __forceinline__ float q4k_chunk_dot_i8(const uint8_t* sb_ptr, uint32_t qs_off,
                                                  const LaneCtx& t) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(sb_ptr);
    const uint4 qa = *reinterpret_cast<const uint4*>(sb_ptr + qs_off);
    const uint4 qb = *reinterpret_cast<const uint4*>(sb_ptr + qs_off + 16);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};

    uint32_t l0 = 0, l1 = 0, h0 = 0, h1 = 0;  // unsigned digits 0, 1
    int l2 = 0, h2 = 0;                       // signed top digit
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint32_t lo4 = w[k] & 0x0F0F0F0Fu;  // bytes 4k..4k+3: elements 4k..4k+3
        const uint32_t hi4 = w[k] & 0xF0F0F0F0u;  // 16 * elements 32+4k..32+4k+3
        dp4a_uu(l0, lo4, t.al[k][0]);
        dp4a_uu(h0, hi4, t.ah[k][0]);
        dp4a_uu(l1, lo4, t.al[k][1]);
        dp4a_uu(h1, hi4, t.ah[k][1]);
        dp4a_us(l2, lo4, t.al[k][2]);
        dp4a_us(h2, hi4, t.ah[k][2]);
    }
    // sum(q_i X_i), X_i = d2 * 65536 + d1 * 256 + d0 (d0, d1 unsigned bytes, d2 signed).  The
    // high-nibble sums carry the factor 16 of the unshifted nibbles.
    const float s_lo = fmaf((float)l2, 65536.0f, (float)(l1 * 256u + l0));
    const float s_hi = fmaf((float)h2, 4096.0f, (float)(h1 * 256u + h0) * 0.0625f);

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
    t1 = (t1 * t.ps_a) * t.ps_b;  // back to the scale of x (two exact power-of-two steps)
    return fmaf(-dmin, t2, d * t1);
}

// Four activations scaled by f1 * f2 (= 2^(21-e)) and rounded to integers -> three digit words:
// word j holds byte j of the four integers (a 4 x 4 byte transpose).
__device__ __forceinline__ uint4 quantize_x4(const float4 v, float f1, float f2) {
    const uint32_t x0 = (uint32_t)__float2int_rn(v.x * f1 * f2);
    const uint32_t x1 = (uint32_t)__float2int_rn(v.y * f1 * f2);
    const uint32_t x2 = (uint32_t)__float2int_rn(v.z * f1 * f2);
    const uint32_t x3 = (uint32_t)__float2int_rn(v.w * f1 * f2);
    const uint32_t t01 = __byte_perm(x0, x1, 0x5140);  // x0.b0 x1.b0 x0.b1 x1.b1
    const uint32_t t23 = __byte_perm(x2, x3, 0x5140);
    const uint32_t u01 = __byte_perm(x0, x1, 0x0062);  // x0.b2 x1.b2 . .
    const uint32_t u23 = __byte_perm(x2, x3, 0x0062);
    return make_uint4(__byte_perm(t01, t23, 0x5410), __byte_perm(t01, t23, 0x7632),
                      __byte_perm(u01, u23, 0x5410), 0u);
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
    uint4* xs = reinterpret_cast<uint4*>(smem + p.xs_offset);    // [16][x_pitch] digit words
    float4* xm = reinterpret_cast<float4*>(smem + p.xm_offset);  // [x_pitch] sums and scale

    // Let the next grid in the stream be scheduled as early as the hardware allows.
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

    auto start_stream = [&]() {
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

    // Quantise x once per CTA.  Four threads share a 64-column chunk position: thread (pos, qt)
    // loads columns 16qt..16qt+15 (coalesced across the warp), i.e. the four nibble words
    // k = 4qt..4qt+3 of that half (qt < 2: low nibbles, qt >= 2: high nibbles), so each float4 is
    // one dp4a operand set.  Stored as xs[k][pos] with an XOR swizzle so that these stores and the
    // per-thread reads below are free of bank conflicts.
    {
        const float4* xg = reinterpret_cast<const float4*>(p.x);
        constexpr uint32_t FULL = 0xFFFFFFFFu;
        const uint32_t n_pos = p.n_sb * 4;
        const uint32_t qt = tid & 3u;
        for (uint32_t pos = tid >> 2; pos < p.x_pos_end; pos += blockDim.x >> 2) {
            const bool valid = pos < n_pos;
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                v[u] = valid ? __ldg(xg + pos * 16 + qt * 4 + u) : make_float4(0.f, 0.f, 0.f, 0.f);
            // largest finite |x| of the chunk (NaNs are ignored by fmaxf) and the half sums
            float m = 0.0f, s = 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
                s += (v[u].x + v[u].y) + (v[u].z + v[u].w);
            }
            m = fmaxf(m, __shfl_xor_sync(FULL, m, 1));
            m = fmaxf(m, __shfl_xor_sync(FULL, m, 2));
            s += __shfl_xor_sync(FULL, s, 1);                     // sum of this 32-column half
            const float s_other = __shfl_xor_sync(FULL, s, 2);   // sum of the other half
            m = fminf(m, __int_as_float(0x7F7FFFFF));  // an infinite x makes the row non-finite anyway
            int e = (int)((__float_as_uint(m) >> 23) & 0xFFu) - 127;
            if (e < -126) e = -126;
            const int up = X_FRAC_BITS - e;  // [-106, 147]: two representable power-of-two steps
            const int up1 = up >> 1;
            const float f1 = exp2i(up1), f2 = exp2i(up - up1);
            if (valid) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t k = qt * 4 + u;
                    xs[k * p.x_pitch + (pos ^ (k & 7u))] = quantize_x4(v[u], f1, f2);
                }
                if (qt == 0) {
                    const int dn = -up, dn1 = dn >> 1;  // e - 21 in [-147, 106]
                    xm[pos] = make_float4(s, s_other, exp2i(dn1), exp2i(dn - dn1));
                }
            }
        }
    }
    if (!p.prefetch_first) start_stream();
    __syncthreads();
    TRACE(2);

    LaneCtx ctx;
    {
        const uint32_t h16 = (c & 1u) * 16u;
        ctx.big = c >= 2;
        ctx.sh0 = h16;
        ctx.sh_m = ctx.big ? h16 + 4 : h16;
        ctx.sh2 = h16 + 2;
        ctx.mask_a = ctx.big ? 0x0F0Fu : 0x3F3Fu;
        ctx.mask_b = ctx.big ? 0x3030u : 0u;
        const uint32_t pos = active ? sb * 4 + c : 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint4 a = xs[k * p.x_pitch + (pos ^ (uint32_t)k)];
            const uint4 b = xs[(8 + k) * p.x_pitch + (pos ^ (uint32_t)k)];
            ctx.al[k][0] = a.x, ctx.al[k][1] = a.y, ctx.al[k][2] = a.z;
            ctx.ah[k][0] = b.x, ctx.ah[k][1] = b.y, ctx.ah[k][2] = b.z;
        }
        const float4 meta = xm[pos];
        ctx.x_lo_sum = meta.x, ctx.x_hi_sum = meta.y, ctx.ps_a = meta.z, ctx.ps_b = meta.w;
    }

    TRACE(3);
    // Lanes past the end of the row read superblock 0 and are zeroed below.
    const uint8_t* lane_base = ring + (active ? sb * Q4K_SB_BYTES : 0u) + row_in_pass * row_bytes;
    const uint32_t pass_stride = p.rows_per_pass * row_bytes;
    const uint32_t wpr = p.warps_per_row;
    float* part_ptr = part + row_in_pass * wpr + warp_in_row;
    const uint32_t part_pass_stride = p.rows_per_pass * wpr;
    const uint32_t part_tile_stride = p.tile_rows * wpr;
    constexpr uint32_t kWriterStep = PASSES == 4 ? 8u : 16u;
    const uint32_t writer_ps = lane / kWriterStep;  // which of the PASSES totals this lane gets
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
            for (int ps = 0; ps < PASSES; ++ps) v[ps] = q4k_chunk_dot_i8(sp + ps * pass_stride, qs_off, ctx);
        } else {
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps)
                v[ps] = ps * p.rows_per_pass + row_in_pass < rows_left
                            ? q4k_chunk_dot_i8(sp + ps * pass_stride, qs_off, ctx)
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
        float sum = part[r * wpr];
        for (uint32_t wv = 1; wv < wpr; ++wv) sum += part[r * wpr + wv];
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
    // `resident` the shared-memory budget (how many CTAs should fit on an SM together; about 118
    // registers per thread allow 16 warps per SM in total).
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
    const size_t xs_bytes = (size_t)16 * p.x_pitch * 16;  // digit words
    const size_t xm_bytes = (size_t)p.x_pitch * 16;       // per-chunk sums and scale
    const size_t fixed = (((size_t)p.part_entries * 4 + 64 + 15) & ~(size_t)15) + xs_bytes + xm_bytes;
    int passes = 4;
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
    if (smem_for(passes, 1) > (size_t)227 * 1024 - 1024) return cudaErrorInvalidConfiguration;
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
    p.xm_offset = (uint32_t)(smem - xm_bytes);
    p.xs_offset = (uint32_t)(smem - xm_bytes - xs_bytes);
    p.x_pos_end = (n_sb * 4 + 7) & ~7u;
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
