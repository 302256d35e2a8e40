// Streaming dequantise + matrix-vector kernel for sm_100a, both 4-bit block formats:
//   Q4_K_M  144-byte superblocks of 256 weights  (examples/q4km_dequant_matvec.axc:1-117)
//   Q4_0     18-byte blocks of 32 weights         (examples/q4_0_dequant_matvec.axc:1-51)
// generalised from the reference's single output to `rows` outputs per launch: row r is one
// reference call on the r-th run of blocks against the shared activation vector x.
// Serves Q4_K_M rows of up to 128 superblocks and Q4_0 rows of an even number of blocks up to
// 1024 (K <= 32768); other shapes take the kernels in q4k_matvec.cu / q4_0_matvec.cu.
//
// Data movement.  A CTA owns a contiguous range of rows, i.e. one contiguous byte range of q,
// and pulls it through a shared-memory ring with untiled bulk async copies (TMA engine), one
// mbarrier per stage.  Issuing a bulk copy costs tens of nanoseconds and never blocks, so one
// thread requests the whole ring up front.  Stages are recycled without any CTA-wide barrier:
// every warp arrives on the stage's "empty" mbarrier when it has read it, and the warp that
// observes the phase complete re-arms and refills it.  (18-byte Q4_0 blocks are only 2-byte
// aligned: a tile is copied as the enclosing 16-byte aligned range and addressed with the
// remainder.)  With programmatic dependent launch the next call's CTAs are scheduled while this
// call drains and fetch their first ring-full of weights before `griddepcontrol.wait`; x is
// read and y written only after it.
//
// Arithmetic.  The 4-bit weights stay integers.  Per CTA the activations are quantised ONCE to
// 24-bit two's-complement fixed point relative to the largest |x| of each 64-column chunk (a
// power-of-two scale: an error of at most 2^-23 of the chunk maximum per element, below what an
// fp32 accumulation of the row keeps; the bound is derived beside X_FRAC_BITS), and the three
// bytes of that integer are used as base-256 digits (two unsigned, the top one signed),
// transposed so that one 32-bit word holds one digit of four neighbouring columns.  A thread owns one 64-weight position of the row (Q4_K_M:
// superblock s, chunk c = 32 nibble bytes, sub-blocks 2c and 2c+1; Q4_0: a pair of blocks) for
// the life of the CTA and keeps its 48 digit words in registers.  Per 32-bit word of nibbles:
// `w & 0x0F0F0F0F` is the four low nibbles as bytes, `w & 0xF0F0F0F0` the four high ones times
// 16 (the 1/16 is folded into the scale), and six dp4a (u8 x u8/s8, exact int32 accumulation)
// multiply them with the digit words: two logic instructions and six integer-dot instructions
// per eight weights, nothing converted per weight.  Per sub-block the exact integer sum is
// rescaled once and combined as d*sc*sum(q_i X_i) - dmin*m*sum(X_i) over the same fixed-point X
// (Q4_0: d*sum((q_i - 8) X_i), the -8 folded into the start value of the integer sums), so weights
// are never materialised here (the bit-exact dequantised values come
// from the dequant kernels, which share the unpack code).  Row sums: transposed warp-shuffle
// reduction, per-warp partials in shared memory, one fixed-order combine per CTA at the end
// (deterministic).
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "axc_device.cuh"
#include "axc_kernels.h"


namespace axc {

constexpr int FMT_Q4K = 0, FMT_Q4_0 = 1;

struct StreamParams {
    const uint8_t* q;
    const float* x;
    const void* x_prepared;  // digit words + metadata made by the prepare kernels (PREPARED kernels)
    uint32_t x_prepared_rms; // PREPARED: scale the result by 1 / sqrt(mean(x^2)) from the image's partial sums
    // Fused x source (XFUSE kernels): x = a [+ b], each either a plain fp32 vector or a vector
    // of (value, epoch) words written by the all-gather epilogue of an earlier call; with
    // x_unit_rms the result is the matvec of x / sqrt(mean(x^2)).
    const float* x2;
    const uint64_t* x_pairs;
    const uint64_t* x2_pairs;
    const uint32_t* x_epoch_ptr;
    uint64_t x_parity_stride;  // words of odd epochs live this many bytes behind those of even epochs
    uint32_t x_unit_rms;
    float* y;
    uint32_t* status;
    uint32_t rows;
    uint32_t row_bytes;      // bytes of q per row
    uint32_t n_pos;          // 64-weight positions per row (Q4_K_M: 4 per superblock; Q4_0: blocks / 2)
    uint32_t warps_per_row;  // ceil(n_pos / 32)
    uint32_t rows_per_pass;  // warps per CTA / warps_per_row
    uint32_t tile_rows;      // PASSES * rows_per_pass
    uint32_t stages;
    uint32_t stage_bytes;    // capacity of one stage
    uint32_t ring_bytes;     // stages * stage_bytes, or the CTA's exact share when all resident
    uint32_t part_entries;   // capacity of the partial-sum array (>= rows per CTA * warps_per_row)
    uint32_t evict_first;
    uint32_t prefetch_first; // start the weight stream before griddepcontrol.wait
    uint32_t independent;    // x and y are untouched by the previous launch: wait only before writing y
    uint32_t x_pitch;        // positions rounded up to 8
    uint32_t xs_offset;      // byte offset of the digit words  uint4[16][x_pitch]
    uint32_t xm_offset;      // byte offset of the position metadata float4[x_pitch]
    uint32_t rows_base;      // rows / grid
    uint32_t rows_rem;       // rows % grid: the first rows_rem CTAs take one row more
    uint32_t tiles_lo, tiles_hi;  // tiles of a CTA with rows_base / rows_base + 1 rows
    uint32_t x_pos_end;      // positions rounded up to a whole warp's worth (8)
    // fused all-gather epilogue (GATHER kernels): every rank stores its y slice, each value
    // paired with the current epoch in one 8-byte word, into every rank's full-length vector
    const uint64_t* y_peer_bases;  // device array [world]: base address of each rank's pair storage
    uint64_t y_offset_bytes;       // offset of this call's vector (uint2[global rows]) in that storage
    uint64_t y_parity_stride;      // odd epochs store this many bytes further on (two alternating copies)
    const uint32_t* epoch_ptr;     // this rank's epoch counter (advanced once per step by the caller)
    uint32_t world, rank, row_offset;
    // completion signal for a host that polls instead of waiting on an event: every CTA counts
    // itself in after its stores of y; the last one writes done_seq to done_flag (host memory)
    uint32_t* done_counter;
    uint32_t* done_flag;
    uint32_t done_seq;
    float* y_host;           // with done_flag: y (device memory) is copied here by the last CTA
    // PREPARED kernels, single-launch host dispatch: x lies in mapped HOST memory.  The first
    // x_n_prod CTAs read it over PCIe and write the quantised image (x_prepared) before they turn
    // to their rows; the last of them publishes x_seq in *x_ready, which every CTA waits for
    // (bounded) before it reads the image.  Producers never wait for anyone and carry the lowest
    // block indices, so they are running or finished whenever a later CTA is waiting.
    const float* x_host;
    uint32_t* x_ready;
    uint32_t* x_prod_counter;
    uint32_t x_seq;
    uint32_t x_n_prod;
};

// Completion for a polling host, called by every thread of a CTA after the CTA's stores of y (to
// device memory).  CTAs count themselves in at device scope (cheap); the last CTA of the grid
// copies the whole of y to the host buffer, then ONE system-scope fence orders that copy before
// the sequence number it publishes where the host polls.  (System-scope fences are expensive when
// stores to host memory are outstanding and they serialise across the GPU: y stored to the host
// by every CTA cost 16 us per launch with a fence per storing thread and 8 us with one per CTA;
// this form costs about as much as the copy.)
__device__ __forceinline__ void signal_cta_done(const StreamParams& p, uint32_t tid) {
    __shared__ uint32_t s_last;
    __syncthreads();   // every thread's stores of y are issued
    if (tid == 0) {
        __threadfence();
        s_last = atomicAdd(p.done_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (p.y_host) {
        const uint32_t n4 = p.rows >> 2;
        const float4* src = reinterpret_cast<const float4*>(p.y);
        float4* dst = reinterpret_cast<float4*>(p.y_host);
        // loads in batches of sixteen before their stores: the loop is latency-bound otherwise
        for (uint32_t base = 0; base < n4; base += 16u * blockDim.x) {
            float4 v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const uint32_t i = base + u * blockDim.x + tid;
                if (i < n4) v[u] = __ldcg(src + i);
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const uint32_t i = base + u * blockDim.x + tid;
                if (i < n4) dst[i] = v[u];
            }
        }
        for (uint32_t i = (n4 << 2) + tid; i < p.rows; i += blockDim.x) p.y_host[i] = __ldcg(p.y + i);
        __syncthreads();
    }
    if (tid == 0) {
        *p.done_counter = 0;
        __threadfence_system();
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.done_flag), "r"(p.done_seq) : "memory");
    }
}

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

// Fixed point of the activations.  With 2^e <= M < 2^(e+1), M the largest finite |x| of a 64-column
// chunk, every x of the chunk becomes X = rn(x * 2^(22-e)) clamped to [-2^23, 2^23 - 1]: a 24-bit
// two's-complement integer, i.e. three byte digits (top one signed, -128..127).  The integer dot
// products with the 4-bit weights are exact, so the only error of the scheme is |x - X 2^(e-22)| <=
// 2^(e-23) <= 2^-23 M per element (one unit more for an element the clamp touches):
//     |y_fixed - y_exact| <= 2^-23 * sum over chunks c of  M_c * sum_{i in c} |w_i|.
// Measured against sum_i |w_i x_i| (the norm-wise bar) that is <= 2^-23 R = 1.2e-7 R when the |x| of a
// chunk lie within a factor R of its maximum: far inside 1e-5 for any realistic spread (R <= 80).  An
// element below 2^-24 of its chunk's maximum is flushed to zero; the bound then still holds but is
// no longer small RELATIVE to that element's own term, which matters only if the larger elements of
// the chunk meet weights that are (nearly) zero: the worst case, one element at M with weight 0
// beside 63 elements of about 2^-24 M, loses those 63 terms entirely, where an fp32 sum keeps 24
// bits of each.  The tests measure log-uniform spreads over 2^30 inside every chunk.
constexpr int X_FRAC_BITS = 22;

// Per-thread constants for the life of the CTA.
struct LaneCtx {
    uint32_t dg[16][3];  // digit words of columns 4k..4k+3 of the position, k = 0..15
    // Q4_K_M: sum of the FIXED-POINT activations over columns 0..31 / 32..63 of the position, in
    // x's units (so the min term sees exactly the x the integer dot products see); NaN if any x of
    // that half is not finite.  Q4_0: 0, or NaN if any x of the block is not finite.
    float sum_a, sum_b;
    float ps_a, ps_b;    // 2^(e - 22) as two representable factors
    uint32_t sh0, sh_m, sh2, mask_a, mask_b;  // Q4_K_M scale/min unpack selectors for chunk c
    bool big;
    // Q4_0: start values of the digit sums, -8 * (sum of the digit over the 16 columns a nibble
    // half meets) and -128 * ... for the high nibbles (which stay multiplied by 16): the sums then
    // come out as sum((q_i - 8) X_i), exactly, and a block of all-8 nibbles gives exactly zero.
    int q40_lo[2][3], q40_hi[2][3];
};

// Exact integer dot of four nibble words with the digit words of columns [4*k0, 4*k0 + 16):
// low nibbles against dg[k0 + j], high nibbles (left unshifted: times 16) against dg[k1 + j].
struct DigitSums {
    uint32_t l0 = 0, l1 = 0, h0 = 0, h1 = 0;  // digits 0, 1 (unsigned digits; sums may start negative)
    int l2 = 0, h2 = 0;                       // signed top digit
    __device__ __forceinline__ void start(const int (&lo)[3], const int (&hi)[3]) {
        l0 = (uint32_t)lo[0], l1 = (uint32_t)lo[1], l2 = lo[2];
        h0 = (uint32_t)hi[0], h1 = (uint32_t)hi[1], h2 = hi[2];
    }
    __device__ __forceinline__ void add(uint32_t w, const uint32_t (&lo)[3], const uint32_t (&hi)[3]) {
        const uint32_t lo4 = w & 0x0F0F0F0Fu, hi4 = w & 0xF0F0F0F0u;
        dp4a_uu(l0, lo4, lo[0]);
        dp4a_uu(h0, hi4, hi[0]);
        dp4a_uu(l1, lo4, lo[1]);
        dp4a_uu(h1, hi4, hi[1]);
        dp4a_us(l2, lo4, lo[2]);
        dp4a_us(h2, hi4, hi[2]);
    }
    // sum(q_i X_i), X_i = d2 * 65536 + d1 * 256 + d0
    __device__ __forceinline__ float low() const { return fmaf((float)l2, 65536.0f, (float)(l1 * 256u + l0)); }
    __device__ __forceinline__ float high() const {  // carries the factor 16 of the unshifted nibbles
        return fmaf((float)h2, 4096.0f, (float)(h1 * 256u + h0) * 0.0625f);
    }
    // the same when the sums may be negative (Q4_0 start values)
    __device__ __forceinline__ float low_signed() const {
        return fmaf((float)l2, 65536.0f, (float)(int)(l1 * 256u + l0));
    }
    __device__ __forceinline__ float high_signed() const {
        return fmaf((float)h2, 4096.0f, (float)(int)(h1 * 256u + h0) * 0.0625f);
    }
};

// Q4_K_M: this thread's contribution to the row sum from one superblock (chunk c of it).
__device__ __forceinline__ float q4k_pos_dot(const uint8_t* sb_ptr, uint32_t qs_off, const LaneCtx& t) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(sb_ptr);
    const uint4 qa = *reinterpret_cast<const uint4*>(sb_ptr + qs_off);
    const uint4 qb = *reinterpret_cast<const uint4*>(sb_ptr + qs_off + 16);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    // byte l of the chunk: low nibble -> element l (columns 0..31), high nibble -> element 32 + l
    DigitSums s;
#pragma unroll
    for (int k = 0; k < 8; ++k) s.add(w[k], t.dg[k], t.dg[8 + k]);
    const float s_lo = s.low(), s_hi = s.high();

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
    float t2 = (float)(m_pair & 0xFFu) * t.sum_a;
    t2 = fmaf((float)(m_pair >> 8), t.sum_b, t2);
    t1 = (t1 * t.ps_a) * t.ps_b;  // back to the scale of x (two exact power-of-two steps)
    return fmaf(-dmin, t2, d * t1);
}

// Q4_0: contribution of one block pair (36 bytes, 4-byte aligned).  Block b: fp16 d, then 16
// bytes; byte k: low nibble -> element k, high nibble -> element k + 16
// (crates/axc-driver/benches/common.rs:240-255).
__device__ __forceinline__ float q40_pos_dot(const uint8_t* pair_ptr, const LaneCtx& t) {
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(pair_ptr);
    uint32_t W[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) W[i] = wp[i];
    DigitSums s0, s1;
    s0.start(t.q40_lo[0], t.q40_hi[0]);
    s1.start(t.q40_lo[1], t.q40_hi[1]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // block 0: its 16 nibble bytes straddle the words by 16 bits
        s0.add(__funnelshift_r(W[j], W[j + 1], 16), t.dg[j], t.dg[4 + j]);
        s1.add(W[5 + j], t.dg[8 + j], t.dg[12 + j]);
    }
    const float d0 = f16_bits_to_f32(W[0] & 0xFFFFu);
    const float d1 = f16_bits_to_f32(W[4] >> 16);
    // d * sum((q_i - 8) x_i) per block; sum_a / sum_b are 0, or NaN for a non-finite x
    const float a0 = ((s0.low_signed() + s0.high_signed()) * t.ps_a) * t.ps_b + t.sum_a;
    const float a1 = ((s1.low_signed() + s1.high_signed()) * t.ps_a) * t.ps_b + t.sum_b;
    return fmaf(d1, a1, d0 * a0);
}

// Four activations scaled by f1 * f2 (= 2^(22-e)) and rounded to integers -> three digit words:
// word j holds byte j of the four integers (a 4 x 4 byte transpose).
__device__ __forceinline__ uint4 quantize_x4(const float4 v, float f1, float f2) {
    constexpr int kTop = (1 << 23) - 1;   // an |x| just below 2^(e+1) would round up to 2^23
    const uint32_t x0 = (uint32_t)min(__float2int_rn(v.x * f1 * f2), kTop);
    const uint32_t x1 = (uint32_t)min(__float2int_rn(v.y * f1 * f2), kTop);
    const uint32_t x2 = (uint32_t)min(__float2int_rn(v.z * f1 * f2), kTop);
    const uint32_t x3 = (uint32_t)min(__float2int_rn(v.w * f1 * f2), kTop);
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

// Quantise the activations of `n_pos` 64-column positions into digit words.  Four threads share
// a position: thread (pos, qt) loads columns 16qt..16qt+15 (coalesced across the warp), i.e. the
// four nibble words k = 4qt..4qt+3, so each float4 is one dp4a operand set.  Stored as
// xs[k][pos] with an XOR swizzle so that these stores and the per-thread reads of the matvec
// are free of shared-memory bank conflicts; xm[pos] = (0 or NaN: is any x of columns 0..31 not
// finite, the same for columns 32..63, two factors of 2^(e-22)).  `nthreads` is a multiple of 32; all threads must call.
// `load16(i, v)` fills v[0..3] with columns 4i..4i+15.  Returns this thread's share of sum(x^2).
template <class Load16>
__device__ __forceinline__ float quantize_x_positions_from(Load16 load16, uint4* xs, float4* xm,
                                                           uint32_t n_pos, uint32_t pos_end, uint32_t pitch,
                                                           uint32_t tid, uint32_t nthreads, uint32_t pos_begin = 0) {
    float sumsq = 0.0f;
    {
        constexpr uint32_t FULL = 0xFFFFFFFFu;
        const uint32_t qt = tid & 3u;
        for (uint32_t pos = pos_begin + (tid >> 2); pos < pos_end; pos += nthreads >> 2) {
            const bool valid = pos < n_pos;
            float4 v[4];
            if (valid) {
                load16(pos * 16 + qt * 4, v);
            } else {
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            // largest finite |x| of the chunk (NaNs are ignored by fmaxf) and the half sums
            float m = 0.0f, s = 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
                s += (v[u].x + v[u].y) + (v[u].z + v[u].w);
                sumsq += (v[u].x * v[u].x + v[u].y * v[u].y) + (v[u].z * v[u].z + v[u].w * v[u].w);
            }
            m = fmaxf(m, __shfl_xor_sync(FULL, m, 1));
            m = fmaxf(m, __shfl_xor_sync(FULL, m, 2));
            s += __shfl_xor_sync(FULL, s, 1);                     // sum of this 32-column half
            const float s_other = __shfl_xor_sync(FULL, s, 2);   // sum of the other half
            m = fminf(m, __int_as_float(0x7F7FFFFF));  // an infinite x makes the row non-finite anyway
            int e = (int)((__float_as_uint(m) >> 23) & 0xFFu) - 127;
            if (e < -126) e = -126;
            const int up = X_FRAC_BITS - e;  // [-105, 148]: two representable power-of-two steps
            const int up1 = up >> 1;
            const float f1 = exp2i(up1), f2 = exp2i(up - up1);
            if (valid) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t k = qt * 4 + u;
                    xs[k * pitch + (pos ^ (k & 7u))] = quantize_x4(v[u], f1, f2);
                }
                if (qt == 0) {
                    const int dn = -up, dn1 = dn >> 1;  // e - 22 in [-148, 105]
                    // 0 (finite) or NaN (an infinite or NaN x in that half): what the integers cannot carry
                    xm[pos] = make_float4(s * 0.0f, s_other * 0.0f, exp2i(dn1), exp2i(dn - dn1));
                }
            }
        }
    }
    return sumsq;
}

__device__ __forceinline__ void quantize_x_positions(const float* __restrict__ x, uint4* xs, float4* xm,
                                                     uint32_t n_pos, uint32_t pos_end, uint32_t pitch,
                                                     uint32_t tid, uint32_t nthreads) {
    const float4* xg = reinterpret_cast<const float4*>(x);
    (void)quantize_x_positions_from(
        [&](uint32_t i, float4* v) {
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldg(xg + i + u);
        },
        xs, xm, n_pos, pos_end, pitch, tid, nthreads);
}

// Sixteen columns (4i .. 4i+15) of a (value, epoch) vector.  All eight 16-byte loads are issued
// together (bypassing L1) as pairs of 64-bit elements, so value and epoch of a word come from one
// store, and the epochs are checked afterwards; only if a word is still old does the thread poll,
// bounded, until all sixteen carry `epoch`.  A word from a LATER epoch means that a producer ran
// ahead of this reader (the storage was reused too early): that is reported, never accepted.
// After one timeout the thread only looks once at later words.
struct PairWait {
    bool gave_up = false, ahead = false;
};

__device__ __forceinline__ void load_pairs16(const uint64_t* base, uint32_t i, uint32_t epoch, PairWait& pw,
                                             float4* v) {
    const uint64_t* src = base + 4 * (size_t)i;
    uint64_t w[16];
    uint32_t it = pw.gave_up ? (1u << 20) - 1u : 0u;
    for (;;) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
            asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];"
                         : "=l"(w[2 * u]), "=l"(w[2 * u + 1]) : "l"(src + 2 * u) : "memory");
        bool ok = true, ahead = false;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int32_t d = (int32_t)((uint32_t)(w[u] >> 32) - epoch);
            ok = ok && d == 0;
            ahead = ahead || d > 0;
        }
        if (ok) break;
        if (ahead) {
            pw.ahead = true;
            break;
        }
        if (++it >= (1u << 20)) {
            pw.gave_up = true;
            break;
        }
        __nanosleep(64);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
        v[u] = make_float4(__uint_as_float((uint32_t)w[4 * u]), __uint_as_float((uint32_t)w[4 * u + 1]),
                           __uint_as_float((uint32_t)w[4 * u + 2]), __uint_as_float((uint32_t)w[4 * u + 3]));
}

__device__ __forceinline__ void report_pair_wait(const PairWait& pw, uint32_t* status) {
    if (!status) return;
    if (pw.gave_up) atomicOr(status, ERR_PEER_WAIT_TIMEOUT);
    if (pw.ahead) atomicOr(status, ERR_EPOCH_AHEAD);
}

template <int FMT, int PASSES, bool PREPARED, bool GATHER, bool XFUSE>
__global__ void __launch_bounds__(512, 1) q4_matvec_stream_kernel(const StreamParams p) {
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

    // A launch declared independent lets the next grid be scheduled at once.  An ordered launch
    // does so only after its own dependency wait (below): a grid scheduled behind it may read its
    // inputs without waiting, and must then find every earlier launch of the stream complete.
    if (p.independent) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Rows owned by this CTA: an even split computed on the host (no CTA has more than one
    // extra row).
    const uint32_t bid = blockIdx.x;
    const uint32_t r0 = bid * p.rows_base + min(bid, p.rows_rem);
    const uint32_t my_rows = p.rows_base + (bid < p.rows_rem ? 1u : 0u);
    const uint32_t r1 = r0 + my_rows;
    if (my_rows == 0) {
        if (p.done_flag) signal_cta_done(p, tid);
        return;
    }
    const uint32_t n_tiles = bid < p.rows_rem ? p.tiles_hi : p.tiles_lo;
    const uint32_t row_bytes = p.row_bytes;

    const uint32_t row_in_pass = warp / p.warps_per_row;
    const uint32_t warp_in_row = warp - row_in_pass * p.warps_per_row;
    const uint32_t my_pos = warp_in_row * 32 + lane;  // this thread's 64-weight position in the row
    const bool active = my_pos < p.n_pos;
    const uint32_t c = lane & 3;                      // Q4_K_M: chunk within the superblock
    const uint32_t qs_off = 16 + c * 32;

    uint64_t policy = 0;
    if (p.evict_first) policy = l2_evict_first_policy();

    auto issue = [&](uint32_t tile, uint32_t s) {  // one thread: arm stage s, start tile's copy
        const uint32_t row_begin = r0 + tile * p.tile_rows;
        const uint32_t nrows = min(p.tile_rows, r1 - row_begin);
        // The enclosing 16-byte aligned range (Q4_K_M rows are already aligned).  It stays inside
        // the 16-byte granules that hold valid bytes, so it never leaves the pages of q.
        const size_t start = (size_t)row_begin * row_bytes;
        const size_t a_start = start & ~(size_t)15;
        const uint32_t bytes = (uint32_t)(((start + (size_t)nrows * row_bytes + 15) & ~(size_t)15) - a_start);
        uint8_t* dst = ring + (size_t)s * p.stage_bytes;
        mbar_expect_tx(&full[s], bytes);
        if (p.evict_first) bulk_g2s_stream(dst, p.q + a_start, bytes, &full[s], policy);
        else bulk_g2s(dst, p.q + a_start, bytes, &full[s]);
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
    // A CTA that produces the x image from host memory (single-launch host dispatch) issues its
    // loads of the first 64 positions first: the PCIe round trip then runs while thread 0 requests
    // the ring.
    [[maybe_unused]] float4 host_first[8];
    [[maybe_unused]] bool host_first_valid = false;
    if constexpr (PREPARED) {
        if (p.x_host && bid < p.x_n_prod && blockDim.x >= 128u) {
            const float4* xh = reinterpret_cast<const float4*>(p.x_host);
            const uint32_t n_f4 = p.n_pos * 16u;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t idx = u * blockDim.x + tid, gi = bid * 1024u + idx;
                host_first[u] = idx < 1024u && gi < n_f4 ? __ldg(xh + gi) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            host_first_valid = true;
        }
    }
    if (p.prefetch_first) start_stream();

    // x may be the output of the previous kernel in the stream; y may still be read by it.
    // A caller that knows neither is the case (say the up projection launched right after the
    // gate projection of the same x) lets the whole prologue overlap the previous kernel.
    if (!p.independent) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    // Fused all-gather: the peer addresses never change; the epoch was advanced by an earlier
    // kernel of the stream, so it is read on this side of the wait (through L2, not a cached line).
    __shared__ uint64_t peer_base[16];
    __shared__ float sumsq_part[16];
    uint32_t epoch = 0;
    if constexpr (GATHER) {
        if (tid < p.world) peer_base[tid] = p.y_peer_bases[tid] + p.y_offset_bytes;
        if (!p.independent) asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(p.epoch_ptr) : "memory");
    }

    if constexpr (PREPARED) {
        // The digit words were produced once by a prepare kernel; every thread reads its own
        // position's words straight into registers below (coalesced: consecutive lanes, consecutive
        // 16-byte words), so there is nothing to stage and nothing to wait for here ...
        if (p.x_host) {
            // ... unless this launch carries its own producers (x in mapped host memory).
            uint4* image = reinterpret_cast<uint4*>(const_cast<void*>(p.x_prepared));
            if (bid < p.x_n_prod) {
                // 64 positions (16 KB of x) at a time: fully coalesced 16-byte loads from host memory,
                // all of a thread's loads issued together (one PCIe round trip), staged in shared
                // memory, then quantised from there.
                const float4* xh = reinterpret_cast<const float4*>(p.x_host);
                float4* stage = reinterpret_cast<float4*>(smem + p.xs_offset);   // 1024 float4
                const uint32_t n_f4 = p.n_pos * 16u;
                for (uint32_t pos0 = bid * 64u; pos0 < p.x_pitch; pos0 += p.x_n_prod * 64u) {
                    for (uint32_t base = 0; base < 1024u; base += 8u * blockDim.x) {   // one round for >= 128 threads
                        float4 v[8];
                        if (host_first_valid && pos0 == bid * 64u) {   // already on their way (base is 0 here)
#pragma unroll
                            for (int u = 0; u < 8; ++u) v[u] = host_first[u];
                        } else {
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const uint32_t idx = base + u * blockDim.x + tid, gi = pos0 * 16u + idx;
                                v[u] = idx < 1024u && gi < n_f4 ? __ldg(xh + gi) : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const uint32_t idx = base + u * blockDim.x + tid;
                            if (idx < 1024u) stage[idx] = v[u];
                        }
                    }
                    __syncthreads();
                    (void)quantize_x_positions_from(
                        [&](uint32_t i, float4* w) {
#pragma unroll
                            for (int u = 0; u < 4; ++u) w[u] = stage[i - pos0 * 16u + u];
                        },
                        image, reinterpret_cast<float4*>(image + 16u * p.x_pitch), p.n_pos, min(pos0 + 64u, p.x_pitch),
                        p.x_pitch, tid, blockDim.x, pos0);
                    __syncthreads();
                }
                __threadfence();
                __syncthreads();
                if (tid == 0) {
                    bool last = p.x_n_prod == 1u;   // a single producer publishes at once
                    if (!last && atomicAdd(p.x_prod_counter, 1u) == p.x_n_prod - 1u) {
                        *p.x_prod_counter = 0;
                        __threadfence();
                        last = true;
                    }
                    if (last) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.x_ready), "r"(p.x_seq) : "memory");
                }
            }
            if (tid == 0) {
                uint32_t it = 0, got = 0;
                for (; it < (1u << 22); ++it) {
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(got) : "l"(p.x_ready) : "memory");
                    if (got == p.x_seq) break;
                    __nanosleep(20);
                }
                if (it == (1u << 22) && p.status) atomicOr(p.status, ERR_BULK_WAIT_TIMEOUT);
            }
            __syncthreads();
        }
    } else if constexpr (XFUSE) {
        uint32_t x_epoch = 0;
        if (p.x_pairs || p.x2_pairs)
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(x_epoch) : "l"(p.x_epoch_ptr) : "memory");
        PairWait pw;
        const float4* xa = reinterpret_cast<const float4*>(p.x);
        const float4* xb = reinterpret_cast<const float4*>(p.x2);
        const size_t x_par = (size_t)(x_epoch & 1u) * (p.x_parity_stride >> 3);   // in words
        const uint64_t* xp1 = p.x_pairs ? p.x_pairs + x_par : nullptr;
        const uint64_t* xp2 = p.x2_pairs ? p.x2_pairs + x_par : nullptr;
        float sq = quantize_x_positions_from(
            [&](uint32_t i, float4* v) {
                if (xp1) {
                    load_pairs16(xp1, i, x_epoch, pw, v);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = __ldg(xa + i + u);
                }
                if (xp2 || xb) {
                    float4 w[4];
                    if (xp2) {
                        load_pairs16(xp2, i, x_epoch, pw, w);
                    } else {
#pragma unroll
                        for (int u = 0; u < 4; ++u) w[u] = __ldg(xb + i + u);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        v[u].x += w[u].x, v[u].y += w[u].y, v[u].z += w[u].z, v[u].w += w[u].w;
                }
            },
            xs, xm, p.n_pos, p.x_pos_end, p.x_pitch, tid, blockDim.x);
        report_pair_wait(pw, p.status);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
        if (lane == 0) sumsq_part[warp] = sq;
    } else {
        quantize_x_positions(p.x, xs, xm, p.n_pos, p.x_pos_end, p.x_pitch, tid, blockDim.x);
    }
    if (!p.prefetch_first) start_stream();
    if constexpr (!PREPARED) __syncthreads();

    LaneCtx ctx;
    {
        const uint32_t h16 = (c & 1u) * 16u;
        ctx.big = c >= 2;
        ctx.sh0 = h16;
        ctx.sh_m = ctx.big ? h16 + 4 : h16;
        ctx.sh2 = h16 + 2;
        ctx.mask_a = ctx.big ? 0x0F0Fu : 0x3F3Fu;
        ctx.mask_b = ctx.big ? 0x3030u : 0u;
        const uint32_t pos = active ? my_pos : 0u;
        const uint4* xs_src = PREPARED ? reinterpret_cast<const uint4*>(p.x_prepared) : xs;
        const float4* xm_src = PREPARED ? reinterpret_cast<const float4*>(xs_src + 16u * p.x_pitch) : xm;
        // a prepared image may have been written by CTAs of this very launch: read it through L2
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const uint4* src = xs_src + k * p.x_pitch + (pos ^ (uint32_t)(k & 7));
            const uint4 a = PREPARED ? __ldcg(src) : *src;
            ctx.dg[k][0] = a.x, ctx.dg[k][1] = a.y, ctx.dg[k][2] = a.z;
        }
        const float4 meta = PREPARED ? __ldcg(xm_src + pos) : xm_src[pos];
        ctx.ps_a = meta.z, ctx.ps_b = meta.w;
        // sums of each digit over a group of columns: bytes dotted with ones (exact)
        auto digit_sums = [&](int k0, int nk, int (&out)[3]) {
            uint32_t s0 = 0, s1 = 0;
            int s2 = 0;
#pragma unroll
            for (int k = k0; k < k0 + nk; ++k) {
                dp4a_uu(s0, ctx.dg[k][0], 0x01010101u);
                dp4a_uu(s1, ctx.dg[k][1], 0x01010101u);
                dp4a_us(s2, 0x01010101u, ctx.dg[k][2]);
            }
            out[0] = (int)s0, out[1] = (int)s1, out[2] = s2;
        };
        if constexpr (FMT == FMT_Q4K) {
            int a[3], b[3];
            digit_sums(0, 8, a);
            digit_sums(8, 8, b);
            // |sum of 32 values below 2^23| < 2^28: exact in int32
            ctx.sum_a = ((float)(a[0] + 256 * a[1] + 65536 * a[2]) * meta.z) * meta.w + meta.x;
            ctx.sum_b = ((float)(b[0] + 256 * b[1] + 65536 * b[2]) * meta.z) * meta.w + meta.y;
        } else {
            ctx.sum_a = meta.x, ctx.sum_b = meta.y;
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                int lo[3], hi[3];
                digit_sums(8 * blk, 4, lo);
                digit_sums(8 * blk + 4, 4, hi);
#pragma unroll
                for (int d = 0; d < 3; ++d) ctx.q40_lo[blk][d] = -8 * lo[d], ctx.q40_hi[blk][d] = -128 * hi[d];
            }
        }
    }

    // Lanes past the end of the row read position 0 and are zeroed below.
    const uint32_t pos_off = !active ? 0u : FMT == FMT_Q4K ? (my_pos >> 2) * Q4K_SB_BYTES : my_pos * 36u;
    const uint8_t* lane_base = ring + pos_off + row_in_pass * row_bytes;
    // Offset of the tile's first byte inside its 16-byte aligned copy (always 0 for Q4_K_M).
    uint32_t delta = (r0 * row_bytes) & 15u;
    const uint32_t delta_step = (p.tile_rows * row_bytes) & 15u;
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
        const uint8_t* sp = lane_base + s * p.stage_bytes + delta;

        float v[PASSES];
        if (rows_left >= p.tile_rows) {
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps)
                v[ps] = FMT == FMT_Q4K ? q4k_pos_dot(sp + ps * pass_stride, qs_off, ctx)
                                       : q40_pos_dot(sp + ps * pass_stride, ctx);
        } else {
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps)
                v[ps] = ps * p.rows_per_pass + row_in_pass >= rows_left ? 0.0f
                        : FMT == FMT_Q4K ? q4k_pos_dot(sp + ps * pass_stride, qs_off, ctx)
                                         : q40_pos_dot(sp + ps * pass_stride, ctx);
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
        delta = (delta + delta_step) & 15u;
        if (++s == p.stages) s = 0, parity ^= 1u;
    }

    __syncthreads();
    if (p.independent) {
        asm volatile("griddepcontrol.wait;" ::: "memory");  // stream order for y
        if constexpr (GATHER)
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(p.epoch_ptr) : "memory");
    }
    // x / sqrt(mean(x^2)) as input = the plain result times 1 / sqrt(mean(x^2)).
    float out_scale = 1.0f;
    if constexpr (PREPARED) {
        if (p.x_prepared_rms) {   // partial sums of x^2, one per 64 positions, behind the image
            const float* partial = reinterpret_cast<const float*>(reinterpret_cast<const uint4*>(p.x_prepared) +
                                                                  17u * p.x_pitch);
            float tot = 0.0f;
            for (uint32_t i = 0; i < (p.n_pos + 63u) / 64u; ++i) tot += partial[i];
            out_scale = 1.0f / sqrtf(tot / (float)(p.n_pos * 64u));
        }
    }
    if constexpr (XFUSE) {
        if (p.x_unit_rms) {
            float tot = 0.0f;
            for (uint32_t w = 0; w < n_warps; ++w) tot += sumsq_part[w];
            out_scale = 1.0f / sqrtf(tot / (float)(p.n_pos * 64u));
        }
    }
    if constexpr (!GATHER) {
        for (uint32_t r = tid; r < my_rows; r += blockDim.x) {
            float sum = part[r * wpr];
            for (uint32_t wv = 1; wv < wpr; ++wv) sum += part[r * wpr + wv];
            if constexpr (XFUSE || PREPARED) sum *= out_scale;
            p.y[r0 + r] = sum;
        }
    } else {
        // All-gather fused into the epilogue: the slice goes straight into every rank's vector
        // (plain peer stores over NVLink; no multicast, no TMA on peer memory).  Each value
        // travels with the epoch in the same naturally aligned 8-byte word, so a reader that sees
        // the epoch sees the value: no fence, no flag exchange, nothing for this CTA to wait for.
        for (uint32_t r = tid; r < my_rows; r += blockDim.x) {
            float sum = part[r * wpr];
            for (uint32_t wv = 1; wv < wpr; ++wv) sum += part[r * wpr + wv];
            if constexpr (XFUSE || PREPARED) sum *= out_scale;
            const uint64_t word = ((uint64_t)epoch << 32) | (uint64_t)__float_as_uint(sum);
            const uint64_t par = (uint64_t)(epoch & 1u) * p.y_parity_stride;
            for (uint32_t pr = 0; pr < p.world; ++pr) {
                uint64_t* dst = reinterpret_cast<uint64_t*>(peer_base[pr] + par) + (p.row_offset + r0 + r);
                asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
            }
        }
    }
    if (p.done_flag) signal_cta_done(p, tid);
}

// ---------------------------------------------------------------------------------------------

// cudaFuncSetAttribute costs a microsecond or two of host time: raise a kernel's dynamic
// shared-memory limit only when a launch needs more than an earlier one set (per device).
static cudaError_t ensure_dynamic_smem(const void* kern, size_t smem) {
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, size_t> limit;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    size_t& have = limit[{dev, kern}];
    if (smem <= have) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) have = smem;
    return e;
}

template <int FMT>
static cudaError_t launch_stream(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                 uint32_t row_bytes, uint32_t n_pos, uint32_t* status,
                                 cudaStream_t stream, const MatvecTuning& tune, int sm_count,
                                 LaunchInfo* info) {
    StreamParams p{};
    p.q = q, p.x = x, p.y = y, p.status = status, p.rows = rows;
    p.x_prepared = tune.x_prepared, p.x_prepared_rms = tune.x_prepared_rms ? 1u : 0u;
    p.row_bytes = row_bytes, p.n_pos = n_pos;
    p.warps_per_row = (n_pos + 31) / 32;
    // CTA shape: whole rows per pass, about `threads` threads.  `ctas_per_sm` sizes the grid,
    // `resident` the shared-memory budget (how many CTAs should fit on an SM together; about 120
    // registers per thread allow 16 warps per SM in total).
    // Calls declared independent of the launch before them (pdl 3) overlap it on every SM: one
    // small CTA per SM per launch (two rows per pass) and shared memory cut for up to four
    // residents, so an SM holds CTAs of up to four consecutive launches and the per-CTA prologue
    // (x staging) is paid once per SM per launch.  Ordered launches cannot overlap: they fill the
    // SM themselves with larger CTAs.
    const bool overlap_launches = tune.pdl == 3 && !tune.x_prepared;
    int threads = tune.threads > 0 ? tune.threads : 256;
    if (tune.threads <= 0 && overlap_launches && p.warps_per_row <= 4) threads = 64 * (int)p.warps_per_row;
    // ordered launches of rows that need 5 to 8 warps: two rows per pass (K = 14336: 11.6 -> 10.8 us)
    if (tune.threads <= 0 && !overlap_launches && p.warps_per_row > 4 && p.warps_per_row <= 8) threads = 512;
    if (p.warps_per_row > 8) threads = 512;
    int rows_per_pass = (threads / 32) / (int)p.warps_per_row;
    if (rows_per_pass < 1) rows_per_pass = 1;
    const int warps = rows_per_pass * (int)p.warps_per_row;
    if (warps > 16) return cudaErrorInvalidConfiguration;
    p.rows_per_pass = (uint32_t)rows_per_pass;
    const int max_resident = 16 / warps > 0 ? 16 / warps : 1;
    int ctas_per_sm = tune.ctas_per_sm > 0 ? tune.ctas_per_sm : (overlap_launches ? 1 : max_resident);
    // A small matrix in an ordered chain is dominated by what every CTA does before its first row
    // (staging x): one CTA per SM halves that work per SM (1280 x 8192: 5.1 -> 4.3 us; Q4_0 4096 x
    // 4096: 4.8 -> 4.1 us); from about 12 MB on, two CTAs per SM hide more latency than that costs.
    if (tune.ctas_per_sm <= 0 && !overlap_launches && (uint64_t)rows * row_bytes < (12ull << 20)) ctas_per_sm = 1;
    if (ctas_per_sm > 16) ctas_per_sm = 16;
    int resident = tune.resident > 0 ? tune.resident
                   : overlap_launches ? (max_resident < 4 ? max_resident : 4)
                                      : (ctas_per_sm < max_resident ? ctas_per_sm : max_resident);
    if (resident > max_resident) resident = max_resident;

    uint32_t grid = (uint32_t)(sm_count * ctas_per_sm);
    // A run of independent launches: every launch takes HALF the SMs (one small CTA each), so
    // consecutive launches land on the SMs their predecessor left free and each SM pays the
    // per-CTA prologue (staging x) for every second launch only, with twice the rows to spread it
    // over (14336 x 4096: 5.64 -> 5.51 us, 4096 x 14336: 8.2 -> 7.4 us, Q4_0 4096 x 4096: 2.05 ->
    // 1.80 us, 1792 x 4096: 1.42 -> 1.12 us per call).  Not for very short rows, whose prologue is
    // cheap (K = 1024 measured slower).
    if (overlap_launches && tune.ctas_per_sm <= 0 && n_pos >= 32 && sm_count >= 2) grid = (uint32_t)(sm_count / 2);
    const uint32_t max_useful = (rows + (uint32_t)rows_per_pass - 1) / (uint32_t)rows_per_pass;
    if (grid > max_useful) grid = max_useful;
    // Keep the per-CTA partial-sum array small: more CTAs (several waves) for very tall matrices.
    const uint32_t max_part_entries = 4096;
    const uint32_t max_rows_per_cta = max_part_entries / p.warps_per_row;
    if ((rows + grid - 1) / grid > max_rows_per_cta) grid = (rows + max_rows_per_cta - 1) / max_rows_per_cta;
    if (grid < 1) grid = 1;
    const uint32_t rows_per_cta = (rows + grid - 1) / grid;
    p.part_entries = rows_per_cta * p.warps_per_row;

    const size_t smem_cap = (size_t)(227 * 1024) / resident - 1024;  // 1 KB per CTA is reserved
    p.x_pitch = (n_pos + 7) & ~7u;
    // digit words and per-position sums/scales; a prepared x is read straight into registers
    // (a launch that quantises x from host memory itself stages 16 KB of it at a time there)
    const size_t xs_bytes = tune.x_prepared ? (tune.host_x ? (size_t)16384 : 0) : (size_t)16 * p.x_pitch * 16;
    const size_t xm_bytes = tune.x_prepared ? 0 : (size_t)p.x_pitch * 16;
    const size_t fixed = (((size_t)p.part_entries * 4 + 64 + 15) & ~(size_t)15) + xs_bytes + xm_bytes;
    int passes = 4;
    if (tune.tile_rows > 0) passes = tune.tile_rows / rows_per_pass;
    if (passes >= 4) passes = 4;
    else if (passes >= 2) passes = 2;
    else passes = 1;
    // Stage capacity: Q4_K_M rows are multiples of 16 bytes; a Q4_0 tile is copied as its
    // enclosing aligned range (up to 15 bytes before and after).
    auto stage_for = [&](int ps) {
        const size_t raw = (size_t)ps * rows_per_pass * row_bytes;
        return FMT == FMT_Q4K ? raw : ((raw + 15) & ~(size_t)15) + 16;
    };
    auto tiles_for = [&](int ps) {
        return (int)((rows_per_cta + (uint32_t)(ps * rows_per_pass) - 1) / (uint32_t)(ps * rows_per_pass));
    };
    // Ring: `st` stages; when every Q4_K_M tile of the CTA has its own stage the last (partial)
    // tile only needs its own rows, so the ring is exactly the CTA's share.
    auto ring_for = [&](int ps, int st) {
        if (FMT == FMT_Q4K && st >= tiles_for(ps)) return (size_t)rows_per_cta * row_bytes;
        return (size_t)st * stage_for(ps);
    };
    auto smem_for = [&](int ps, int st) {
        return ((ring_for(ps, st) + (size_t)st * 20 + 15) & ~(size_t)15) + fixed;
    };
    while (passes > 1 && smem_for(passes, 2) > smem_cap) passes >>= 1;
    if (smem_for(passes, 1) > (size_t)227 * 1024 - 1024) return cudaErrorInvalidConfiguration;
    p.tile_rows = (uint32_t)(passes * rows_per_pass);
    p.stage_bytes = (uint32_t)stage_for(passes);
    const int tiles_per_cta = tiles_for(passes);
    int stages = tune.stages > 0 ? tune.stages : tiles_per_cta;  // whole share resident if it fits
    if (stages > tiles_per_cta) stages = tiles_per_cta;
    if (stages > 64) stages = 64;
    while (stages > 1 && smem_for(passes, stages) > smem_cap) --stages;
    const size_t smem = smem_for(passes, stages);
    p.stages = (uint32_t)stages;
    p.ring_bytes = (uint32_t)ring_for(passes, stages);
    p.xm_offset = (uint32_t)(smem - xm_bytes);
    p.xs_offset = (uint32_t)(smem - xm_bytes - xs_bytes);
    p.x_pos_end = (n_pos + 7) & ~7u;
    p.rows_base = rows / grid, p.rows_rem = rows % grid;
    p.tiles_lo = (p.rows_base + p.tile_rows - 1) / p.tile_rows;
    p.tiles_hi = (p.rows_base + 1 + p.tile_rows - 1) / p.tile_rows;
    p.evict_first = tune.evict_first > 0 ? 1u : 0u;
    p.prefetch_first = tune.pdl >= 2 || tune.pdl < 0 || tune.host_x ? 1u : 0u;
    // a prepared x is the output of the launch directly before: never read it ahead of the wait
    p.independent = tune.pdl == 3 && !tune.x_prepared ? 1u : 0u;
    if (tune.done) {
        p.done_counter = tune.done->counter, p.done_flag = tune.done->flag, p.done_seq = tune.done->seq;
        p.y_host = tune.done->y_host;
    }
    if (tune.host_x) {
        if (!tune.x_prepared) return cudaErrorInvalidValue;
        p.x_host = tune.host_x->x_host, p.x_ready = tune.host_x->ready, p.x_prod_counter = tune.host_x->counter;
        p.x_seq = tune.host_x->seq;
        p.x_n_prod = (p.x_pitch + 63u) / 64u;
        if (p.x_n_prod > grid) p.x_n_prod = grid;
    }

    void (*kern)(StreamParams) = nullptr;
    if (tune.gather) {
        const GatherArgs& g = *tune.gather;
        p.y_peer_bases = g.y_peer_bases, p.y_offset_bytes = g.y_offset_bytes, p.epoch_ptr = g.epoch_ptr;
        p.world = g.world, p.rank = g.rank, p.row_offset = g.row_offset;
        p.y_parity_stride = g.parity_stride_bytes;
    }
    if (tune.xsrc) {
        if (FMT != FMT_Q4K || tune.x_prepared) return cudaErrorInvalidValue;
        const XSource& s = *tune.xsrc;
        p.x = s.x, p.x2 = s.x2, p.x_pairs = s.x_pairs, p.x2_pairs = s.x2_pairs;
        p.x_epoch_ptr = s.epoch_ptr, p.x_unit_rms = s.unit_rms ? 1u : 0u;
        p.x_parity_stride = s.parity_stride_bytes;
        if constexpr (FMT == FMT_Q4K) {
            if (tune.gather) {
                switch (passes) {
                    case 1: kern = q4_matvec_stream_kernel<FMT, 1, false, true, true>; break;
                    case 2: kern = q4_matvec_stream_kernel<FMT, 2, false, true, true>; break;
                    default: kern = q4_matvec_stream_kernel<FMT, 4, false, true, true>; break;
                }
            } else {
                switch (passes) {
                    case 1: kern = q4_matvec_stream_kernel<FMT, 1, false, false, true>; break;
                    case 2: kern = q4_matvec_stream_kernel<FMT, 2, false, false, true>; break;
                    default: kern = q4_matvec_stream_kernel<FMT, 4, false, false, true>; break;
                }
            }
        }
    } else if (tune.gather && tune.x_prepared) {
        switch (passes) {
            case 1: kern = q4_matvec_stream_kernel<FMT, 1, true, true, false>; break;
            case 2: kern = q4_matvec_stream_kernel<FMT, 2, true, true, false>; break;
            default: kern = q4_matvec_stream_kernel<FMT, 4, true, true, false>; break;
        }
    } else if (tune.gather) {
        switch (passes) {
            case 1: kern = q4_matvec_stream_kernel<FMT, 1, false, true, false>; break;
            case 2: kern = q4_matvec_stream_kernel<FMT, 2, false, true, false>; break;
            default: kern = q4_matvec_stream_kernel<FMT, 4, false, true, false>; break;
        }
    } else if (tune.x_prepared) {
        switch (passes) {
            case 1: kern = q4_matvec_stream_kernel<FMT, 1, true, false, false>; break;
            case 2: kern = q4_matvec_stream_kernel<FMT, 2, true, false, false>; break;
            default: kern = q4_matvec_stream_kernel<FMT, 4, true, false, false>; break;
        }
    } else {
        switch (passes) {
            case 1: kern = q4_matvec_stream_kernel<FMT, 1, false, false, false>; break;
            case 2: kern = q4_matvec_stream_kernel<FMT, 2, false, false, false>; break;
            default: kern = q4_matvec_stream_kernel<FMT, 4, false, false, false>; break;
        }
    }
    if (info) {
        info->grid = (int)grid, info->block = warps * 32, info->smem = smem;
        info->tile_rows = (int)p.tile_rows, info->stages = stages, info->seg = (int)n_pos;
        info->n_seg = 1;
    }
    if (tune.dry_run) return cudaSuccess;
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem);
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

// Consumer side of the fused all-gather: waits until every (value, epoch) word of `pairs` carries
// the current epoch and writes the values out as a plain fp32 vector.  Bounded (about two seconds
// per element that never arrives), then ERR_PEER_WAIT_TIMEOUT and the stale value is written; a
// word from a later epoch (a producer ran ahead: the storage was reused too early) sets
// ERR_EPOCH_AHEAD.  With `overlap` the kernel does not wait for the launch before it (whose words
// it polls for anyway): the caller guarantees that launch neither advances the epoch nor touches
// `out`.  With `sync` the last CTA to finish ends the step for this rank: it tells every rank that
// this rank has consumed epoch e (a peer store into each rank's `done` array), waits (bounded)
// until every rank has consumed epoch e - 1, i.e. until the copy of the storage that epoch e + 1
// writes into is free everywhere, and advances the epoch counter.
struct FinishSync {
    const uint64_t* done_peer_bases;  // device array [world]: address of each rank's uint32 done[world]
    const uint32_t* done_local;       // this rank's own done[world]
    uint32_t* arrive_counter;         // CTAs of this launch that are done; reset by the last one
    uint32_t* epoch_rw;               // the epoch counter, advanced at the end
    uint32_t world, rank;
};

__global__ void gather_finish_kernel(const uint64_t* __restrict__ pairs, const uint32_t* __restrict__ epoch_ptr,
                                     float* __restrict__ out, uint32_t n, uint32_t* status, uint32_t overlap,
                                     uint64_t parity_stride, const FinishSync sync) {
    // bit 0 of `overlap`: do not wait for the launch before this one; bit 1: let the launches behind
    // this one be scheduled at once (they then overlap this kernel as independent matvec launches
    // overlap each other: the caller states that they read nothing this launch writes before their
    // own dependency wait).
    if (overlap & 2u) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!(overlap & 1u)) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!(overlap & 2u)) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // ordered: only after the wait
    uint32_t epoch;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(epoch_ptr) : "memory");
    pairs += (size_t)(epoch & 1u) * (parity_stride >> 3);
    bool gave_up = false, ahead = false;
    // Eight words per thread are requested together (one round trip to L2 for all of them when they
    // have arrived, which is the common case); a word that has not is then polled on its own.
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t base = blockIdx.x * blockDim.x + threadIdx.x; base < n; base += 8u * stride) {
        uint64_t w8[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t i = base + (uint32_t)u * stride;
            w8[u] = 0;
            if (i < n) asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w8[u]) : "l"(pairs + i) : "memory");
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t i = base + (uint32_t)u * stride;
            if (i >= n) continue;
            uint64_t w = w8[u];
            int32_t d = (int32_t)((uint32_t)(w >> 32) - epoch);
            if (d < 0) {
                uint32_t it = gave_up ? (1u << 22) - 1u : 0u;   // after one timeout the rest get a single look
                for (; it < (1u << 22); ++it) {
                    __nanosleep(100);
                    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(pairs + i) : "memory");
                    d = (int32_t)((uint32_t)(w >> 32) - epoch);
                    if (d >= 0) break;
                }
                if (it == (1u << 22)) gave_up = true;
            }
            if (d > 0) ahead = true;
            out[i] = __uint_as_float((uint32_t)w);
        }
    }
    if (status) {
        if (gave_up) atomicOr(status, ERR_PEER_WAIT_TIMEOUT);
        if (ahead) atomicOr(status, ERR_EPOCH_AHEAD);
    }
    if (sync.arrive_counter == nullptr) return;
    __syncthreads();   // every thread of the CTA has read its words
    if (threadIdx.x != 0) return;
    __threadfence();
    if (atomicAdd(sync.arrive_counter, 1u) != gridDim.x - 1) return;
    *sync.arrive_counter = 0;   // for the next launch (stream order)
    for (uint32_t r = 0; r < sync.world; ++r) {
        uint32_t* dst = reinterpret_cast<uint32_t*>(sync.done_peer_bases[r]) + sync.rank;
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
    }
    bool late = false;
    for (uint32_t r = 0; r < sync.world; ++r) {
        uint32_t it = 0;
        for (; it < (1u << 22); ++it) {
            uint32_t d;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(d) : "l"(sync.done_local + r) : "memory");
            if ((int32_t)(d - (epoch - 1u)) >= 0) break;
            __nanosleep(100);
        }
        late = late || it == (1u << 22);
    }
    if (late && status) atomicOr(status, ERR_PEER_WAIT_TIMEOUT);
    *sync.epoch_rw = epoch + 1u;
}

__global__ void gather_next_epoch_kernel(uint32_t* epoch_ptr) { *epoch_ptr += 1; }

// Consumer side of a K-sharded linear: every rank stored its full-length vector of PARTIAL sums
// into its own part of the (value, epoch) storage of every rank (the all-gather epilogue with
// row offset 0 and one part per rank); this kernel waits (bounded, as gather_finish_kernel) for
// all `n_parts` words of each element and writes their sum, taken in part order on every rank
// (so all ranks obtain bit-identical vectors), as a plain fp32 vector.
__global__ void gather_reduce_finish_kernel(const uint64_t* __restrict__ pairs, const uint32_t* __restrict__ epoch_ptr,
                                            float* __restrict__ out, uint32_t n, uint32_t n_parts, uint64_t part_stride,
                                            uint32_t* status, uint32_t overlap, uint64_t parity_stride) {
    if (!overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t epoch;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(epoch_ptr) : "memory");
    pairs += (size_t)(epoch & 1u) * (parity_stride >> 3);
    const size_t stride_w = part_stride >> 3;
    bool gave_up = false, ahead = false;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float sum = 0.0f;
        uint32_t pending = n_parts >= 32u ? 0xFFFFFFFFu : (1u << n_parts) - 1u;
        float part[16];
        uint32_t it = gave_up ? (1u << 22) - 1u : 0u;
        for (; pending && it < (1u << 22); ++it) {
            // all pending parts are requested before the first is looked at: one round trip, not one per part
            uint64_t w[16];
#pragma unroll
            for (uint32_t r = 0; r < 16u; ++r) {
                w[r] = 0;
                if (r < n_parts && (pending >> r & 1u))
                    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w[r]) : "l"(pairs + r * stride_w + i) : "memory");
            }
#pragma unroll
            for (uint32_t r = 0; r < 16u; ++r) {
                if (r < n_parts && (pending >> r & 1u)) {
                    const int32_t d = (int32_t)((uint32_t)(w[r] >> 32) - epoch);
                    if (d >= 0) {
                        part[r] = __uint_as_float((uint32_t)w[r]);
                        pending &= ~(1u << r);
                        ahead = ahead || d > 0;
                    }
                }
            }
            if (pending) __nanosleep(100);
        }
        if (pending) {
            gave_up = true;
#pragma unroll
            for (uint32_t r = 0; r < 16u; ++r)
                if (pending >> r & 1u) part[r] = 0.0f;
        }
#pragma unroll
        for (uint32_t r = 0; r < 16u; ++r)
            if (r < n_parts) sum += part[r];
        out[i] = sum;
    }
    if (status) {
        if (gave_up) atomicOr(status, ERR_PEER_WAIT_TIMEOUT);
        if (ahead) atomicOr(status, ERR_EPOCH_AHEAD);
    }
}

cudaError_t launch_gather_reduce_finish(const uint64_t* pairs, const uint32_t* epoch_ptr, float* out, uint32_t n,
                                        uint32_t n_parts, uint64_t part_stride, uint32_t* status, cudaStream_t stream,
                                        bool overlap, uint64_t parity_stride) {
    if (n == 0) return cudaSuccess;
    if (n_parts == 0 || n_parts > 16) return cudaErrorInvalidValue;
    uint32_t blocks = (n + 127) / 128;
    if (blocks > 592) blocks = 592;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks), cfg.blockDim = dim3(128), cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_reduce_finish_kernel, pairs, epoch_ptr, out, n, n_parts, part_stride, status,
                              overlap ? 1u : 0u, parity_stride);
}

cudaError_t launch_gather_finish(const uint64_t* pairs, const uint32_t* epoch_ptr, float* out, uint32_t n,
                                 uint32_t* status, cudaStream_t stream, bool overlap, uint64_t parity_stride,
                                 const GatherSync* gs, bool let_next_start) {
    if (n == 0 && !gs) return cudaSuccess;
    uint32_t blocks = (n + 255) / 256;
    // A launch that lets its successors start sits on the SMs beside them while it waits for the
    // launch before it: one CTA per SM, so that it does not take their registers.
    const uint32_t cap = let_next_start ? 148u : 592u;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    FinishSync fs{};
    if (gs) {
        fs.done_peer_bases = gs->done_peer_bases, fs.done_local = gs->done_local;
        fs.arrive_counter = gs->arrive_counter, fs.epoch_rw = gs->epoch_rw, fs.world = gs->world, fs.rank = gs->rank;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks), cfg.blockDim = dim3(256), cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_finish_kernel, pairs, epoch_ptr, out, n, status,
                              (overlap ? 1u : 0u) | (let_next_start ? 2u : 0u), parity_stride, fs);
}

cudaError_t launch_gather_next_epoch(uint32_t* epoch_ptr, cudaStream_t stream) {
    gather_next_epoch_kernel<<<1, 1, 0, stream>>>(epoch_ptr);
    return cudaGetLastError();
}

// Stand-alone quantisers: they write what the matvec kernel otherwise builds in shared memory
// (uint4 digit words [16][pitch], float4 metadata [pitch], then 32 floats: the sum of x^2 of
// each group of 64 positions) to global memory, once per vector, for every CTA of the consumer.
__global__ void q4_quantize_x_kernel(const float* __restrict__ x, uint4* __restrict__ out, uint32_t n_pos,
                                     uint32_t pitch) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    quantize_x_positions(x, out, reinterpret_cast<float4*>(out + 16 * pitch), n_pos, pitch, pitch,
                         threadIdx.x, blockDim.x);
}

// The same from a fused source (x = a [+ b], plain vectors or (value, epoch) words of an
// all-gather): one CTA per 64 positions.  Optionally also writes x as a plain fp32 vector.
// `overlap`: do not wait for the launch before (the sources are epoch words it polls for).
struct PrepareParams {
    const float* x;
    const float* x2;
    const uint64_t* x_pairs;
    const uint64_t* x2_pairs;
    const uint32_t* epoch_ptr;
    uint64_t parity_stride;
    uint4* image;
    float* plain_out;
    uint32_t* status;
    uint32_t n_pos, pitch, overlap;
};

__global__ void __launch_bounds__(256) q4_prepare_x_kernel(const PrepareParams p) {
    if (!p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // ordered: only after the wait
    __shared__ float warp_sq[8];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint32_t epoch = 0;
    if (p.x_pairs || p.x2_pairs)
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(p.epoch_ptr) : "memory");
    PairWait pw;
    const float4* xa = reinterpret_cast<const float4*>(p.x);
    const float4* xb = reinterpret_cast<const float4*>(p.x2);
    const size_t x_par = (size_t)(epoch & 1u) * (p.parity_stride >> 3);
    const uint64_t* xp1 = p.x_pairs ? p.x_pairs + x_par : nullptr;
    const uint64_t* xp2 = p.x2_pairs ? p.x2_pairs + x_par : nullptr;
    float4* po = reinterpret_cast<float4*>(p.plain_out);
    // whole warps stay in the loop together (it shuffles): the end is rounded up to 8 positions,
    // positions past n_pos are skipped inside
    const uint32_t pos0 = blockIdx.x * 64u;
    const uint32_t pos1 = min(pos0 + 64u, p.pitch);
    float sq = quantize_x_positions_from(
        [&](uint32_t i, float4* v) {
            if (xp1) {
                load_pairs16(xp1, i, epoch, pw, v);
            } else {
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = __ldg(xa + i + u);
            }
            if (xp2 || xb) {
                float4 w[4];
                if (xp2) {
                    load_pairs16(xp2, i, epoch, pw, w);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) w[u] = __ldg(xb + i + u);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u].x += w[u].x, v[u].y += w[u].y, v[u].z += w[u].z, v[u].w += w[u].w;
            }
            if (po) {
#pragma unroll
                for (int u = 0; u < 4; ++u) po[i + u] = v[u];
            }
        },
        p.image, reinterpret_cast<float4*>(p.image + 16u * p.pitch), p.n_pos, pos1, p.pitch, tid, blockDim.x, pos0);
    report_pair_wait(pw, p.status);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, o);
    if (lane == 0) warp_sq[warp] = sq;
    __syncthreads();
    if (tid == 0) {
        float tot = 0.0f;
        for (uint32_t w = 0; w < 8u; ++w) tot += warp_sq[w];
        reinterpret_cast<float*>(p.image + 17u * p.pitch)[blockIdx.x] = tot;
    }
}

// Loads (without launching) the kernels of the prepared-x Q4_K_M path on the current device: the
// stand-alone quantiser and the three tile heights of the matvec.  With lazy module loading the
// first use of a kernel otherwise loads it at that moment, which may allocate device memory.
cudaError_t preload_q4k_prepared_path() {
    cudaFuncAttributes a;
    cudaError_t e = cudaFuncGetAttributes(&a, q4_quantize_x_kernel);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, q4_matvec_stream_kernel<FMT_Q4K, 1, true, false, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, q4_matvec_stream_kernel<FMT_Q4K, 2, true, false, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, q4_matvec_stream_kernel<FMT_Q4K, 4, true, false, false>);
    if (e == cudaSuccess) {
        // the largest dynamic shared-memory request any launch of these kernels makes
        const size_t smem = (size_t)227 * 1024 - 1024;
        e = ensure_dynamic_smem(reinterpret_cast<const void*>(q4_matvec_stream_kernel<FMT_Q4K, 1, true, false, false>), smem);
        if (e == cudaSuccess) e = ensure_dynamic_smem(reinterpret_cast<const void*>(q4_matvec_stream_kernel<FMT_Q4K, 2, true, false, false>), smem);
        if (e == cudaSuccess) e = ensure_dynamic_smem(reinterpret_cast<const void*>(q4_matvec_stream_kernel<FMT_Q4K, 4, true, false, false>), smem);
    }
    return e;
}

size_t q4_prepared_x_bytes(uint32_t n_pos) { return (size_t)17 * ((n_pos + 7) & ~7u) * 16 + 128; }

cudaError_t launch_q4_quantize_x(const float* x, void* out, uint32_t n_pos, cudaStream_t stream) {
    if (n_pos == 0) return cudaSuccess;
    const uint32_t pitch = (n_pos + 7) & ~7u;
    q4_quantize_x_kernel<<<1, 512, 0, stream>>>(x, reinterpret_cast<uint4*>(out), n_pos, pitch);
    return cudaGetLastError();
}

cudaError_t launch_q4_prepare_x(const XSource& src, void* image, float* plain_out, uint32_t n_pos, uint32_t* status,
                                cudaStream_t stream, bool overlap) {
    if (n_pos == 0) return cudaSuccess;
    if (n_pos > 2048) return cudaErrorInvalidValue;   // 32 partial sums of 64 positions each
    PrepareParams p{};
    p.x = src.x, p.x2 = src.x2, p.x_pairs = src.x_pairs, p.x2_pairs = src.x2_pairs, p.epoch_ptr = src.epoch_ptr;
    p.parity_stride = src.parity_stride_bytes;
    p.image = reinterpret_cast<uint4*>(image), p.plain_out = plain_out, p.status = status;
    p.n_pos = n_pos, p.pitch = (n_pos + 7) & ~7u, p.overlap = overlap ? 1u : 0u;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((n_pos + 63) / 64), cfg.blockDim = dim3(256), cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, q4_prepare_x_kernel, p);
}

cudaError_t launch_q4k_matvec_segmented(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                        uint32_t n_sb, uint32_t* status, cudaStream_t stream,
                                        const MatvecTuning& tune, int sm_count, LaunchInfo* info);
cudaError_t launch_q4_0_matvec_rowwarp(const uint8_t* q, const float* x, float* y, uint32_t rows,
                                       uint32_t n_blocks, cudaStream_t stream, LaunchInfo* info);

cudaError_t launch_q4k_matvec(const uint8_t* q, const float* x, float* y, uint32_t rows,
                              uint32_t n_sb, uint32_t* status, cudaStream_t stream,
                              const MatvecTuning& tune, int sm_count, LaunchInfo* info) {
    if (rows == 0 || n_sb == 0) return cudaSuccess;
    if (n_sb > 128) return launch_q4k_matvec_segmented(q, x, y, rows, n_sb, status, stream, tune, sm_count, info);
    return launch_stream<FMT_Q4K>(q, x, y, rows, n_sb * Q4K_SB_BYTES, n_sb * 4, status, stream, tune, sm_count, info);
}

cudaError_t launch_q4_0_matvec(const uint8_t* q, const float* x, float* y, uint32_t rows,
                               uint32_t n_blocks, uint32_t* status, cudaStream_t stream,
                               const MatvecTuning& tune, int sm_count, LaunchInfo* info) {
    if (rows == 0 || n_blocks == 0) return cudaSuccess;
    if ((n_blocks & 1u) || n_blocks > 1024u) return launch_q4_0_matvec_rowwarp(q, x, y, rows, n_blocks, stream, info);
    return launch_stream<FMT_Q4_0>(q, x, y, rows, n_blocks * Q4_0_BLK_BYTES, n_blocks / 2, status, stream, tune, sm_count, info);
}

}  // namespace axc
