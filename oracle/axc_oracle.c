/*
 * axc_oracle.c -- CPU restatement of AXIOM-Compute's Q4_K_M / Q4_0 dequant-matvec
 * reference functions.  TEST INFRASTRUCTURE ONLY: nothing under the product package may
 * link, import or execute this file; it exists so that tests, the smoke check and the CPU
 * leg of the benchmark can check and time the reference algorithm.
 *
 * The reference implementation is scalar Rust that cannot be compiled where this project is
 * built (no Rust toolchain), so every function here restates one reference function, in the
 * same operation order and with the same rounding points:
 *
 *   axc_oracle_unpack_scale_min_k4   crates/axc-driver/tests/common_helpers.rs:365-381
 *   axc_oracle_q4km_dequant_matvec   crates/axc-driver/tests/common_helpers.rs:411-461
 *   axc_oracle_q4_0_dequant_matvec   crates/axc-driver/benches/common.rs:212-259
 *   axc_oracle_generate_q4km_test_data  crates/axc-driver/tests/common_helpers.rs:476-519
 *   axc_oracle_q4km_axc_body         examples/q4km_dequant_matvec.axc:13-117  (second,
 *   axc_oracle_q4_0_axc_body         examples/q4_0_dequant_matvec.axc:13-51    independent
 *                                    restatement made from the kernel source itself)
 *   f16 <-> f32                      `half` crate 2.7.1 (Cargo.lock:478-479), a third-party
 *                                    dependency not vendored in the reference: IEEE-754
 *                                    binary16 <-> binary32, exact widening, round-to-nearest-
 *                                    even narrowing.
 *
 * Parity pinning: the reference stores no numeric outputs for its random fixtures (its tests
 * compute CPU and GPU in the same run).  What it does pin, and what tests/ check this file
 * against, are its known-answer tests: the eight hand-verified scale/min pairs and the
 * s[j]-not-s[j-4] discriminator of AT-1312 (compile_q4km_dequant_matvec.rs:484-584), the
 * Q4_0 layout fixtures -128.0 / -96.0 (common_helpers.rs:272-333) and "n = 0 gives +0.0"
 * (compile_q4km_dequant_matvec.rs:850-856).  Beyond those, the two restatements in this
 * file and a numpy twin must agree bit for bit on the reference's LCG fixture.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -pthread -shared -fPIC (see Makefile).
 * -ffp-contract=off matters: the reference rounds every product before the add.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#include <math.h>
#include <pthread.h>
#include <unistd.h>

#define Q4KM_SB_BYTES 144
#define Q4KM_SB_ELEMS 256
#define Q4_0_BLK_BYTES 18
#define Q4_0_BLK_ELEMS 32

/* ---- binary16 <-> binary32 (what half::f16::{from_bits,to_f32,from_f32} compute) ---- */

float axc_oracle_f16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13); /* Inf / NaN payload kept */
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t axc_oracle_f32_to_f16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFF) { /* Inf / NaN */
        if (man == 0) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7C00u | 0x200u | (man >> 13));
    }
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u); /* overflow -> Inf */
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign; /* underflow -> signed zero */
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++; /* may carry into exp: correct */
    return (uint16_t)(sign | half);
}

/* ---- get_scale_min_k4 (common_helpers.rs:365-381) ---- */

void axc_oracle_unpack_scale_min_k4(const uint8_t* scales, int j, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = scales[j] & 63;
        *m = scales[j + 4] & 63;
    } else {
        uint8_t sc_lo = scales[j + 4] & 0x0F;
        uint8_t sc_hi = (scales[j - 4] >> 6) & 0x03;
        *sc = (uint8_t)(sc_lo | (sc_hi << 4));
        uint8_t m_lo = (scales[j + 4] >> 4) & 0x0F;
        uint8_t m_hi = (scales[j] >> 6) & 0x03; /* scales[j], not scales[j-4] */
        *m = (uint8_t)(m_lo | (m_hi << 4));
    }
}

/* Inverse of the above: pack eight (sc, m) pairs, each 0..63, into the 12-byte field.
 * Has no reference counterpart (the reference only unpacks); it exists so that synthetic
 * inputs "6-bit scale and min uniform 0..63, packed in ggml layout" can be generated. */
void axc_oracle_pack_scale_min_k4(const uint8_t* sc, const uint8_t* m, uint8_t* scales) {
    for (int j = 0; j < 4; j++) {
        scales[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        scales[j + 4] = (uint8_t)((m[j] & 63) | ((m[j + 4] >> 4) << 6));
        scales[j + 8] = (uint8_t)((sc[j + 4] & 0x0F) | ((m[j + 4] & 0x0F) << 4));
    }
}

/* ---- Q4_K_M: one row = one reference call (common_helpers.rs:411-461) ---- */

static inline float q4km_row_seq(const uint8_t* q, const float* x, size_t n_sb) {
    float sum = 0.0f;
    for (size_t sb = 0; sb < n_sb; sb++) {
        size_t base = sb * Q4KM_SB_BYTES;
        float d = axc_oracle_f16_bits_to_f32((uint16_t)(q[base] | (q[base + 1] << 8)));
        float dmin = axc_oracle_f16_bits_to_f32((uint16_t)(q[base + 2] | (q[base + 3] << 8)));
        const uint8_t* scales = q + base + 4;
        for (size_t chunk = 0; chunk < 4; chunk++) {
            uint8_t sc0, m0, sc1, m1;
            axc_oracle_unpack_scale_min_k4(scales, (int)(chunk * 2), &sc0, &m0);
            axc_oracle_unpack_scale_min_k4(scales, (int)(chunk * 2 + 1), &sc1, &m1);
            float d1 = d * (float)sc0;
            float m1f = dmin * (float)m0;
            float d2 = d * (float)sc1;
            float m2f = dmin * (float)m1;
            size_t qs = base + 16 + chunk * 32;
            const float* xs = x + sb * Q4KM_SB_ELEMS + chunk * 64;
            for (size_t l = 0; l < 32; l++) {
                uint8_t byte = q[qs + l];
                float lo = (float)(byte & 0x0F);
                float hi = (float)((byte >> 4) & 0x0F);
                float lo_f = d1 * lo - m1f;
                float hi_f = d2 * hi - m2f;
                sum += lo_f * xs[l];
                sum += hi_f * xs[32 + l];
            }
        }
    }
    return sum;
}

float axc_oracle_q4km_dequant_matvec(const uint8_t* q, const float* x, size_t n_superblocks) {
    return q4km_row_seq(q, x, n_superblocks);
}

/* Dequantised weights of one row, element order = x index order. */
void axc_oracle_q4km_dequant_row(const uint8_t* q, size_t n_sb, float* w) {
    for (size_t sb = 0; sb < n_sb; sb++) {
        size_t base = sb * Q4KM_SB_BYTES;
        float d = axc_oracle_f16_bits_to_f32((uint16_t)(q[base] | (q[base + 1] << 8)));
        float dmin = axc_oracle_f16_bits_to_f32((uint16_t)(q[base + 2] | (q[base + 3] << 8)));
        const uint8_t* scales = q + base + 4;
        for (size_t chunk = 0; chunk < 4; chunk++) {
            uint8_t sc0, m0, sc1, m1;
            axc_oracle_unpack_scale_min_k4(scales, (int)(chunk * 2), &sc0, &m0);
            axc_oracle_unpack_scale_min_k4(scales, (int)(chunk * 2 + 1), &sc1, &m1);
            float d1 = d * (float)sc0, m1f = dmin * (float)m0;
            float d2 = d * (float)sc1, m2f = dmin * (float)m1;
            size_t qs = base + 16 + chunk * 32;
            float* ws = w + sb * Q4KM_SB_ELEMS + chunk * 64;
            for (size_t l = 0; l < 32; l++) {
                uint8_t byte = q[qs + l];
                ws[l] = d1 * (float)(byte & 0x0F) - m1f;
                ws[32 + l] = d2 * (float)((byte >> 4) & 0x0F) - m2f;
            }
        }
    }
}

/* ---- Q4_0: one row = one reference call (benches/common.rs:212-259) ---- */

static inline float q4_0_row_seq(const uint8_t* q, const float* x, size_t n_blocks) {
    float acc = 0.0f;
    for (size_t b = 0; b < n_blocks; b++) {
        size_t off = b * Q4_0_BLK_BYTES;
        float scale = axc_oracle_f16_bits_to_f32((uint16_t)(q[off] | (q[off + 1] << 8)));
        const float* xs = x + b * Q4_0_BLK_ELEMS;
        for (size_t k = 0; k < 16; k++) {
            uint8_t packed = q[off + 2 + k];
            float w_lo = ((float)(packed & 0x0F) - 8.0f) * scale;
            acc += w_lo * xs[k];
            float w_hi = ((float)((packed >> 4) & 0x0F) - 8.0f) * scale;
            acc += w_hi * xs[k + 16];
        }
    }
    return acc;
}

float axc_oracle_q4_0_dequant_matvec(const uint8_t* q, const float* x, size_t n_blocks) {
    return q4_0_row_seq(q, x, n_blocks);
}

void axc_oracle_q4_0_dequant_row(const uint8_t* q, size_t n_blocks, float* w) {
    for (size_t b = 0; b < n_blocks; b++) {
        size_t off = b * Q4_0_BLK_BYTES;
        float scale = axc_oracle_f16_bits_to_f32((uint16_t)(q[off] | (q[off + 1] << 8)));
        for (size_t k = 0; k < 16; k++) {
            uint8_t packed = q[off + 2 + k];
            w[b * 32 + k] = ((float)(packed & 0x0F) - 8.0f) * scale;
            w[b * 32 + k + 16] = ((float)((packed >> 4) & 0x0F) - 8.0f) * scale;
        }
    }
}

/* ---- second restatement: the .axc kernel bodies, written with the kernel's own u32
 *      operations (ptr_read_u8_zext / ptr_read_u16_zext / band / bor / shl / lshr /
 *      f16_bits_to_f32 / f32_from_u32), examples/q4km_dequant_matvec.axc:17-115 ---- */

static inline uint32_t rd8(const uint8_t* q, uint32_t off) { return (uint32_t)q[off]; }
static inline uint32_t rd16(const uint8_t* q, uint32_t off) {
    return (uint32_t)q[off] | ((uint32_t)q[off + 1] << 8);
}

static void axc_scale_min(const uint8_t* q, uint32_t scales_base, uint32_t is, uint32_t* sc,
                          uint32_t* m) {
    if (is < 4u) {
        *sc = rd8(q, scales_base + is) & 63u;
        *m = rd8(q, scales_base + is + 4u) & 63u;
    } else {
        uint32_t lo4_sc = rd8(q, scales_base + is + 4u) & 0x0Fu;
        uint32_t hi2_sc = (rd8(q, scales_base + is - 4u) >> 6) & 0x03u;
        *sc = lo4_sc | (hi2_sc << 4);
        uint32_t lo4_m = (rd8(q, scales_base + is + 4u) >> 4) & 0x0Fu;
        uint32_t hi2_m = (rd8(q, scales_base + is) >> 6) & 0x03u;
        *m = lo4_m | (hi2_m << 4);
    }
}

float axc_oracle_q4km_axc_body(const uint8_t* q, const float* x, uint32_t n_superblocks) {
    float sum = 0.0f;
    for (uint32_t sb = 0; sb < n_superblocks; sb++) {
        uint32_t base = sb * 144u;
        float d = axc_oracle_f16_bits_to_f32((uint16_t)rd16(q, base));
        float dmin = axc_oracle_f16_bits_to_f32((uint16_t)rd16(q, base + 2u));
        uint32_t scales_base = base + 4u;
        uint32_t qs_base = base + 16u;
        for (uint32_t chunk = 0; chunk < 4u; chunk++) {
            uint32_t is0 = chunk * 2u, is1 = is0 + 1u;
            uint32_t sc0, m0, sc1, m1v;
            axc_scale_min(q, scales_base, is0, &sc0, &m0);
            axc_scale_min(q, scales_base, is1, &sc1, &m1v);
            float d1 = d * (float)sc0;
            float m1f = dmin * (float)m0;
            float d2 = d * (float)sc1;
            float m2f = dmin * (float)m1v;
            for (uint32_t l = 0; l < 32u; l++) {
                uint32_t byte = rd8(q, qs_base + chunk * 32u + l);
                uint32_t lo_nib = byte & 0x0Fu;
                uint32_t hi_nib = (byte >> 4) & 0x0Fu;
                float lo_f = d1 * (float)lo_nib - m1f;
                float hi_f = d2 * (float)hi_nib - m2f;
                float x_lo = x[sb * 256u + chunk * 64u + l];
                float x_hi = x[sb * 256u + chunk * 64u + 32u + l];
                float a = lo_f * x_lo;
                float b = hi_f * x_hi;
                sum = sum + a + b; /* left to right: (sum + a) + b */
            }
        }
    }
    return sum;
}

float axc_oracle_q4_0_axc_body(const uint8_t* q, const float* x, uint32_t n_blocks) {
    float sum = 0.0f;
    for (uint32_t b = 0; b < n_blocks; b++) {
        uint32_t base = b * 18u;
        float scale = axc_oracle_f16_bits_to_f32((uint16_t)rd16(q, base));
        for (uint32_t k = 0; k < 16u; k++) {
            uint32_t byte = rd8(q, base + 2u + k);
            float lo_signed = (float)(byte & 0x0Fu) - 8.0f;
            float hi_signed = (float)((byte >> 4) & 0x0Fu) - 8.0f;
            float lo_value = lo_signed * scale;
            float hi_value = hi_signed * scale;
            float a = lo_value * x[b * 32u + k];
            float c = hi_value * x[b * 32u + k + 16u];
            sum = sum + a + c;
        }
    }
    return sum;
}

/* ---- rows x K generalisation: row r is one reference call on q[r] with the shared x ---- */

int axc_oracle_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (int)n;
}

/* Minimal static-schedule parallel-for over rows on POSIX threads: rows are independent
 * reference calls, so splitting them across host cores changes no result bit. */
typedef void (*row_fn)(long r, void* ctx);
typedef struct { row_fn fn; void* ctx; long begin, end; } row_span;

static void* row_span_run(void* p) {
    row_span* s = (row_span*)p;
    for (long r = s->begin; r < s->end; r++) s->fn(r, s->ctx);
    return NULL;
}

static void parallel_rows(long rows, int threads, row_fn fn, void* ctx) {
    if (threads <= 0) threads = axc_oracle_max_threads();
    if (threads > 256) threads = 256;
    if ((long)threads > rows) threads = rows > 0 ? (int)rows : 1;
    if (threads <= 1) {
        for (long r = 0; r < rows; r++) fn(r, ctx);
        return;
    }
    pthread_t tid[256];
    row_span span[256];
    int started = 0;
    for (int t = 0; t < threads; t++) {
        span[t].fn = fn;
        span[t].ctx = ctx;
        span[t].begin = rows * t / threads;
        span[t].end = rows * (t + 1) / threads;
        if (t == threads - 1) { /* run the last span on the calling thread */
            row_span_run(&span[t]);
        } else if (pthread_create(&tid[t], NULL, row_span_run, &span[t]) == 0) {
            started = t + 1;
        } else {
            row_span_run(&span[t]); /* could not spawn: do it here */
            tid[t] = 0;
        }
    }
    for (int t = 0; t < started; t++)
        if (tid[t]) pthread_join(tid[t], NULL);
}

typedef struct {
    const uint8_t* q; const float* x; float* y; double* y64; double* abs_sum; float* w;
    const float* a; float* c; size_t n, m_rows, n_rows;
} row_args;

static void q4km_row_job(long r, void* p) {
    row_args* a = (row_args*)p;
    a->y[r] = q4km_row_seq(a->q + (size_t)r * a->n * Q4KM_SB_BYTES, a->x, a->n);
}

void axc_oracle_q4km_matvec_rows(const uint8_t* q, const float* x, float* y, size_t rows,
                                 size_t n_sb, int threads) {
    row_args a = {0};
    a.q = q; a.x = x; a.y = y; a.n = n_sb;
    parallel_rows((long)rows, threads, q4km_row_job, &a);
}

static void q4_0_row_job(long r, void* p) {
    row_args* a = (row_args*)p;
    a->y[r] = q4_0_row_seq(a->q + (size_t)r * a->n * Q4_0_BLK_BYTES, a->x, a->n);
}

void axc_oracle_q4_0_matvec_rows(const uint8_t* q, const float* x, float* y, size_t rows,
                                 size_t n_blocks, int threads) {
    row_args a = {0};
    a.q = q; a.x = x; a.y = y; a.n = n_blocks;
    parallel_rows((long)rows, threads, q4_0_row_job, &a);
}

/* fp64 "truth" of the same dot products (weights are the bit-exact fp32 dequantised values,
 * products and sums in double) and the per-row magnitude sum_i |w_i x_i| used for the
 * norm-wise error figure.  Not a reference function; a measuring stick. */
static void q4km_f64_job(long r, void* p) {
    row_args* a = (row_args*)p;
    float w[Q4KM_SB_ELEMS];
    double s = 0.0, m = 0.0;
    for (size_t sb = 0; sb < a->n; sb++) {
        axc_oracle_q4km_dequant_row(a->q + ((size_t)r * a->n + sb) * Q4KM_SB_BYTES, 1, w);
        for (int i = 0; i < Q4KM_SB_ELEMS; i++) {
            double t = (double)w[i] * (double)a->x[sb * Q4KM_SB_ELEMS + i];
            s += t;
            m += fabs(t);
        }
    }
    a->y64[r] = s;
    if (a->abs_sum) a->abs_sum[r] = m;
}

void axc_oracle_q4km_matvec_rows_f64(const uint8_t* q, const float* x, double* y64,
                                     double* abs_sum, size_t rows, size_t n_sb, int threads) {
    row_args a = {0};
    a.q = q; a.x = x; a.y64 = y64; a.abs_sum = abs_sum; a.n = n_sb;
    parallel_rows((long)rows, threads, q4km_f64_job, &a);
}

static void q4_0_f64_job(long r, void* p) {
    row_args* a = (row_args*)p;
    float w[Q4_0_BLK_ELEMS];
    double s = 0.0, m = 0.0;
    for (size_t b = 0; b < a->n; b++) {
        axc_oracle_q4_0_dequant_row(a->q + ((size_t)r * a->n + b) * Q4_0_BLK_BYTES, 1, w);
        for (int i = 0; i < Q4_0_BLK_ELEMS; i++) {
            double t = (double)w[i] * (double)a->x[b * Q4_0_BLK_ELEMS + i];
            s += t;
            m += fabs(t);
        }
    }
    a->y64[r] = s;
    if (a->abs_sum) a->abs_sum[r] = m;
}

void axc_oracle_q4_0_matvec_rows_f64(const uint8_t* q, const float* x, double* y64,
                                     double* abs_sum, size_t rows, size_t n_blocks,
                                     int threads) {
    row_args a = {0};
    a.q = q; a.x = x; a.y64 = y64; a.abs_sum = abs_sum; a.n = n_blocks;
    parallel_rows((long)rows, threads, q4_0_f64_job, &a);
}

static void q4km_dq_job(long r, void* p) {
    row_args* a = (row_args*)p;
    axc_oracle_q4km_dequant_row(a->q + (size_t)r * a->n * Q4KM_SB_BYTES, a->n,
                                a->w + (size_t)r * a->n * Q4KM_SB_ELEMS);
}

void axc_oracle_q4km_dequant_rows(const uint8_t* q, float* w, size_t rows, size_t n_sb,
                                  int threads) {
    row_args a = {0};
    a.q = q; a.w = w; a.n = n_sb;
    parallel_rows((long)rows, threads, q4km_dq_job, &a);
}

static void q4_0_dq_job(long r, void* p) {
    row_args* a = (row_args*)p;
    axc_oracle_q4_0_dequant_row(a->q + (size_t)r * a->n * Q4_0_BLK_BYTES, a->n,
                                a->w + (size_t)r * a->n * Q4_0_BLK_ELEMS);
}

void axc_oracle_q4_0_dequant_rows(const uint8_t* q, float* w, size_t rows, size_t n_blocks,
                                  int threads) {
    row_args a = {0};
    a.q = q; a.w = w; a.n = n_blocks;
    parallel_rows((long)rows, threads, q4_0_dq_job, &a);
}

/* ---- batched prefill oracle: C[m][n] = sum_k bf16(A[m][k]) * bf16(W[n][k]), fp32
 *      accumulate in k order; W = bit-exact dequantised Q4_K_M weights rounded to bf16 (RNE).
 *      There is no reference function for M > 1; this is "dequant, then GEMM" spelled out. ---- */

static inline float bf16_round(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) { /* Inf/NaN: truncate, keep NaN a NaN */
        if (u & 0x007FFFFFu) u |= 0x00400000u;
        u &= 0xFFFF0000u;
    } else {
        u += 0x7FFFu + ((u >> 16) & 1u);
        u &= 0xFFFF0000u;
    }
    memcpy(&f, &u, 4);
    return f;
}

float axc_oracle_bf16_round(float f) { return bf16_round(f); }

static void prefill_job(long n, void* p) {
    row_args* g = (row_args*)p;
    size_t k = g->n * Q4KM_SB_ELEMS;
    float w[Q4KM_SB_ELEMS];
    for (size_t m = 0; m < g->m_rows; m++) g->c[m * g->n_rows + (size_t)n] = 0.0f;
    for (size_t sb = 0; sb < g->n; sb++) {
        axc_oracle_q4km_dequant_row(g->q + ((size_t)n * g->n + sb) * Q4KM_SB_BYTES, 1, w);
        for (int i = 0; i < Q4KM_SB_ELEMS; i++) w[i] = bf16_round(w[i]);
        for (size_t m = 0; m < g->m_rows; m++) {
            const float* am = g->a + m * k + sb * Q4KM_SB_ELEMS;
            float acc = g->c[m * g->n_rows + (size_t)n];
            for (int i = 0; i < Q4KM_SB_ELEMS; i++) acc += bf16_round(am[i]) * w[i];
            g->c[m * g->n_rows + (size_t)n] = acc;
        }
    }
}

void axc_oracle_q4km_prefill(const uint8_t* q, const float* a /* [m_rows][k] */, float* c
                             /* [m_rows][n_rows] */, size_t m_rows, size_t n_rows, size_t n_sb,
                             int threads) {
    row_args g = {0};
    g.q = q; g.a = a; g.c = c; g.n = n_sb; g.m_rows = m_rows; g.n_rows = n_rows;
    parallel_rows((long)n_rows, threads, prefill_job, &g);
}

/* ---- the reference's reproducible Q4_K_M fixture (common_helpers.rs:476-519) ---- */

static inline uint64_t lcg_next(uint64_t* s) {
    *s = *s * 6364136223846793005ULL + 1442695040888963407ULL;
    return *s;
}

void axc_oracle_generate_q4km_test_data(uint32_t n_superblocks, uint64_t seed, uint8_t* q_out,
                                        float* x_out) {
    uint64_t state = seed ^ 0x9E3779B97F4A7C15ULL;
    const float u64_max_f = (float)UINT64_MAX; /* rounds to 2^64, as `u64::MAX as f32` does */
    size_t p = 0;
    for (uint32_t i = 0; i < n_superblocks; i++) {
        float d_raw = 0.1f + ((float)lcg_next(&state) / u64_max_f) * 1.9f;
        uint16_t d16 = axc_oracle_f32_to_f16_bits(d_raw);
        q_out[p++] = (uint8_t)(d16 & 0xFF);
        q_out[p++] = (uint8_t)(d16 >> 8);
        float dmin_raw = ((float)lcg_next(&state) / u64_max_f) * 0.5f;
        uint16_t m16 = axc_oracle_f32_to_f16_bits(dmin_raw);
        q_out[p++] = (uint8_t)(m16 & 0xFF);
        q_out[p++] = (uint8_t)(m16 >> 8);
        for (int k = 0; k < 12; k++) q_out[p++] = (uint8_t)(lcg_next(&state) & 0xFF);
        for (int k = 0; k < 128; k++) q_out[p++] = (uint8_t)(lcg_next(&state) & 0xFF);
    }
    size_t nx = (size_t)n_superblocks * Q4KM_SB_ELEMS;
    for (size_t i = 0; i < nx; i++)
        x_out[i] = ((float)lcg_next(&state) / u64_max_f) * 2.0f - 1.0f;
}
