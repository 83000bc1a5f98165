/*
 * CPU oracle for meganeura's Q4/Q8 quantized matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library and
 * the timed CPU baseline of the benchmark.  Nothing in the product path
 * (meganeura_b200/) may link, import or call it.
 *
 * It is a plain-C restatement of the reference's own algorithm, function by
 * function (paths are relative to the meganeura source tree):
 *
 *   orc_quantize_q4 / orc_dequantize_q4   src/runtime.rs:2035-2102 / 2105-2138
 *   orc_quantize_q8 / orc_dequantize_q8   src/runtime.rs:2143-2188 / 2191-2215
 *   orc_f16_bits_to_f32_shader            src/codegen.rs:739-746 (q4_decode_f16)
 *   orc_dequant_q4_shader                 src/codegen.rs:748-769 (dequant_q4)
 *   orc_dequant_q8_shader                 src/codegen.rs:785-805 (dequant_q8)
 *   orc_matmul_f32                        src/shaders/matmul.wgsl:42-108 (k ascending, f32)
 *                                         + " + src[idx]" addend, src/codegen.rs:1017-1018
 *   orc_packed_bytes                      src/graph.rs:52-68 (TensorType::size_bytes)
 *
 * The only third-party arithmetic the reference uses on this path is the
 * `half` crate (half = "2"): f16::from_f32 / to_f32 are IEEE-754 binary16
 * conversions with round-to-nearest-even; they are restated below
 * (orc_f32_to_f16_bits / orc_f16_bits_to_f32_ieee).
 *
 * Parity pin: the reference cannot be compiled in this environment (no Rust
 * toolchain) and holds no byte-level golden vectors for this path.  The
 * oracle is pinned against the reference's own known-answer tests restated
 * with the same formulas and tolerances (src/runtime.rs:2221-2290,
 * tests/gpu_smoke.rs:2680-2771) and against an independent numpy restatement
 * whose byte outputs are committed under tests/golden/.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_FMT_Q4 2
#define ORC_FMT_Q8 3

/* ---- binary16 <-> binary32 (half crate semantics) ------------------------ */

static uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* IEEE binary16 -> binary32, exact (half::f16::to_f32). */
float orc_f16_bits_to_f32_ieee(uint16_t h)
{
    uint32_t sign = ((uint32_t)h >> 15) & 1u;
    uint32_t expo = ((uint32_t)h >> 10) & 0x1Fu;
    uint32_t mant = (uint32_t)h & 0x3FFu;
    if (expo == 0) {
        if (mant == 0) return bits_f32(sign << 31);
        /* subnormal: mant * 2^-24 */
        float v = (float)mant * 5.9604644775390625e-8f;
        return sign ? -v : v;
    }
    if (expo == 31) return bits_f32((sign << 31) | 0x7F800000u | (mant << 13));
    return bits_f32((sign << 31) | ((expo + 112u) << 23) | (mant << 13));
}

/* The shader's decode: exponent 0 gives +-0 (subnormals flushed), exponent 31
 * is not special-cased.  src/codegen.rs:739-746. */
float orc_f16_bits_to_f32_shader(uint16_t h)
{
    uint32_t bits = h;
    uint32_t sign = (bits >> 15) & 1u;
    uint32_t expo = (bits >> 10) & 0x1Fu;
    uint32_t mant = bits & 0x3FFu;
    uint32_t out = (sign << 31) | ((expo + 112u) << 23) | (mant << 13);
    if (expo == 0) out = sign << 31;
    return bits_f32(out);
}

/* binary32 -> binary16, round to nearest even (half::f16::from_f32). */
uint16_t orc_f32_to_f16_bits(float f)
{
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t expo = (x >> 23) & 0xFFu;
    uint32_t mant = x & 0x7FFFFFu;
    if (expo == 0xFF) {                       /* inf / nan */
        if (mant == 0) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7C00u | 0x200u | (mant >> 13));
    }
    int32_t e = (int32_t)expo - 127 + 15;     /* rebias */
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);          /* overflow -> inf */
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;                  /* underflow -> 0 */
        mant |= 0x800000u;                                   /* implicit one */
        uint32_t shift = (uint32_t)(14 - e);                 /* 14..24 */
        uint32_t half_mant = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_mant & 1u))) half_mant++;
        return (uint16_t)(sign | half_mant);
    }
    uint32_t half = ((uint32_t)e << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;   /* may carry into inf */
    return (uint16_t)(sign | half);
}

/* ---- buffer sizing -------------------------------------------------------- */

size_t orc_packed_bytes(int fmt, size_t k, size_t n)
{
    size_t blocks = (k * n + 31) / 32;
    if (fmt == ORC_FMT_Q4) return blocks * 20;
    if (fmt == ORC_FMT_Q8) return blocks * 36;
    return 0;
}

/* ---- quantizers (host, row-major [rows=K, cols=N] f32 in) ----------------- */

/* Rust `x.clamp(lo,hi) as u8/i8` after `round()`; round() is half away from zero. */
static float round_clamp(float v, float lo, float hi)
{
    float r = roundf(v);
    if (r < lo) r = lo;
    if (r > hi) r = hi;
    return r;
}

int orc_quantize_q4(const float *data, size_t rows, size_t cols, uint8_t *buf)
{
    if (rows % 32 != 0) return 1;
    size_t bpc = rows / 32, num_blocks = bpc * cols;
    memset(buf, 0, num_blocks * 20);
    for (size_t col = 0; col < cols; col++) {
        for (size_t blk = 0; blk < bpc; blk++) {
            size_t block_idx = col * bpc + blk;
            float bmin = INFINITY, bmax = -INFINITY;
            for (int i = 0; i < 32; i++) {
                float val = data[(blk * 32 + i) * cols + col];
                if (val < bmin) bmin = val;
                if (val > bmax) bmax = val;
            }
            float d = (bmax > bmin) ? (bmax - bmin) / 15.0f : 1.0f;
            float m = bmin;
            uint32_t dm = (uint32_t)orc_f32_to_f16_bits(d) | ((uint32_t)orc_f32_to_f16_bits(m) << 16);
            memcpy(buf + block_idx * 4, &dm, 4);
            size_t base = num_blocks * 4 + block_idx * 16;
            float d_inv = (d > 0.0f) ? 1.0f / d : 0.0f;
            for (int i = 0; i < 32; i++) {
                float val = data[(blk * 32 + i) * cols + col];
                uint8_t nib = (uint8_t)round_clamp((val - m) * d_inv, 0.0f, 15.0f);
                if (i % 2 == 0) buf[base + i / 2] |= nib;
                else            buf[base + i / 2] |= (uint8_t)(nib << 4);
            }
        }
    }
    return 0;
}

int orc_dequantize_q4(const uint8_t *buf, size_t rows, size_t cols, float *out)
{
    if (rows % 32 != 0) return 1;
    size_t bpc = rows / 32, num_blocks = bpc * cols;
    for (size_t col = 0; col < cols; col++) {
        for (size_t blk = 0; blk < bpc; blk++) {
            size_t block = col * bpc + blk;
            uint32_t dm; memcpy(&dm, buf + block * 4, 4);
            float d = orc_f16_bits_to_f32_ieee((uint16_t)(dm & 0xFFFFu));
            float m = orc_f16_bits_to_f32_ieee((uint16_t)(dm >> 16));
            const uint8_t *nb = buf + num_blocks * 4 + block * 16;
            for (int i = 0; i < 32; i++) {
                uint32_t nib = (i & 1) ? (nb[i / 2] >> 4) : (nb[i / 2] & 0xF);
                out[(blk * 32 + i) * cols + col] = (float)nib * d + m;
            }
        }
    }
    return 0;
}

int orc_quantize_q8(const float *data, size_t rows, size_t cols, uint8_t *buf)
{
    if (rows % 32 != 0) return 1;
    size_t bpc = rows / 32, num_blocks = bpc * cols;
    memset(buf, 0, num_blocks * 36);
    for (size_t col = 0; col < cols; col++) {
        for (size_t blk = 0; blk < bpc; blk++) {
            size_t base = (col * bpc + blk) * 36;
            float absmax = 0.0f;
            for (int i = 0; i < 32; i++) {
                float a = fabsf(data[(blk * 32 + i) * cols + col]);
                if (a > absmax) absmax = a;
            }
            float scale = (absmax > 0.0f) ? absmax / 127.0f : 1.0f;
            uint16_t sb = orc_f32_to_f16_bits(scale);
            buf[base] = (uint8_t)(sb & 0xFF);
            buf[base + 1] = (uint8_t)(sb >> 8);
            float inv = (scale > 0.0f) ? 1.0f / scale : 0.0f;
            for (int i = 0; i < 32; i++) {
                float val = data[(blk * 32 + i) * cols + col];
                int8_t q = (int8_t)round_clamp(val * inv, -128.0f, 127.0f);
                buf[base + 4 + i] = (uint8_t)q;
            }
        }
    }
    return 0;
}

int orc_dequantize_q8(const uint8_t *buf, size_t rows, size_t cols, float *out)
{
    if (rows % 32 != 0) return 1;
    size_t bpc = rows / 32;
    for (size_t col = 0; col < cols; col++) {
        for (size_t blk = 0; blk < bpc; blk++) {
            size_t base = (col * bpc + blk) * 36;
            uint16_t sb = (uint16_t)(buf[base] | (buf[base + 1] << 8));
            float scale = orc_f16_bits_to_f32_ieee(sb);
            for (int i = 0; i < 32; i++) {
                int8_t q = (int8_t)buf[base + 4 + i];
                out[(blk * 32 + i) * cols + col] = (float)q * scale;
            }
        }
    }
    return 0;
}

/* ---- the shader's per-element dequant (u32 view of the buffer) ------------ */

float orc_dequant_q4_shader(const uint32_t *b, uint32_t k_idx, uint32_t n_idx, uint32_t k, uint32_t n)
{
    uint32_t bpc = k / 32u, num_blocks = bpc * n;
    uint32_t block = n_idx * bpc + k_idx / 32u;
    uint32_t in_block = k_idx % 32u;
    uint32_t dm = b[block];
    float d = orc_f16_bits_to_f32_shader((uint16_t)(dm & 0xFFFFu));
    float m = orc_f16_bits_to_f32_shader((uint16_t)(dm >> 16));
    uint32_t byte_in_block = in_block / 2u;
    uint32_t data = b[num_blocks + block * 4u + byte_in_block / 4u];
    uint32_t shift = (byte_in_block % 4u) * 8u + ((in_block & 1u) ? 4u : 0u);
    uint32_t nib = (data >> shift) & 0xFu;
    return (float)nib * d + m;
}

float orc_dequant_q8_shader(const uint32_t *b, uint32_t k_idx, uint32_t n_idx, uint32_t k, uint32_t n)
{
    (void)n;
    uint32_t bpc = k / 32u;
    uint32_t block = n_idx * bpc + k_idx / 32u;
    uint32_t in_block = k_idx % 32u;
    uint32_t base = block * 9u;
    float scale = orc_f16_bits_to_f32_shader((uint16_t)(b[base] & 0xFFFFu));
    uint32_t data = b[base + 1u + in_block / 4u];
    uint32_t raw = (data >> ((in_block % 4u) * 8u)) & 0xFFu;
    int32_t s = (int32_t)raw - (raw >= 128u ? 256 : 0);
    return (float)s * scale;
}

/* ---- direct packers: codes + f16 bit patterns -> reference layout --------- */

/* codes[k*n] row-major, nibble values 0..15; d_bits/m_bits[n*bpc] indexed by block. */
int orc_pack_q4(const uint8_t *codes, const uint16_t *d_bits, const uint16_t *m_bits,
                size_t k, size_t n, uint8_t *buf)
{
    if (k % 32 != 0) return 1;
    size_t bpc = k / 32, num_blocks = bpc * n;
    memset(buf, 0, num_blocks * 20);
    for (size_t col = 0; col < n; col++)
        for (size_t blk = 0; blk < bpc; blk++) {
            size_t block = col * bpc + blk;
            uint32_t dm = (uint32_t)d_bits[block] | ((uint32_t)m_bits[block] << 16);
            memcpy(buf + block * 4, &dm, 4);
            uint8_t *nb = buf + num_blocks * 4 + block * 16;
            for (int i = 0; i < 32; i++) {
                uint8_t c = codes[(blk * 32 + i) * n + col] & 0xF;
                nb[i / 2] |= (i & 1) ? (uint8_t)(c << 4) : c;
            }
        }
    return 0;
}

int orc_pack_q8(const int8_t *codes, const uint16_t *scale_bits, size_t k, size_t n, uint8_t *buf)
{
    if (k % 32 != 0) return 1;
    size_t bpc = k / 32, num_blocks = bpc * n;
    memset(buf, 0, num_blocks * 36);
    for (size_t col = 0; col < n; col++)
        for (size_t blk = 0; blk < bpc; blk++) {
            size_t block = col * bpc + blk;
            uint8_t *p = buf + block * 36;
            p[0] = (uint8_t)(scale_bits[block] & 0xFF);
            p[1] = (uint8_t)(scale_bits[block] >> 8);
            for (int i = 0; i < 32; i++) p[4 + i] = (uint8_t)codes[(blk * 32 + i) * n + col];
        }
    return 0;
}

/* ---- dequantize one column into a contiguous f32 vector ------------------- */

/* variant 0: CPU functions (IEEE f16 decode, src/runtime.rs:2105-2215)
 * variant 1: shader functions (src/codegen.rs:738-806) */
static void column_f32(int fmt, const uint8_t *buf, size_t k, size_t n, size_t col, int variant, float *w)
{
    size_t bpc = k / 32, num_blocks = bpc * n;
    if (variant == 1) {
        const uint32_t *b32 = (const uint32_t *)buf;
        for (size_t kk = 0; kk < k; kk++)
            w[kk] = (fmt == ORC_FMT_Q4)
                ? orc_dequant_q4_shader(b32, (uint32_t)kk, (uint32_t)col, (uint32_t)k, (uint32_t)n)
                : orc_dequant_q8_shader(b32, (uint32_t)kk, (uint32_t)col, (uint32_t)k, (uint32_t)n);
        return;
    }
    for (size_t blk = 0; blk < bpc; blk++) {
        size_t block = col * bpc + blk;
        if (fmt == ORC_FMT_Q4) {
            uint32_t dm; memcpy(&dm, buf + block * 4, 4);
            float d = orc_f16_bits_to_f32_ieee((uint16_t)(dm & 0xFFFFu));
            float m = orc_f16_bits_to_f32_ieee((uint16_t)(dm >> 16));
            const uint8_t *nb = buf + num_blocks * 4 + block * 16;
            for (int i = 0; i < 32; i++) {
                uint32_t nib = (i & 1) ? (nb[i / 2] >> 4) : (nb[i / 2] & 0xF);
                w[blk * 32 + i] = (float)nib * d + m;
            }
        } else {
            const uint8_t *p = buf + block * 36;
            float scale = orc_f16_bits_to_f32_ieee((uint16_t)(p[0] | (p[1] << 8)));
            for (int i = 0; i < 32; i++) w[blk * 32 + i] = (float)(int8_t)p[4 + i] * scale;
        }
    }
}

/* ---- matmul: C[m,n] = A[m,k] . dequant(W)[k,n] (+ addend[m,n]) ------------ */

typedef struct {
    int fmt, variant, wide, failed;
    const float *a; const uint8_t *w; const float *addend;
    float *c32; double *c64;
    size_t m, k, n, c0, c1;
} mm_job;

static void *mm_worker(void *arg)
{
    mm_job *j = (mm_job *)arg;
    float *col = (float *)malloc(j->k * sizeof(float));
    if (!col) { j->failed = 1; return NULL; }
    for (size_t cc = j->c0; cc < j->c1; cc++) {
        column_f32(j->fmt, j->w, j->k, j->n, cc, j->variant, col);
        for (size_t r = 0; r < j->m; r++) {
            const float *ar = j->a + r * j->k;
            if (j->wide) {
                double s = 0.0;
                for (size_t kk = 0; kk < j->k; kk++) s += (double)ar[kk] * (double)col[kk];
                if (j->addend) s += (double)j->addend[r * j->n + cc];
                j->c64[r * j->n + cc] = s;
            } else {
                float s = 0.0f;
                for (size_t kk = 0; kk < j->k; kk++) s += ar[kk] * col[kk];
                if (j->addend) s += j->addend[r * j->n + cc];
                j->c32[r * j->n + cc] = s;
            }
        }
    }
    free(col);
    return NULL;
}

/* Columns are split into contiguous ranges, one per thread. */
static int mm_run(int fmt, const float *a, const uint8_t *w, const float *addend, float *c32, double *c64,
                  size_t m, size_t k, size_t n, int variant, int nthreads)
{
    if (k % 32 != 0 || (fmt != ORC_FMT_Q4 && fmt != ORC_FMT_Q8)) return 1;
    if (nthreads < 1) nthreads = 1;
    if ((size_t)nthreads > n) nthreads = n ? (int)n : 1;
    mm_job *jobs = (mm_job *)calloc((size_t)nthreads, sizeof(mm_job));
    pthread_t *tids = (pthread_t *)calloc((size_t)nthreads, sizeof(pthread_t));
    if (!jobs || !tids) { free(jobs); free(tids); return 2; }
    int failed = 0;
    for (int t = 0; t < nthreads; t++) {
        mm_job *j = &jobs[t];
        j->fmt = fmt; j->variant = variant; j->wide = (c64 != NULL);
        j->a = a; j->w = w; j->addend = addend; j->c32 = c32; j->c64 = c64;
        j->m = m; j->k = k; j->n = n;
        j->c0 = n * (size_t)t / (size_t)nthreads;
        j->c1 = n * (size_t)(t + 1) / (size_t)nthreads;
        if (t > 0 && pthread_create(&tids[t], NULL, mm_worker, j) != 0) { mm_worker(j); tids[t] = 0; }
    }
    mm_worker(&jobs[0]);
    for (int t = 1; t < nthreads; t++) if (tids[t]) pthread_join(tids[t], NULL);
    for (int t = 0; t < nthreads; t++) failed |= jobs[t].failed;
    free(jobs); free(tids);
    return failed ? 2 : 0;
}

/* f32, k ascending, separate multiply and add per term like the tiled shader
 * (WGSL `s += a*b` may or may not contract to an FMA on a given driver; either
 * rounding is far inside the comparison tolerance). */
int orc_matmul_f32(int fmt, const float *a, const uint8_t *w, const float *addend, float *c,
                   size_t m, size_t k, size_t n, int variant, int nthreads)
{
    return mm_run(fmt, a, w, addend, c, NULL, m, k, n, variant, nthreads);
}

/* f64 accumulation of the same f32 dequantized values: the comparison truth. */
int orc_matmul_f64(int fmt, const float *a, const uint8_t *w, const float *addend, double *c,
                   size_t m, size_t k, size_t n, int variant, int nthreads)
{
    return mm_run(fmt, a, w, addend, NULL, c, m, k, n, variant, nthreads);
}

/* ---- column sharding (no reference counterpart: new for multi-GPU) -------- */

/* Columns [n0, n1) of a packed [k, n] weight as a self-contained packed [k, n1-n0]. */
int orc_shard_columns(int fmt, const uint8_t *w, size_t k, size_t n, size_t n0, size_t n1, uint8_t *out)
{
    if (k % 32 != 0 || n0 > n1 || n1 > n) return 1;
    size_t bpc = k / 32, nb = bpc * n, sb = bpc * (n1 - n0);
    if (fmt == ORC_FMT_Q8) {
        memcpy(out, w + n0 * bpc * 36, sb * 36);
    } else if (fmt == ORC_FMT_Q4) {
        memcpy(out, w + n0 * bpc * 4, sb * 4);
        memcpy(out + sb * 4, w + nb * 4 + n0 * bpc * 16, sb * 16);
    } else return 1;
    return 0;
}
