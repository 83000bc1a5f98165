// Host-side pieces of libmgq: status/error plumbing, buffer sizing, the quantizers that
// Session::set_parameter runs on upload, and column sharding of packed weights.
//
// Counterparts in meganeura: TensorType::size_bytes (src/graph.rs:52-68), quantize_q4_0 /
// dequantize_q4_0 / quantize_q8_0 / dequantize_q8_0 (src/runtime.rs:2035-2215).  The
// f16 conversions follow the `half` crate (IEEE binary16, round to nearest even).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include <unordered_map>
#include <unordered_set>
#include <algorithm>
#include "mgq_internal.h"

namespace mgq {

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

// ---- binary16 conversions ------------------------------------------------------------

static inline uint32_t bits_of(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
static inline float float_of(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

static uint16_t f16_from_f32(float f)
{
    const uint32_t x = bits_of(f);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t ex = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (ex == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0u));
    const int e = (int)ex - 112;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const uint32_t sh = (uint32_t)(14 - e);
        uint32_t hm = man >> sh;
        const uint32_t rem = man & ((1u << sh) - 1u), mid = 1u << (sh - 1);
        if (rem > mid || (rem == mid && (hm & 1u))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t h = ((uint32_t)e << 10) | (man >> 13);
    const uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

static float f16_to_f32(uint16_t h)
{
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t ex = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    if (ex == 0) {
        const float v = (float)man * 5.9604644775390625e-8f;   // man * 2^-24
        return sign ? -v : v;
    }
    if (ex == 31) return float_of(sign | 0x7F800000u | (man << 13));
    return float_of(sign | ((ex + 112u) << 23) | (man << 13));
}

// Rust's f32::round (halves away from zero) followed by clamp.
static inline float round_clamp(float v, float lo, float hi)
{
    float r = std::round(v);
    return r < lo ? lo : (r > hi ? hi : r);
}

// Columns are independent, so the one-time O(K*N) quantizer is split over host threads.
template <class F>
static void for_columns(size_t n, F body)
{
    unsigned hw = std::thread::hardware_concurrency();
    size_t nt = hw ? hw : 1;
    if (nt > n / 64 + 1) nt = n / 64 + 1;
    if (nt <= 1) { body(0, n); return; }
    std::vector<std::thread> pool;
    for (size_t t = 0; t < nt; t++)
        pool.emplace_back([=] { body(n * t / nt, n * (t + 1) / nt); });
    for (auto &th : pool) th.join();
}

}  // namespace mgq

using namespace mgq;

extern "C" {

const char *mgq_last_error(void) { return mgq::g_err; }
const char *mgq_version(void) { return "mgq 0.1 (sm_100a)"; }

size_t mgq_packed_bytes(int fmt, size_t k, size_t n)
{
    const size_t blocks = (k * n + 31) / 32;
    if (fmt == MGQ_FMT_Q4) return blocks * 20;
    if (fmt == MGQ_FMT_Q8) return blocks * 36;
    return 0;
}

static int check_qargs(const void *a, const void *b, size_t k, size_t n)
{
    if (!a || !b) return fail(MGQ_ERR_NULL, "null pointer");
    if (k == 0 || n == 0) return fail(MGQ_ERR_SHAPE, "empty matrix %zux%zu", k, n);
    if (k % 32 != 0) return fail(MGQ_ERR_SHAPE, "rows (K dim) must be a multiple of 32, got %zu", k);
    return MGQ_OK;
}

int mgq_quantize_q4(const float *w, size_t k, size_t n, uint8_t *out)
{
    if (int rc = check_qargs(w, out, k, n)) return rc;
    const size_t bpc = k / 32, nb = bpc * n;
    for_columns(n, [=](size_t c0, size_t c1) {
        for (size_t col = c0; col < c1; col++)
            for (size_t blk = 0; blk < bpc; blk++) {
                const size_t bi = col * bpc + blk;
                float v[32], lo = INFINITY, hi = -INFINITY;
                for (int i = 0; i < 32; i++) {
                    v[i] = w[(blk * 32 + i) * n + col];
                    if (v[i] < lo) lo = v[i];
                    if (v[i] > hi) hi = v[i];
                }
                const float d = hi > lo ? (hi - lo) / 15.0f : 1.0f;
                const uint32_t hdr = (uint32_t)f16_from_f32(d) | ((uint32_t)f16_from_f32(lo) << 16);
                std::memcpy(out + bi * 4, &hdr, 4);
                const float inv = d > 0.0f ? 1.0f / d : 0.0f;   // codes use the unrounded f32 step
                uint8_t *dst = out + nb * 4 + bi * 16;
                for (int j = 0; j < 16; j++) {
                    const uint8_t a = (uint8_t)round_clamp((v[2 * j] - lo) * inv, 0.0f, 15.0f);
                    const uint8_t b = (uint8_t)round_clamp((v[2 * j + 1] - lo) * inv, 0.0f, 15.0f);
                    dst[j] = (uint8_t)(a | (b << 4));
                }
            }
    });
    return MGQ_OK;
}

int mgq_dequantize_q4(const uint8_t *packed, size_t k, size_t n, float *out)
{
    if (int rc = check_qargs(packed, out, k, n)) return rc;
    const size_t bpc = k / 32, nb = bpc * n;
    for_columns(n, [=](size_t c0, size_t c1) {
        for (size_t col = c0; col < c1; col++)
            for (size_t blk = 0; blk < bpc; blk++) {
                const size_t bi = col * bpc + blk;
                uint32_t hdr;
                std::memcpy(&hdr, packed + bi * 4, 4);
                const float d = f16_to_f32((uint16_t)(hdr & 0xFFFF)), mn = f16_to_f32((uint16_t)(hdr >> 16));
                const uint8_t *src = packed + nb * 4 + bi * 16;
                for (int i = 0; i < 32; i++) {
                    const unsigned q = (i & 1) ? (src[i >> 1] >> 4) : (src[i >> 1] & 0xF);
                    out[(blk * 32 + i) * n + col] = (float)q * d + mn;
                }
            }
    });
    return MGQ_OK;
}

int mgq_quantize_q8(const float *w, size_t k, size_t n, uint8_t *out)
{
    if (int rc = check_qargs(w, out, k, n)) return rc;
    const size_t bpc = k / 32;
    for_columns(n, [=](size_t c0, size_t c1) {
        for (size_t col = c0; col < c1; col++)
            for (size_t blk = 0; blk < bpc; blk++) {
                uint8_t *dst = out + (col * bpc + blk) * 36;
                float v[32], amax = 0.0f;
                for (int i = 0; i < 32; i++) {
                    v[i] = w[(blk * 32 + i) * n + col];
                    const float a = std::fabs(v[i]);
                    if (a > amax) amax = a;
                }
                const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
                const uint16_t sb = f16_from_f32(scale);
                dst[0] = (uint8_t)(sb & 0xFF);
                dst[1] = (uint8_t)(sb >> 8);
                dst[2] = dst[3] = 0;
                const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
                for (int i = 0; i < 32; i++) dst[4 + i] = (uint8_t)(int8_t)round_clamp(v[i] * inv, -128.0f, 127.0f);
            }
    });
    return MGQ_OK;
}

int mgq_dequantize_q8(const uint8_t *packed, size_t k, size_t n, float *out)
{
    if (int rc = check_qargs(packed, out, k, n)) return rc;
    const size_t bpc = k / 32;
    for_columns(n, [=](size_t c0, size_t c1) {
        for (size_t col = c0; col < c1; col++)
            for (size_t blk = 0; blk < bpc; blk++) {
                const uint8_t *src = packed + (col * bpc + blk) * 36;
                const float scale = f16_to_f32((uint16_t)(src[0] | (src[1] << 8)));
                for (int i = 0; i < 32; i++) out[(blk * 32 + i) * n + col] = (float)(int8_t)src[4 + i] * scale;
            }
    });
    return MGQ_OK;
}

int mgq_shard_columns(int fmt, const uint8_t *packed, size_t k, size_t n, size_t n0, size_t n1, uint8_t *out)
{
    if (int rc = check_qargs(packed, out, k, n)) return rc;
    if (!is_quant(fmt)) return fail(MGQ_ERR_FORMAT, "shard_columns: format %d is not Q4/Q8", fmt);
    if (n0 >= n1 || n1 > n) return fail(MGQ_ERR_SHAPE, "column range [%zu,%zu) outside [0,%zu)", n0, n1, n);
    const size_t bpc = k / 32, nb = bpc * n, sb = bpc * (n1 - n0);
    if (fmt == MGQ_FMT_Q8) {
        std::memcpy(out, packed + n0 * bpc * 36, sb * 36);
    } else {
        std::memcpy(out, packed + n0 * bpc * 4, sb * 4);                     // headers of the range
        std::memcpy(out + sb * 4, packed + nb * 4 + n0 * bpc * 16, sb * 16); // then its nibbles
    }
    return MGQ_OK;
}

}  // extern "C"

// f32 -> binary16 with the `half` crate's rounding (IEEE round to nearest even), what the reference
// stores for parameter_f16 weights (src/runtime.rs:2335).
extern "C" int mgq_convert_f16(const float *src, size_t len, uint16_t *dst)
{
    if (!src || !dst) return mgq::fail(MGQ_ERR_NULL, "null pointer");
    for (size_t i = 0; i < len; i++) dst[i] = f16_from_f32(src[i]);
    return MGQ_OK;
}

// Barrier groups of a dispatch list, the reference's reorder_by_level + compute_groups
// (src/runtime.rs:1202-1256).  inputs / outputs hold up to four buffer ids per dispatch (-1: none).
// Level of a dispatch = 0 when no earlier dispatch produced any of its inputs, else 1 + the highest
// level among those producers; a stable sort by level gives the reference's order; a new group starts
// whenever a dispatch reads a buffer written earlier in the current group.
extern "C" int mgq_barrier_groups(const int32_t *inputs, const int32_t *outputs, size_t n, int reorder)
{
    if (n == 0) return 0;
    if (!inputs || !outputs) return -mgq::fail(MGQ_ERR_NULL, "null dispatch list");
    std::vector<size_t> order(n);
    for (size_t i = 0; i < n; i++) order[i] = i;
    if (reorder) {
        std::vector<uint32_t> level(n, 0);
        std::unordered_map<int32_t, size_t> producer;
        for (size_t i = 0; i < n; i++) {
            uint32_t lv = 0;
            for (int j = 0; j < 4; j++) {
                const int32_t b = inputs[i * 4 + j];
                if (b < 0) continue;
                auto it = producer.find(b);
                if (it != producer.end()) lv = std::max(lv, level[it->second] + 1);
            }
            level[i] = lv;
            for (int j = 0; j < 4; j++)
                if (outputs[i * 4 + j] >= 0) producer[outputs[i * 4 + j]] = i;
        }
        std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return level[a] < level[b]; });
    }
    int groups = 0;
    std::unordered_set<int32_t> dirty;
    for (size_t pos = 0; pos < n; pos++) {
        const size_t i = order[pos];
        bool hazard = false;
        for (int j = 0; j < 4; j++)
            if (inputs[i * 4 + j] >= 0 && dirty.count(inputs[i * 4 + j])) hazard = true;
        if (hazard) {
            groups++;
            dirty.clear();
        }
        for (int j = 0; j < 4; j++)
            if (outputs[i * 4 + j] >= 0) dirty.insert(outputs[i * 4 + j]);
    }
    return groups + 1;
}
