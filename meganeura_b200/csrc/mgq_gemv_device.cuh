// Device-side building blocks shared by the GEMV kernels (mgq_gemv.cu) and the persistent plan
// kernel (mgq_plan.cu): cp.async helpers, the block-fixed-point activation format, the dp4a block
// dot products and the per-round column reduction.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace mgq {
namespace dev {

constexpr uint32_t kQ8WarpStage = 1152;       // 32 blocks * 36 B per warp and stage

struct GemvParams {
    const float *x;
    const uint8_t *w;
    const float *addend;
    float *y;
    uint32_t k, n, bpc;
    uint32_t cpi;          // columns per iteration
    uint32_t active;       // cpi * bpc threads carry a block (a multiple of 4)
    uint32_t total_iters;  // ceil(n / cpi)
    uint32_t red_shift;    // log2(lanes that finish one column sum)
    uint32_t red_chunk;    // partials summed by each finishing lane = ceil(bpc / lanes)
    unsigned long long num_blocks;
    // multi-GPU exchange (all null / zero on a single GPU)
    const struct ExchangePush *push;          // where the leading columns of y also go: every peer's gathered vector
    const float2 *wait_vec;                   // local gathered {value, stamp} vector (length k) that must carry this token's stamps
    const unsigned long long *epoch;          // local token index
    unsigned int *xerror;                     // raised when the bounded wait runs out
    unsigned long long wait_ns;               // time limit of the stamp poll
};

// Fused all-gather of a column-sharded GEMV.  Instead of a collective after the kernel, the lane
// that finishes a column stores it straight into every rank's copy of the gathered vector (plain
// peer stores over NVLink; remote data always lands in the consumer GPU's own memory).  Each
// element travels as one 8-byte {value, stamp} pair written by a single 64-bit store, stamp = token
// index + 1, so the data carries its own validity: a consumer polls the stamps of exactly the 32
// elements it is about to use (with an iteration limit) and needs no fence, counter or atomic.
constexpr int kMaxPeers = 8;
struct ExchangePush {                          // one per exchanging GEMV, in device memory (mgq_exchange_push)
    uint32_t world, rank;
    uint32_t gather_cols;                      // leading columns of this rank's y that every rank needs
    uint32_t reserved;
    float2 *dst[kMaxPeers];                    // rank p's gathered {value, stamp} vector; this rank fills [rank*gather_cols, +gather_cols)
};

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t exchange_stamp(const unsigned long long *epoch)
{
    unsigned long long token;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(token) : "l"(epoch) : "memory");
    return (uint32_t)token + 1u;
}

// Before block b of x is used: wait until all 32 of its elements carry this token's stamp.  Peer
// stores land in this GPU's L2, so the poll uses L1-bypassing GPU-scope loads (system-scope loads
// of this volume -- every thread of every CTA reads its 256 bytes -- were measured 8x slower); a
// stale read only costs another iteration because every element carries its own stamp.
__device__ __forceinline__ void exchange_poll(const GemvParams &p, uint32_t b)
{
    if (!p.wait_vec) return;
    const uint32_t stamp = exchange_stamp(p.epoch);
    const uint32_t lane = threadIdx.x & 31u;
    // When a warp's 32 blocks are consecutive (K a multiple of 1024) the warp polls its 8 KB region
    // together, lane l reading consecutive 16-byte pieces: fully coalesced, no sector read twice.
    const bool together = (p.bpc & 31u) == 0;
    const uint4 *src = together ? reinterpret_cast<const uint4 *>(p.wait_vec + 32u * (b - lane)) + lane
                                : reinterpret_cast<const uint4 *>(p.wait_vec + 32u * b);
    const uint32_t step = together ? 32u : 1u;
    unsigned long long t0 = 0;
    for (uint32_t spins = 0;; spins++) {
        uint32_t ok = 1;
#pragma unroll
        for (uint32_t j = 0; j < 16; j++) {
            uint4 v;
            asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + j * step) : "memory");
            ok &= (v.y == stamp) & (v.w == stamp);
        }
        if (together) ok = __all_sync(0xffffffffu, ok);
        if (ok) break;
        if ((spins & 31u) == 31u) {
            // once any thread of the step has given up, the step is lost: later waiters leave at once
            if (*reinterpret_cast<const volatile uint32_t *>(p.xerror) != 0u) break;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > p.wait_ns) { atomicExch(p.xerror, 1u); break; }
        }
    }
}

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem)
{
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void *smem, const void *gmem)
{
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Programmatic dependent launch: a GEMV launched with the stream-serialization attribute may
// start while the previous kernel of the stream is still draining.  Everything before
// grid_dependency_wait() must not touch memory that an earlier kernel writes: only the packed
// weights (immutable after upload) are fetched there.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// dp4a with mixed signedness (a: packed codes, b: packed activation bytes).
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// The 32 activations of one block as three byte planes, packed four to a word in the order
// the codes come out of the packed weight words.
struct XBlock {
    uint32_t p0[8], p1[8], p2[8];   // plane 0, 1: unsigned bytes; plane 2: signed bytes
    float inv;                      // 2^(E-21): turns the integer dot product back into x units
    float sum;                      // plain f32 sum of the 32 activations (for Q4's "+ m")
};

// ORDER 0 (Q8): word j holds elements 4j .. 4j+3.
// ORDER 1 (Q4): word 2j holds elements 8j+{0,2,4,6} (low nibbles of nibble word j),
//               word 2j+1 holds elements 8j+{1,3,5,7} (high nibbles).
// Turns 32 activations (already in registers) into the three byte planes, scale and sum.
// SIGNED_DIGITS: all three planes are signed bytes, X = p2*65536 + p1*256 + p0 with every digit in
// [-128, 127] (what an int8 tensor-core operand wants); otherwise planes 0 and 1 are unsigned.
template <int ORDER, bool SIGNED_DIGITS = false>
__device__ __forceinline__ void prepare_x(const float (&v)[32], XBlock &xb)
{
    float amax = 0.f, s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        amax = fmaxf(amax, fmaxf(fabsf(v[i]), fabsf(v[i + 1])));
        s0 += v[i];
        s1 += v[i + 1];
    }
    xb.sum = s0 + s1;
    // biased exponent of the largest magnitude, clamped so that both 2^(21-E) and 2^(E-21) are normal
    uint32_t eb = (__float_as_uint(amax) >> 23) & 0xFFu;
    const bool finite = eb != 0xFFu;
    eb = min(max(eb, 24u), 254u);
    const float scale = __uint_as_float((275u - eb) << 23);           // 2^(21-E)
    xb.inv = finite ? __uint_as_float((eb - 21u) << 23) : __int_as_float(0x7FC00000);   // 2^(E-21), NaN for inf/NaN input
    // x*scale + 1.5*2^23 leaves X + 2^22 in the low 23 mantissa bits (|X| <= 2^22): bytes 0..2 of the
    // float's bit pattern are the planes, the top one offset by 64.
    uint32_t bits[32];
#pragma unroll
    // (signed digits: adding 128 to the two low bytes, with carries, makes byte - 128 the balanced digit)
    for (int i = 0; i < 32; i++) bits[i] = __float_as_uint(fmaf(v[i], scale, 12582912.f)) + (SIGNED_DIGITS ? 0x8080u : 0u);
#pragma unroll
    for (int w = 0; w < 8; w++) {
        int e0, e1, e2, e3;
        if (ORDER == 0) { e0 = 4 * w; e1 = e0 + 1; e2 = e0 + 2; e3 = e0 + 3; }
        else            { e0 = 8 * (w >> 1) + (w & 1); e1 = e0 + 2; e2 = e0 + 4; e3 = e0 + 6; }
        const uint32_t a = bits[e0], bb = bits[e1], c = bits[e2], d = bits[e3];
        xb.p0[w] = __byte_perm(__byte_perm(a, bb, 0x0040), __byte_perm(c, d, 0x0040), 0x5410) ^ (SIGNED_DIGITS ? 0x80808080u : 0u);
        xb.p1[w] = __byte_perm(__byte_perm(a, bb, 0x0051), __byte_perm(c, d, 0x0051), 0x5410) ^ (SIGNED_DIGITS ? 0x80808080u : 0u);
        const uint32_t top = __byte_perm(__byte_perm(a, bb, 0x0062), __byte_perm(c, d, 0x0062), 0x5410);
        xb.p2[w] = (top + 0x40404040u) ^ 0x80808080u;                  // (u + 64) - 128 = u - 64 as int8; u <= 127: no carries
    }
}

// COHERENT: read through L2 (the producer may be another CTA of the same persistent kernel).
template <int ORDER, bool COHERENT = false>
__device__ __forceinline__ void load_x(const float *xrow, uint32_t b, XBlock &xb)
{
    const float4 *xp = reinterpret_cast<const float4 *>(xrow + 32u * b);
    float v[32];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float4 t = COHERENT ? __ldcg(xp + j) : __ldg(xp + j);
        v[4 * j + 0] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
    prepare_x<ORDER>(v, xb);
}

// Block b of x taken from a gathered {value, stamp} vector whose stamps have already been checked.
template <int ORDER>
__device__ __forceinline__ void load_x_gathered(const float2 *vec, uint32_t b, XBlock &xb)
{
    const uint4 *src = reinterpret_cast<const uint4 *>(vec + 32u * b);
    float v[32];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        uint4 t;
        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(t.x), "=r"(t.y), "=r"(t.z), "=r"(t.w) : "l"(src + j) : "memory");
        v[2 * j] = __uint_as_float(t.x);
        v[2 * j + 1] = __uint_as_float(t.z);
    }
    prepare_x<ORDER>(v, xb);
}

// Exact sum over one block of X[i] * code[i], returned in f32.  The three plane sums are recombined in
// integer arithmetic: |sum| <= 15 * 32 * (64 * 65536 + 255 * 256 + 255) < 2^31, so the exact value
// fits and a single conversion rounds it (one I2F instead of three, no FMAs).
__device__ __forceinline__ float dot_q4(const uint4 &q, const XBlock &xb)
{
    const uint32_t wv[4] = {q.x, q.y, q.z, q.w};
    int a0 = 0, a1 = 0, a2 = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t lo = wv[j] & 0x0F0F0F0Fu, hi = (wv[j] >> 4) & 0x0F0F0F0Fu;
        a0 = dp4a_uu(lo, xb.p0[2 * j], a0);
        a1 = dp4a_uu(lo, xb.p1[2 * j], a1);
        a2 = dp4a_us(lo, xb.p2[2 * j], a2);
        a0 = dp4a_uu(hi, xb.p0[2 * j + 1], a0);
        a1 = dp4a_uu(hi, xb.p1[2 * j + 1], a1);
        a2 = dp4a_us(hi, xb.p2[2 * j + 1], a2);
    }
    return (float)(a2 * 65536 + a1 * 256 + a0);
}

// bp points at the 8 code words (int8 x 4) of a Q8 block.
__device__ __forceinline__ float dot_q8(const uint32_t *bp, const XBlock &xb)
{
    int a0 = 0, a1 = 0, a2 = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint32_t c = bp[j];
        a0 = dp4a_su(c, xb.p0[j], a0);
        a1 = dp4a_su(c, xb.p1[j], a1);
        a2 = dp4a_ss(c, xb.p2[j], a2);
    }
    return fmaf((float)a2, 65536.f, fmaf((float)a1, 256.f, (float)a0));
}

// Which column sum a thread finishes after each round; the same for every round, so it is
// worked out once.  A round holds ROUND*cpi columns; each is finished by 2^red_shift
// neighbouring lanes that first add up a contiguous run of red_chunk partials each.
struct ReduceSlot {
    uint32_t src;        // float offset of this lane's run inside one row of the staging array
    uint32_t cnt;        // partials in the run (0: lane idle)
    uint32_t iter;       // iteration inside the round the column belongs to
    uint32_t cs;         // column inside that iteration
    bool writer;         // lane that stores the finished sum
    bool vec;            // run is float4-readable
};

// STRIDE: floats between consecutive rows of the staging array (0: one row per thread of the CTA).
template <int ROUND, int STRIDE = 0>
__device__ __forceinline__ ReduceSlot make_slot(const GemvParams &p)
{
    const uint32_t T = STRIDE ? (uint32_t)STRIDE : blockDim.x, t = threadIdx.x;
    const uint32_t R = 1u << p.red_shift;
    const uint32_t slot = t >> p.red_shift, li = t & (R - 1);
    ReduceSlot s{};
    if (slot < ROUND * p.cpi) {
        s.iter = slot / p.cpi;
        s.cs = slot % p.cpi;
        const uint32_t first = li * p.red_chunk;
        s.cnt = first < p.bpc ? min(p.red_chunk, p.bpc - first) : 0u;
        s.src = s.iter * T + s.cs * p.bpc + first;
        s.writer = li == 0;
        s.vec = (p.bpc % 4 == 0) && (p.red_chunk % 4 == 0);
    }
    return s;
}

template <int MT, int ROUND, bool COHERENT = false, int STRIDE = 0>
__device__ __forceinline__ void reduce_store(const GemvParams &p, const ReduceSlot &slot, float *red,
                                             const float (&part)[MT][ROUND], uint32_t it_base, uint32_t it_end,
                                             float *push_stage = nullptr)
{
    const uint32_t T = STRIDE ? (uint32_t)STRIDE : blockDim.x, t = threadIdx.x;
#pragma unroll
    for (int r = 0; r < MT; r++)
#pragma unroll
        for (int u = 0; u < ROUND; u++) red[(r * ROUND + u) * T + t] = part[r][u];
    __syncthreads();
#pragma unroll
    for (int r = 0; r < MT; r++) {
        const float *src = red + r * ROUND * T + slot.src;
        float s = 0.f;
        if (slot.vec) {
            for (uint32_t j = 0; j < slot.cnt; j += 4) {
                const float4 v = *reinterpret_cast<const float4 *>(src + j);
                s += (v.x + v.y) + (v.z + v.w);
            }
        } else {
            for (uint32_t j = 0; j < slot.cnt; j++) s += src[j];
        }
        if (p.red_shift > 4) s += __shfl_xor_sync(0xffffffffu, s, 16);
        if (p.red_shift > 3) s += __shfl_xor_sync(0xffffffffu, s, 8);
        if (p.red_shift > 2) s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (p.red_shift > 1) s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (p.red_shift > 0) s += __shfl_xor_sync(0xffffffffu, s, 1);
        const uint32_t it = it_base + slot.iter;
        const uint32_t col = it * p.cpi + slot.cs;
        if (slot.writer && it < it_end && col < p.n) {
            const size_t o = (size_t)r * p.n + col;
            const float add = p.addend ? (COHERENT ? __ldcg(p.addend + o) : p.addend[o]) : 0.f;
            const float v = p.addend ? s + add : s;
            p.y[o] = v;
            if (push_stage && r == 0) push_stage[slot.iter * p.cpi + slot.cs] = v;     // column offset inside the round
        }
    }
    if (push_stage) {
        // The round's columns are consecutive: consecutive lanes send consecutive {value, stamp} pairs, so
        // a peer receives a few full 128-byte writes instead of one 8-byte write per column.
        __syncthreads();
        const ExchangePush &px = *p.push;
        const uint32_t first = it_base * p.cpi;
        uint32_t ncols = min((uint32_t)ROUND, it_end - it_base) * p.cpi;
        ncols = min(ncols, p.n - first);
        if (first < px.gather_cols) {
            ncols = min(ncols, px.gather_cols - first);
            const uint32_t stamp = exchange_stamp(p.epoch);
            for (uint32_t idx = t; idx < ncols * px.world; idx += blockDim.x) {
                const uint32_t q = idx / ncols, c = idx - q * ncols;
                px.dst[q][(size_t)px.rank * px.gather_cols + first + c] = make_float2(push_stage[c], __uint_as_float(stamp));
            }
        }
    }
}

}  // namespace dev
}  // namespace mgq
