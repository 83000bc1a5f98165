// Dequantize-fused GEMV for Q4/Q8 weights on sm_100a:  y[m,n] = x[m,k] . dequant(W)[k,n] (+ addend).
//
// Stands in for meganeura's MatMulGemv / MatMulGemvAdd dispatches (src/compile.rs:1390-1406,
// 1498-1509) with the weight semantics of dequant_q4 / dequant_q8 (src/codegen.rs:748-805).
//
// The kernel is HBM-bound and uses no tensor cores.  Design:
//
//  * In the reference layout all 32-element blocks of one output column are contiguous
//    (block = n*(K/32) + k/32), so consecutive threads take consecutive blocks of the packed
//    stream: thread t of a CTA owns block-in-column b = t % bpc of column (t / bpc) of the
//    current group of `cpi` columns, and every iteration advances by cpi columns.  The CTA
//    therefore sweeps the weight bytes linearly and every byte is read exactly once.
//  * b is fixed per thread, so the 32 activations a thread needs stay in registers for the
//    whole kernel (no shared-memory traffic for x in the inner loop).
//  * Weights are brought in with cp.async into a multi-stage shared-memory ring, so many KB
//    per SM are in flight without holding registers.  Q4: each thread copies its own 16
//    nibble bytes + 4 header bytes (no barrier needed).  Q8: a 36-byte block is only 4-byte
//    aligned, so each warp copies its 32 blocks (1152 contiguous bytes) as 16-byte pieces
//    and lanes then read their block at a 36-byte stride (9 is odd: conflict-free).
//  * The 32 products of a block are integer dot products (dp4a, full rate on sm_100 while
//    logic ops and int->float conversions are not).  The block's activations are held as
//    block-fixed-point: X[i] = round(x[i] * 2^(21-E)), 2^E <= max|x| < 2^(E+1), |X| <= 2^22,
//    split into three byte planes (two unsigned, the top one signed).  Q8 codes are already
//    int8x4 words; Q4 needs three logic ops per eight nibbles.  Within a block the sum is
//    exact integer arithmetic; the three plane sums are recombined in f32 and the per-block
//    scale is applied once per 32 products, accumulating over blocks in f32:
//        Q4:  d * sum(x*nib) + m * sum(x)          Q8:  s * sum(x*q)
//    The fixed-point step costs at most 2^-22 of the block's largest |x| per activation.
//  * Column sums are finished through shared memory + warp shuffles in a fixed order that
//    depends only on K, so a column's result does not depend on N or on its position in the
//    grid (column shards reproduce the unsharded result bit for bit).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>
#include <vector>

#include "mgq_internal.h"

namespace mgq {
namespace {

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
#ifdef MGQ_GEMV_TRACE
    unsigned long long *trace;   // [gridDim.x][4] globaltimer stamps: start, after dependency wait, first block done, end
#endif
};

#ifdef MGQ_GEMV_TRACE
__device__ __forceinline__ unsigned long long now_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define MGQ_STAMP(p, slot) do { if ((p).trace && threadIdx.x == 0) (p).trace[blockIdx.x * 4 + (slot)] = now_ns(); } while (0)
#else
#define MGQ_STAMP(p, slot) do { } while (0)
#endif

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
template <int ORDER>
__device__ __forceinline__ void load_x(const float *xrow, uint32_t b, XBlock &xb)
{
    const float4 *xp = reinterpret_cast<const float4 *>(xrow + 32u * b);
    float v[32];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float4 t = __ldg(xp + j);
        v[4 * j + 0] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
    }
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
    for (int i = 0; i < 32; i++) bits[i] = __float_as_uint(fmaf(v[i], scale, 12582912.f));
#pragma unroll
    for (int w = 0; w < 8; w++) {
        int e0, e1, e2, e3;
        if (ORDER == 0) { e0 = 4 * w; e1 = e0 + 1; e2 = e0 + 2; e3 = e0 + 3; }
        else            { e0 = 8 * (w >> 1) + (w & 1); e1 = e0 + 2; e2 = e0 + 4; e3 = e0 + 6; }
        const uint32_t a = bits[e0], bb = bits[e1], c = bits[e2], d = bits[e3];
        xb.p0[w] = __byte_perm(__byte_perm(a, bb, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
        xb.p1[w] = __byte_perm(__byte_perm(a, bb, 0x0051), __byte_perm(c, d, 0x0051), 0x5410);
        const uint32_t top = __byte_perm(__byte_perm(a, bb, 0x0062), __byte_perm(c, d, 0x0062), 0x5410);
        xb.p2[w] = (top + 0x40404040u) ^ 0x80808080u;                  // (u + 64) - 128 = u - 64 as int8; u <= 127: no carries
    }
}

// Exact sum over one block of X[i] * code[i], returned in f32 (planes recombined with two FMAs).
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
    return fmaf((float)a2, 65536.f, fmaf((float)a1, 256.f, (float)a0));
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

template <int ROUND>
__device__ __forceinline__ ReduceSlot make_slot(const GemvParams &p)
{
    const uint32_t T = blockDim.x, t = threadIdx.x;
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

template <int MT, int ROUND>
__device__ __forceinline__ void reduce_store(const GemvParams &p, const ReduceSlot &slot, float *red,
                                             const float (&part)[MT][ROUND], uint32_t it_base, uint32_t it_end)
{
    const uint32_t T = blockDim.x, t = threadIdx.x;
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
        for (uint32_t o = (1u << p.red_shift) >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const uint32_t it = it_base + slot.iter;
        const uint32_t col = it * p.cpi + slot.cs;
        if (slot.writer && it < it_end && col < p.n) {
            const size_t o = (size_t)r * p.n + col;
            p.y[o] = p.addend ? s + p.addend[o] : s;
        }
    }
}

// ------------------------------------------------------------------------------------ Q4

template <int MT, int STAGES, int TMAX>
__global__ void __launch_bounds__(TMAX) gemv_q4_kernel(const GemvParams p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t T = blockDim.x, t = threadIdx.x;
    uint4 *s_nib = reinterpret_cast<uint4 *>(smem) + t;                                   // [STAGES][T], own slot
    uint32_t *s_hdr = reinterpret_cast<uint32_t *>(smem + (size_t)STAGES * T * 16) + t;   // [STAGES][T], own slot
    float *s_red = reinterpret_cast<float *>(smem + (size_t)STAGES * T * 20);             // [2][MT][STAGES][T]
    MGQ_STAMP(p, 0);

    const uint32_t it0 = (uint32_t)((unsigned long long)blockIdx.x * p.total_iters / gridDim.x);
    const uint32_t it1 = (uint32_t)((unsigned long long)(blockIdx.x + 1) * p.total_iters / gridDim.x);
    const uint32_t n_it = it1 - it0;
    const bool has_block = t < p.active;
    const uint32_t b = t % p.bpc, csub = t / p.bpc;
    // iterations in which this thread has a column: all of them, except that the very last
    // iteration of the matrix may hold fewer than cpi columns
    uint32_t my_n = has_block ? n_it : 0u;
    if (has_block && it1 == p.total_iters && n_it > 0 && (p.total_iters - 1) * p.cpi + csub >= p.n) my_n = n_it - 1;

    const unsigned long long g0 = (unsigned long long)it0 * p.active + t;                // = col*bpc + b
    const uint32_t *hdr_next = reinterpret_cast<const uint32_t *>(p.w) + g0;
    const uint4 *nib_next = reinterpret_cast<const uint4 *>(p.w + p.num_blocks * 4) + g0;
    const uint32_t stride = p.active;

    auto issue = [&](int stage, bool ok) {
        if (ok) {
            cp_async16(s_nib + stage * T, nib_next);
            cp_async4(s_hdr + stage * T, hdr_next);
        }
        nib_next += stride;
        hdr_next += stride;
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) issue(s, (uint32_t)s < my_n);     // weights first: they depend on nothing
    grid_launch_dependents();
    grid_dependency_wait();                                                 // x, addend and y belong to earlier kernels
    MGQ_STAMP(p, 1);

    XBlock xb[MT];
#pragma unroll
    for (int r = 0; r < MT; r++) load_x<1>(p.x + (size_t)r * p.k, b, xb[r]);
    const ReduceSlot slot = make_slot<STAGES>(p);

    auto block_sum = [&](int stage, float (&out)[MT]) {
        const uint4 q = s_nib[stage * T];
        const uint32_t h = s_hdr[stage * T];
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&h));       // (d, m), IEEE
#pragma unroll
        for (int r = 0; r < MT; r++) out[r] = fmaf(dm.x * xb[r].inv, dot_q4(q, xb[r]), dm.y * xb[r].sum);
    };

    uint32_t round = 0;
    for (uint32_t i = 0; i < n_it; i += STAGES, round++) {
        float part[MT][STAGES];
        if (i + 2 * STAGES - 1 <= my_n) {                  // whole round and everything it prefetches is in range
#pragma unroll
            for (int u = 0; u < STAGES; u++) {
                issue((u + STAGES - 1) % STAGES, true);
                cp_async_wait<STAGES - 1>();
                float out[MT];
                block_sum(u, out);
#pragma unroll
                for (int r = 0; r < MT; r++) part[r][u] = out[r];
            }
        } else {
#pragma unroll
            for (int u = 0; u < STAGES; u++) {
                issue((u + STAGES - 1) % STAGES, i + u + STAGES - 1 < my_n);
                cp_async_wait<STAGES - 1>();
                float out[MT];
#pragma unroll
                for (int r = 0; r < MT; r++) out[r] = 0.f;
                if (i + u < my_n) block_sum(u, out);
#pragma unroll
                for (int r = 0; r < MT; r++) part[r][u] = out[r];
            }
        }
        if (round == 0) MGQ_STAMP(p, 2);
        reduce_store<MT, STAGES>(p, slot, s_red + (size_t)(round & 1) * MT * STAGES * T, part, it0 + i, it1);
    }
    cp_async_wait<0>();
    MGQ_STAMP(p, 3);
}

// ------------------------------------------------------------------------------------ Q8

template <int MT, int STAGES, int TMAX>
__global__ void __launch_bounds__(TMAX) gemv_q8_kernel(const GemvParams p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t T = blockDim.x, t = threadIdx.x, lane = t & 31u, warp = t >> 5, W = T >> 5;
    uint8_t *s_w = smem + (size_t)warp * STAGES * kQ8WarpStage;                         // this warp's ring
    float *s_red = reinterpret_cast<float *>(smem + (size_t)W * STAGES * kQ8WarpStage);   // [2][MT][STAGES][T]

    const uint32_t it0 = (uint32_t)((unsigned long long)blockIdx.x * p.total_iters / gridDim.x);
    const uint32_t it1 = (uint32_t)((unsigned long long)(blockIdx.x + 1) * p.total_iters / gridDim.x);
    const uint32_t n_it = it1 - it0;
    const bool has_block = t < p.active;
    const uint32_t b = t % p.bpc, csub = t / p.bpc;
    uint32_t my_n = has_block ? n_it : 0u;
    if (has_block && it1 == p.total_iters && n_it > 0 && (p.total_iters - 1) * p.cpi + csub >= p.n) my_n = n_it - 1;

    // A warp owns 32 consecutive blocks of each iteration: `full` of them in every iteration, and
    // `last` of them in the final iteration of the matrix (which may hold fewer columns).  active
    // is a multiple of 4 and 4 blocks are 144 B, so every source address is 16-byte aligned.
    const uint32_t w0 = warp * 32u;
    const uint32_t full = p.active > w0 ? min(32u, p.active - w0) : 0u;
    const uint32_t last_live = (p.n - (p.total_iters - 1) * p.cpi) * p.bpc;
    const uint32_t last = last_live > w0 ? min(32u, last_live - w0) : 0u;
    const bool ends_matrix = it1 == p.total_iters;
    const uint8_t *src_next = p.w + ((unsigned long long)it0 * p.active + w0) * 36ull + 16u * lane;
    const uint32_t stride = p.active * 36u;

    auto issue = [&](int stage, uint32_t iter, bool in_range) {       // iter: index inside this CTA's range
        if (in_range) {
            const uint32_t cnt = (ends_matrix && iter == n_it - 1) ? last : full;
            const uint32_t pieces = (cnt * 36u + 15u) >> 4;
            uint8_t *dst = s_w + stage * kQ8WarpStage + 16u * lane;
            if (lane < pieces) cp_async16(dst, src_next);
            if (lane + 32u < pieces) cp_async16(dst + 512, src_next + 512);
            if (lane + 64u < pieces) cp_async16(dst + 1024, src_next + 1024);
        }
        src_next += stride;
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) issue(s, (uint32_t)s, (uint32_t)s < n_it);
    grid_launch_dependents();
    grid_dependency_wait();

    XBlock xb[MT];
#pragma unroll
    for (int r = 0; r < MT; r++) load_x<0>(p.x + (size_t)r * p.k, b, xb[r]);
    const ReduceSlot slot = make_slot<STAGES>(p);

    auto block_sum = [&](int stage, float (&out)[MT]) {
        const uint32_t *bp = reinterpret_cast<const uint32_t *>(s_w + stage * kQ8WarpStage + 36u * lane);
        const uint32_t sw = bp[0];
        const float scale = __half2float(__ushort_as_half((unsigned short)(sw & 0xFFFFu)));
#pragma unroll
        for (int r = 0; r < MT; r++) out[r] = scale * xb[r].inv * dot_q8(bp + 1, xb[r]);
    };

    uint32_t round = 0;
    for (uint32_t i = 0; i < n_it; i += STAGES, round++) {
        float part[MT][STAGES];
#pragma unroll
        for (int u = 0; u < STAGES; u++) {
            __syncwarp();                                   // every lane is done reading the stage refilled next
            issue((u + STAGES - 1) % STAGES, i + u + STAGES - 1, i + u + STAGES - 1 < n_it);
            cp_async_wait<STAGES - 1>();
            __syncwarp();                                   // the other lanes' copies for this stage are visible
            float out[MT];
#pragma unroll
            for (int r = 0; r < MT; r++) out[r] = 0.f;
            if (i + u < my_n) block_sum(u, out);
#pragma unroll
            for (int r = 0; r < MT; r++) part[r][u] = out[r];
        }
        reduce_store<MT, STAGES>(p, slot, s_red + (size_t)(round & 1) * MT * STAGES * T, part, it0 + i, it1);
    }
    cp_async_wait<0>();
}

// ------------------------------------------------------------------------------ generic path

// Any K (multiple of 32), any N, any alignment of the nibble region: one warp per column, plain
// 4-byte loads.  Used only for shapes the streaming kernels do not take (K > 32768, or a packed
// buffer whose size is not a multiple of 16 bytes, K < 256).
template <int FMT>
__global__ void __launch_bounds__(256) gemv_generic_kernel(const GemvParams p, uint32_t m)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (col >= p.n) return;
    const uint32_t *w32 = reinterpret_cast<const uint32_t *>(p.w);
    for (uint32_t r = 0; r < m; r++) {
        const float *x = p.x + (size_t)r * p.k;
        float acc = 0.f;
        for (uint32_t b = lane; b < p.bpc; b += 32u) {
            const unsigned long long g = (unsigned long long)col * p.bpc + b;
            float dot = 0.f, xsum = 0.f;
            if (FMT == MGQ_FMT_Q4) {
                const uint32_t h = w32[g];
                const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&h));
                const uint32_t *nb = w32 + p.num_blocks + g * 4;
                for (int j = 0; j < 4; j++) {
                    const uint32_t wv = nb[j];
                    for (int e = 0; e < 8; e++) {
                        const float xv = x[32u * b + 8 * j + e];
                        dot = fmaf((float)((wv >> (4 * e)) & 0xFu), xv, dot);
                        xsum += xv;
                    }
                }
                acc += fmaf(dm.x, dot, dm.y * xsum);
            } else {
                const uint32_t *bp = w32 + g * 9;
                const float scale = __half2float(__ushort_as_half((unsigned short)(bp[0] & 0xFFFFu)));
                for (int j = 0; j < 8; j++) {
                    const uint32_t wv = bp[1 + j];
                    for (int e = 0; e < 4; e++)
                        dot = fmaf((float)(int)(signed char)((wv >> (8 * e)) & 0xFFu), x[32u * b + 4 * j + e], dot);
                }
                acc += scale * dot;
            }
        }
        for (uint32_t o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            const size_t o = (size_t)r * p.n + col;
            p.y[o] = p.addend ? acc + p.addend[o] : acc;
        }
    }
}

// ------------------------------------------------------------------------------ launch logic

struct Config {
    uint32_t threads, cpi, red_shift, red_chunk;
    int stages;
};

// Largest column count per iteration that fits `threads` and keeps cpi*bpc a multiple of 4
// (so that a Q8 warp's 36-byte blocks always start on a 16-byte boundary).
uint32_t columns_for(uint32_t threads, uint32_t bpc)
{
    uint32_t cpi = threads / bpc;
    const uint32_t need = bpc % 4 == 0 ? 1u : (bpc % 2 == 0 ? 2u : 4u);
    return cpi - cpi % need;
}

// Depends on K only, so that a column's summation order is the same for every N.
Config choose_config(uint32_t bpc)
{
    Config c{};
    if (bpc <= 256) {
        uint32_t best_t = 0;
        double best_u = -1.0;
        for (uint32_t t = 128; t <= 256; t += 32) {
            const double util = (double)(columns_for(t, bpc) * bpc) / t;
            if (util > best_u + 1e-9) { best_u = util; best_t = t; }
        }
        c.threads = best_t;
    } else {
        c.threads = (bpc + 31u) & ~31u;
    }
    c.cpi = columns_for(c.threads, bpc);
    c.stages = c.threads <= 512 ? 8 : 4;
    // finishing lanes per column: a power of two, at most 32, with stages*cpi*lanes <= threads
    const uint32_t slots = (uint32_t)c.stages * c.cpi;
    c.red_shift = 0;
    while (c.red_shift < 5 && (slots << (c.red_shift + 1)) <= c.threads && (2u << c.red_shift) <= bpc) c.red_shift++;
    const uint32_t lanes = 1u << c.red_shift;
    c.red_chunk = (bpc + lanes - 1) / lanes;
    if (c.red_chunk % 4 != 0 && bpc % 4 == 0 && c.red_chunk > 4) c.red_chunk = (c.red_chunk + 3u) & ~3u;
    return c;
}

size_t smem_bytes(int fmt, const Config &c, int mt)
{
    const size_t red = (size_t)2 * mt * c.stages * c.threads * sizeof(float);
    if (fmt == MGQ_FMT_Q4) return (size_t)c.stages * c.threads * 20 + red;
    return (size_t)(c.threads / 32) * c.stages * kQ8WarpStage + red;
}

using KernelFn = void (*)(const GemvParams);

KernelFn pick_kernel(int fmt, int mt, const Config &c)
{
    if (fmt == MGQ_FMT_Q4) {
        if (c.threads <= 256) return mt == 2 ? gemv_q4_kernel<2, 8, 256> : gemv_q4_kernel<1, 8, 256>;
        if (c.threads <= 512) return mt == 2 ? gemv_q4_kernel<2, 8, 512> : gemv_q4_kernel<1, 8, 512>;
        return mt == 1 ? gemv_q4_kernel<1, 4, 1024> : nullptr;
    }
    if (c.threads <= 256) return mt == 2 ? gemv_q8_kernel<2, 8, 256> : gemv_q8_kernel<1, 8, 256>;
    if (c.threads <= 512) return mt == 2 ? gemv_q8_kernel<2, 8, 512> : gemv_q8_kernel<1, 8, 512>;
    return mt == 1 ? gemv_q8_kernel<1, 4, 1024> : nullptr;
}

struct DeviceInfo {
    int sms = 0;
    bool ok = false;
};

int device_info(DeviceInfo &out)
{
    static std::mutex mu;
    static DeviceInfo cache[64];
    int dev = 0;
    MGQ_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64) return fail(MGQ_ERR_CUDA, "device index %d out of range", dev);
    if (!cache[dev].ok) {
        MGQ_CUDA(cudaDeviceGetAttribute(&cache[dev].sms, cudaDevAttrMultiProcessorCount, dev));
        cache[dev].ok = true;
    }
    out = cache[dev];
    return MGQ_OK;
}

// Returns resident CTAs per SM for (kernel, threads, smem).  The first use of a kernel on a
// device opts it into the device's largest dynamic shared memory size (one setting per kernel:
// a later, smaller request must not lower it).  Answers are remembered: both calls cost
// microseconds.
int kernel_occupancy(KernelFn fn, uint32_t threads, size_t smem, int &occ)
{
    struct Entry { int dev; KernelFn fn; uint32_t threads; size_t smem; int occ; };
    static std::mutex mu;
    static std::vector<Entry> seen;
    int dev = 0;
    MGQ_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    bool opted_in = false;
    for (const Entry &e : seen) {
        if (e.dev != dev || e.fn != fn) continue;
        opted_in = true;
        if (e.threads == threads && e.smem == smem) { occ = e.occ; return MGQ_OK; }
    }
    int optin = 0;
    MGQ_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if (smem > (size_t)optin) return fail(MGQ_ERR_SHAPE, "GEMV needs %zu B of shared memory, device allows %d", smem, optin);
    if (!opted_in) MGQ_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, optin));
    MGQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, fn, (int)threads, smem));
    if (occ < 1) return fail(MGQ_ERR_CUDA, "GEMV kernel does not fit on an SM (threads=%u smem=%zu)", threads, smem);
    seen.push_back({dev, fn, threads, smem, occ});
    return MGQ_OK;
}

// MGQ_SERIAL_DISPATCH=1 turns programmatic dependent launch off (every kernel then starts only
// after its predecessor has finished), like the reference's MEGANEURA_SERIAL_DISPATCH debugging
// switch (src/runtime.rs:1703-1707).
bool overlap_allowed()
{
    static const bool allowed = [] {
        const char *v = std::getenv("MGQ_SERIAL_DISPATCH");
        return !(v && v[0] == '1');
    }();
    return allowed;
}

#ifdef MGQ_GEMV_TRACE
unsigned long long *g_trace = nullptr;
#endif

}  // namespace

#ifdef MGQ_GEMV_TRACE
extern "C" void mgq_debug_set_trace(unsigned long long *dev_buffer) { g_trace = dev_buffer; }
#endif

int launch_gemv(int fmt, const float *x, const void *w, const float *addend, float *y,
                uint32_t m, uint32_t k, uint32_t n, void *stream_v)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const uint32_t bpc = k / 32;
    GemvParams p{};
    p.k = k; p.n = n; p.bpc = bpc;
    p.num_blocks = (unsigned long long)bpc * n;
    p.w = static_cast<const uint8_t *>(w);

    const bool streamable = bpc >= 8 && bpc <= 1024 && (p.num_blocks % 4 == 0) &&
                            (reinterpret_cast<uintptr_t>(x) % 16 == 0);
    if (!streamable) {
        p.x = x; p.addend = addend; p.y = y;
        const uint32_t warps = 8, grid = (n + warps - 1) / warps;
        if (fmt == MGQ_FMT_Q4) gemv_generic_kernel<MGQ_FMT_Q4><<<grid, warps * 32, 0, stream>>>(p, m);
        else                   gemv_generic_kernel<MGQ_FMT_Q8><<<grid, warps * 32, 0, stream>>>(p, m);
        MGQ_CUDA(cudaGetLastError());
        return MGQ_OK;
    }

    const Config cfg = choose_config(bpc);
    p.cpi = cfg.cpi;
    p.active = cfg.cpi * bpc;
    p.red_shift = cfg.red_shift;
    p.red_chunk = cfg.red_chunk;
    p.total_iters = (n + cfg.cpi - 1) / cfg.cpi;
    DeviceInfo di;
    if (int rc = device_info(di)) return rc;

    // Rows are processed two at a time (their activations live in registers); more rows re-read W.
    for (uint32_t r0 = 0; r0 < m;) {
        int mt = (m - r0 >= 2 && cfg.threads <= 512) ? 2 : 1;
        KernelFn fn = pick_kernel(fmt, mt, cfg);
        if (!fn) return fail(MGQ_ERR_SHAPE, "no GEMV kernel for K=%u", k);
        const size_t smem = smem_bytes(fmt, cfg, mt);
        int occ = 0;
        if (int rc = kernel_occupancy(fn, cfg.threads, smem, occ)) return rc;
        uint32_t grid = (uint32_t)di.sms * (uint32_t)occ;
        if (grid > p.total_iters) grid = p.total_iters;
        p.x = x + (size_t)r0 * k;
        p.addend = addend ? addend + (size_t)r0 * n : nullptr;
        p.y = y + (size_t)r0 * n;
#ifdef MGQ_GEMV_TRACE
        p.trace = g_trace;
        if (g_trace) g_trace += (size_t)grid * 4;
#endif
        cudaLaunchConfig_t lc{};
        lc.gridDim = dim3(grid, 1, 1);
        lc.blockDim = dim3(cfg.threads, 1, 1);
        lc.dynamicSmemBytes = smem;
        lc.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = overlap_allowed() ? 1 : 0;
        MGQ_CUDA(cudaLaunchKernelEx(&lc, fn, p));
        r0 += mt;
    }
    return MGQ_OK;
}

}  // namespace mgq
