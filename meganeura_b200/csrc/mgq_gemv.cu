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
#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "mgq_gemv_device.cuh"
#include "mgq_internal.h"

namespace mgq {
namespace {

using namespace dev;

// ------------------------------------------------------------------------------------ Q4

// A "group" is cpi consecutive columns: one block for each of the `active` threads.  A CTA owns
// the groups [g0, g1); a pipeline stage holds C consecutive groups, so a thread works on C
// columns with the same activations before it touches the ring again.
//
// TS is the launch bound and the stride of every shared-memory array (threads <= TS), so that all
// shared-memory addressing folds into immediates.  Threads beyond `active` shadow the last active
// thread: they fetch and compute like everybody else, and nothing ever reads what they produce.
// A CTA runs "fast" rounds, in which every fetch and every block is known to be in range and the
// code carries no predicates, and then at most a few "checked" rounds at the end of its range.
constexpr int kStages = 4;

struct CtaRange {
    uint32_t g0, g1, n_g;
    uint32_t n_full;     // leading groups of the range in which every column of the group exists (CTA-uniform)
};

__device__ __forceinline__ CtaRange cta_range(const GemvParams &p)
{
    CtaRange r;
    r.g0 = (uint32_t)((unsigned long long)blockIdx.x * p.total_iters / gridDim.x);
    r.g1 = (uint32_t)((unsigned long long)(blockIdx.x + 1) * p.total_iters / gridDim.x);
    r.n_g = r.g1 - r.g0;
    const bool ragged_end = r.g1 == p.total_iters && r.n_g > 0 && p.total_iters * p.cpi != p.n;
    r.n_full = ragged_end ? r.n_g - 1 : r.n_g;
    return r;
}

template <int MT, int C, int TS>
__global__ void __launch_bounds__(TS) gemv_q4_kernel(const GemvParams p)
{
    constexpr int STAGES = kStages, ROUND = kStages * C;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t t = threadIdx.x;
    uint4 *s_nib = reinterpret_cast<uint4 *>(smem) + t;                                  // [ROUND][TS], own slot
    uint32_t *s_hdr = reinterpret_cast<uint32_t *>(smem + ROUND * TS * 16) + t;          // [ROUND][TS], own slot
    float *s_red = reinterpret_cast<float *>(smem + ROUND * TS * 20);                    // [2][MT][ROUND][TS] (+ [TS])

    const CtaRange cr = cta_range(p);
    const uint32_t tt = t < p.active ? t : p.active - 1;
    const uint32_t b = tt % p.bpc, csub = tt / p.bpc;
    // groups in which this thread's column exists: all, except that the very last group of the
    // matrix may hold fewer than cpi columns
    const uint32_t my_n = (cr.n_full != cr.n_g && (p.total_iters - 1) * p.cpi + csub >= p.n) ? cr.n_g - 1 : cr.n_g;

    const unsigned long long first = (unsigned long long)cr.g0 * p.active + tt;          // = col*bpc + b
    const uint32_t *hdr_base = reinterpret_cast<const uint32_t *>(p.w) + first;
    const uint4 *nib_base = reinterpret_cast<const uint4 *>(p.w + p.num_blocks * 4) + first;
    const uint32_t stride = p.active;
    uint32_t off = 0;                                                                    // blocks from `first` to the next fetch
    uint32_t g_next = 0;                                                                 // next group to fetch

    auto issue = [&](int stage, auto checked) {
#pragma unroll
        for (int j = 0; j < C; j++) {
            if (!decltype(checked)::value || g_next + j < my_n) {
                cp_async16(s_nib + (stage * C + j) * TS, nib_base + off);
                cp_async4(s_hdr + (stage * C + j) * TS, hdr_base + off);
            }
            off += stride;
        }
        if (decltype(checked)::value) g_next += C;
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) issue(s, std::true_type{});       // weights first: they depend on nothing
    grid_launch_dependents();
    grid_dependency_wait();                                                 // x, addend and y belong to earlier kernels
    exchange_poll(p, t % p.bpc);                                            // ... or to other GPUs

    XBlock xb[MT];
#pragma unroll
    for (int r = 0; r < MT; r++) {
        // x is either a local vector (read-only path: the CTAs of an SM share one fetch) or, when the
        // caller passed none, the gathered vector that was just polled (written by other GPUs: L2 only)
        if (p.x) load_x<1, false>(p.x + (size_t)r * p.k, b, xb[r]);
        else          load_x_gathered<1>(p.wait_vec, b, xb[r]);
    }
    const ReduceSlot slot = make_slot<ROUND, TS>(p);

    auto block_sum = [&](int idx, float (&part)[MT][ROUND]) {
        const uint4 q = s_nib[idx * TS];
        const uint32_t h = s_hdr[idx * TS];
        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&h));       // (d, m), IEEE
#pragma unroll
        for (int r = 0; r < MT; r++) part[r][idx] = fmaf(dm.x * xb[r].inv, dot_q4(q, xb[r]), dm.y * xb[r].sum);
    };

    auto do_round = [&](uint32_t g, uint32_t round, auto checked) {
        float part[MT][ROUND];
#pragma unroll
        for (int u = 0; u < STAGES; u++) {
            issue((u + STAGES - 1) % STAGES, checked);
            cp_async_wait<STAGES - 1>();
#pragma unroll
            for (int j = 0; j < C; j++) {
                // past the end of the range the slot holds stale bytes; what is computed from them
                // belongs to no column, but skipping it saves the time
                if (!decltype(checked)::value || g + u * C + j < cr.n_g) block_sum(u * C + j, part);
                else {
#pragma unroll
                    for (int r = 0; r < MT; r++) part[r][u * C + j] = 0.f;
                }
            }
        }
        reduce_store<MT, ROUND, true, TS>(p, slot, s_red + (round & 1) * MT * ROUND * TS, part, cr.g0 + g, cr.g1,
                                          p.push ? s_red + 2 * MT * ROUND * TS : nullptr);
    };

    uint32_t g = 0, round = 0;
    // fast rounds: the round itself and everything it prefetches (STAGES-1 stages ahead) is in range
    for (; g + 2 * ROUND - C <= cr.n_full; g += ROUND, round++) do_round(g, round, std::false_type{});
    g_next = g + (STAGES - 1) * C;
    for (; g < cr.n_g; g += ROUND, round++) do_round(g, round, std::true_type{});
    cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------ Q8

template <int MT, int C, int TS>
__global__ void __launch_bounds__(TS) gemv_q8_kernel(const GemvParams p)
{
    constexpr int STAGES = kStages, ROUND = kStages * C;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t t = threadIdx.x, lane = t & 31u, warp = t >> 5;
    uint8_t *s_w = smem + warp * (ROUND * kQ8WarpStage);                                 // this warp's ring [ROUND][1152]
    float *s_red = reinterpret_cast<float *>(smem + (TS / 32) * ROUND * kQ8WarpStage);   // [2][MT][ROUND][TS] (+ [TS])

    const CtaRange cr = cta_range(p);
    const uint32_t tt = t < p.active ? t : p.active - 1;
    const uint32_t b = tt % p.bpc;

    // A warp owns 32 consecutive blocks of each group: `full` of them in every group, and `last`
    // of them in the final group of the matrix (which may hold fewer columns).  active is a
    // multiple of 4 and 4 blocks are 144 B, so every source address is 16-byte aligned.
    const uint32_t w0 = warp * 32u;
    const uint32_t full = p.active > w0 ? min(32u, p.active - w0) : 0u;
    const uint32_t last_live = (p.n - (p.total_iters - 1) * p.cpi) * p.bpc;
    const uint32_t last = last_live > w0 ? min(32u, last_live - w0) : 0u;
    const uint32_t last_group = cr.g1 == p.total_iters ? cr.n_g - 1 : 0xFFFFFFFFu;       // index inside this CTA's range
    const uint8_t *src_base = p.w + ((unsigned long long)cr.g0 * p.active + w0) * 36ull + 16u * lane;
    const uint32_t stride = p.active * 36u;
    uint32_t off = 0;                                                                    // bytes from src_base to the next fetch
    uint32_t g_next = 0;
    const bool whole_warp = full == 32u;                                                 // 1152 bytes per group: 72 pieces

    auto issue = [&](int stage, auto checked) {
#pragma unroll
        for (int j = 0; j < C; j++) {
            uint8_t *dst = s_w + (stage * C + j) * kQ8WarpStage + 16u * lane;
            const uint8_t *src = src_base + off;
            if (!decltype(checked)::value && whole_warp) {
                cp_async16(dst, src);
                cp_async16(dst + 512, src + 512);
                if (lane < 8u) cp_async16(dst + 1024, src + 1024);
            } else {
                const uint32_t gi = g_next + j;
                if (!decltype(checked)::value || gi < cr.n_g) {
                    const uint32_t cnt = (decltype(checked)::value && gi == last_group) ? last : full;
                    const uint32_t pieces = (cnt * 36u + 15u) >> 4;
                    if (lane < pieces) cp_async16(dst, src);
                    if (lane + 32u < pieces) cp_async16(dst + 512, src + 512);
                    if (lane + 64u < pieces) cp_async16(dst + 1024, src + 1024);
                }
            }
            off += stride;
        }
        if (decltype(checked)::value) g_next += C;
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) issue(s, std::true_type{});
    grid_launch_dependents();
    grid_dependency_wait();
    exchange_poll(p, t % p.bpc);

    XBlock xb[MT];
#pragma unroll
    for (int r = 0; r < MT; r++) {
        if (p.x) load_x<0, false>(p.x + (size_t)r * p.k, b, xb[r]);
        else          load_x_gathered<0>(p.wait_vec, b, xb[r]);
    }
    const ReduceSlot slot = make_slot<ROUND, TS>(p);

    auto block_sum = [&](int idx, float (&part)[MT][ROUND]) {
        const uint32_t *bp = reinterpret_cast<const uint32_t *>(s_w + idx * kQ8WarpStage + 36u * lane);
        const uint32_t sw = bp[0];
        const float scale = __half2float(__ushort_as_half((unsigned short)(sw & 0xFFFFu)));
#pragma unroll
        for (int r = 0; r < MT; r++) part[r][idx] = scale * xb[r].inv * dot_q8(bp + 1, xb[r]);
    };

    auto do_round = [&](uint32_t g, uint32_t round, auto checked) {
        float part[MT][ROUND];
#pragma unroll
        for (int u = 0; u < STAGES; u++) {
            __syncwarp();                                   // every lane is done reading the stage refilled next
            issue((u + STAGES - 1) % STAGES, checked);
            cp_async_wait<STAGES - 1>();
            __syncwarp();                                   // the other lanes' copies for this stage are visible
#pragma unroll
            for (int j = 0; j < C; j++) {
                if (!decltype(checked)::value || g + u * C + j < cr.n_g) block_sum(u * C + j, part);
                else {
#pragma unroll
                    for (int r = 0; r < MT; r++) part[r][u * C + j] = 0.f;
                }
            }
        }
        reduce_store<MT, ROUND, true, TS>(p, slot, s_red + (round & 1) * MT * ROUND * TS, part, cr.g0 + g, cr.g1,
                                          p.push ? s_red + 2 * MT * ROUND * TS : nullptr);
    };

    uint32_t g = 0, round = 0;
    for (; g + 2 * ROUND - C <= cr.n_full; g += ROUND, round++) do_round(g, round, std::false_type{});
    g_next = g + (STAGES - 1) * C;
    for (; g < cr.n_g; g += ROUND, round++) do_round(g, round, std::true_type{});
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
    uint32_t threads, cpi, cols_per_thread, red_shift, red_chunk;
};

// Tunables (0 = automatic), settable through mgq_set_option.
struct Tuning {
    int cols_per_thread = 0;   // "gemv.columns_per_thread": 1 or 2
    int ctas_per_sm = 0;       // "gemv.ctas_per_sm"
    int serial = -1;           // "gemv.serial_dispatch": 1 turns programmatic dependent launch off
    int batch_mma = 1;          // "gemv.batch_mma": 3..16 rows run on the mma kernel (0: pairs of rows on the streaming kernels)
    long wait_us = 0;           // "gemv.wait_us": time limit of the exchange's stamp polls (0: 2000000; peers may launch seconds apart)
};
Tuning g_tuning;

// Largest column count per group that fits `threads` and keeps cpi*bpc a multiple of 4
// (so that a Q8 warp's 36-byte blocks always start on a 16-byte boundary).
uint32_t columns_for(uint32_t threads, uint32_t bpc)
{
    uint32_t cpi = threads / bpc;
    const uint32_t need = bpc % 4 == 0 ? 1u : (bpc % 2 == 0 ? 2u : 4u);
    return cpi - cpi % need;
}

// Shared-memory stride class of a thread count: the kernels are instantiated for these bounds.
uint32_t stride_class(uint32_t threads)
{
    for (uint32_t ts : {128u, 256u, 384u, 512u}) if (threads <= ts) return ts;
    return 1024u;
}

size_t smem_bytes(int fmt, uint32_t threads, int c, int mt)
{
    const size_t ts = stride_class(threads);
    const size_t round = (size_t)kStages * c;
    const size_t red = 2 * mt * round * ts * sizeof(float) + ts * sizeof(float);   // + one round of finished columns (exchange)
    if (fmt == MGQ_FMT_Q4) return round * ts * 20 + red;
    return (ts / 32) * round * kQ8WarpStage + red;
}

// Thread count and summation order depend on K only, so that a column's result is the same for
// every N (column shards reproduce the unsharded result bit for bit).  The number of columns a
// thread handles per stage depends on N, but does not change any sum.
Config choose_config(int fmt, uint32_t bpc, uint32_t n, int mt, int sms)
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
    const uint32_t groups = (n + c.cpi - 1) / c.cpi;
    // columns per thread and stage: as many as keep every CTA of a two-per-SM grid busy, fit
    // in ~100 KB of shared memory and leave one finishing lane per column of a round
    int cols = 1;
    for (int cand : {2}) {
        if (g_tuning.cols_per_thread && cand != g_tuning.cols_per_thread) continue;
        if (c.threads > 512) continue;
        if ((uint32_t)(kStages * cand) * c.cpi > c.threads) continue;
        if (smem_bytes(fmt, c.threads, cand, mt) > 100 * 1024) continue;
        if (!g_tuning.cols_per_thread && groups / cand < 3u * (uint32_t)sms) continue;
        cols = cand;
        break;
    }
    c.cols_per_thread = (uint32_t)cols;
    // finishing lanes per column: a power of two, at most 32, sized for the widest round
    // (4 columns per thread) whatever `cols` is, so that the summation order depends on K only
    const uint32_t slots = (uint32_t)(kStages * 4) * c.cpi;
    c.red_shift = 0;
    while (c.red_shift < 5 && (slots << (c.red_shift + 1)) <= c.threads && (2u << c.red_shift) <= bpc) c.red_shift++;
    // (when even one lane per column does not fit the widest round, `cols` was capped above)
    const uint32_t lanes = 1u << c.red_shift;
    c.red_chunk = (bpc + lanes - 1) / lanes;
    if (c.red_chunk % 4 != 0 && bpc % 4 == 0 && c.red_chunk > 4) c.red_chunk = (c.red_chunk + 3u) & ~3u;
    return c;
}

using KernelFn = void (*)(const GemvParams);

template <int MT, int C>
KernelFn pick_by_threads(int fmt, uint32_t threads)
{
    const bool q4 = fmt == MGQ_FMT_Q4;
    switch (stride_class(threads)) {
        case 128: return q4 ? (KernelFn)gemv_q4_kernel<MT, C, 128> : (KernelFn)gemv_q8_kernel<MT, C, 128>;
        case 256: return q4 ? (KernelFn)gemv_q4_kernel<MT, C, 256> : (KernelFn)gemv_q8_kernel<MT, C, 256>;
        case 384: return q4 ? (KernelFn)gemv_q4_kernel<MT, C, 384> : (KernelFn)gemv_q8_kernel<MT, C, 384>;
        case 512: return q4 ? (KernelFn)gemv_q4_kernel<MT, C, 512> : (KernelFn)gemv_q8_kernel<MT, C, 512>;
        default: return nullptr;
    }
}

KernelFn pick_kernel(int fmt, int mt, const Config &c)
{
    if (c.threads > 512) {
        if (mt != 1 || c.cols_per_thread != 1) return nullptr;
        return fmt == MGQ_FMT_Q4 ? (KernelFn)gemv_q4_kernel<1, 1, 1024> : (KernelFn)gemv_q8_kernel<1, 1, 1024>;
    }
    if (c.cols_per_thread == 2) return mt == 2 ? pick_by_threads<2, 2>(fmt, c.threads) : pick_by_threads<1, 2>(fmt, c.threads);
    return mt == 2 ? pick_by_threads<2, 1>(fmt, c.threads) : pick_by_threads<1, 1>(fmt, c.threads);
}

struct DeviceInfo {
    int sms = 0;
    size_t smem_per_sm = 0, smem_reserved = 0;     // shared memory of an SM, and what every resident CTA costs on top of its request
    size_t smem_optin = 0;                         // largest dynamic request one CTA may make
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
        int per_sm = 0, reserved = 0;
        MGQ_CUDA(cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev));
        MGQ_CUDA(cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev));
        cache[dev].smem_per_sm = (size_t)per_sm;
        cache[dev].smem_reserved = (size_t)reserved;
        int optin = 0;
        MGQ_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        cache[dev].smem_optin = (size_t)optin;
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
    if (g_tuning.serial >= 0) return g_tuning.serial == 0;
    static const bool allowed = [] {
        const char *v = std::getenv("MGQ_SERIAL_DISPATCH");
        return !(v && v[0] == '1');
    }();
    return allowed;
}

unsigned long long exchange_wait_ns() { return (unsigned long long)(g_tuning.wait_us > 0 ? g_tuning.wait_us : 2000000) * 1000ull; }

}  // namespace

int set_gemv_option(const char *name, long value)
{
    if (!std::strcmp(name, "gemv.columns_per_thread")) {
        if (value != 0 && value != 1 && value != 2) return fail(MGQ_ERR_SHAPE, "%s must be 0, 1 or 2", name);
        g_tuning.cols_per_thread = (int)value;
    } else if (!std::strcmp(name, "gemv.ctas_per_sm")) {
        if (value < 0 || value > 32) return fail(MGQ_ERR_SHAPE, "%s out of range", name);
        g_tuning.ctas_per_sm = (int)value;
    } else if (!std::strcmp(name, "gemv.serial_dispatch")) {
        g_tuning.serial = value < 0 ? -1 : (value ? 1 : 0);
    } else if (!std::strcmp(name, "gemv.batch_mma")) {
        g_tuning.batch_mma = value ? 1 : 0;
    } else if (!std::strcmp(name, "gemv.wait_us")) {
        if (value < 0 || value > 10000000) return fail(MGQ_ERR_SHAPE, "%s out of range", name);
        g_tuning.wait_us = value;
    } else {
        return fail(MGQ_ERR_NAME, "unknown option: %s", name);
    }
    return MGQ_OK;
}

// Ends a token on this GPU: waits (bounded) until every element of the last gathered vector carries
// this token's stamp, then the block that finishes last advances the local token index.
__global__ void exchange_finish_kernel(const float2 *last_vec, uint32_t length, unsigned long long *epoch,
                                       unsigned int *error, unsigned int *blocks_done, unsigned long long wait_ns)
{
    const uint32_t stamp = dev::exchange_stamp(epoch);
    if (last_vec) {
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < length; i += gridDim.x * blockDim.x) {
            unsigned long long t0 = 0;
            for (uint32_t spins = 0;; spins++) {
                uint32_t got;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(got) : "l"(&last_vec[i].y) : "memory");
                if (got == stamp) break;
                if ((spins & 31u) == 31u) {
                    const unsigned long long now = dev::global_timer_ns();
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > wait_ns) { atomicExch(error, 1u); break; }
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(blocks_done, 1u) == gridDim.x - 1) {
            atomicExch(blocks_done, 0u);
            *reinterpret_cast<volatile unsigned long long *>(epoch) = (unsigned long long)stamp;   // token + 1
            __threadfence();
        }
    }
}

int launch_exchange_finish(const void *last_vec, uint32_t length, unsigned long long *epoch,
                           unsigned int *error, unsigned int *blocks_done, void *stream_v)
{
    const uint32_t threads = 256;
    uint32_t grid = last_vec ? (length + threads * 4 - 1) / (threads * 4) : 1;
    if (grid > 148) grid = 148;
    if (grid < 1) grid = 1;
    exchange_finish_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream_v)>>>(
        static_cast<const float2 *>(last_vec), length, epoch, error, blocks_done, exchange_wait_ns());
    MGQ_CUDA(cudaGetLastError());
    return MGQ_OK;
}

// All-gather of a plain vector slice over peer memory, for the operators between the GEMVs of a
// column-sharded model (attention output, SwiGLU output) and for turning a gathered vector back into
// a plain one: every CTA first stores its part of this rank's slice as {value, stamp} elements into
// every rank's gathered vector (skipped when the producing GEMV has already pushed it), then waits
// -- bounded -- for its part of the whole local vector and writes the values out plain.  The waits
// are for other GPUs' stores and for stores of this launch's own CTAs made before they wait, so the
// grid is kept small enough to be resident at once.
__global__ void __launch_bounds__(256) all_gather_kernel(const float *slice, const mgq_exchange_push *push, const float2 *local_vec,
                                                         float *out, uint32_t rows, uint32_t cols, uint32_t pitch, uint32_t world,
                                                         const unsigned long long *epoch, unsigned int *error, unsigned long long wait_ns)
{
    // A rank's slice is `rows` rows of `cols` columns (row stride `pitch`); in a gathered vector the
    // slices stand rank after rank, each row-major; `out` is the whole [rows, world * cols] matrix.
    const uint32_t stamp = dev::exchange_stamp(epoch);
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
    const uint32_t slice_len = rows * cols;
    if (slice) {
        const size_t at = (size_t)push->rank * push->gather_cols;
        for (uint32_t i = tid; i < slice_len; i += nthreads) {
            const uint32_t r = i / cols, c = i - r * cols;
            const float v = slice[(size_t)r * pitch + c];
            const unsigned long long e = (unsigned long long)__float_as_uint(v) | ((unsigned long long)stamp << 32);
            for (uint32_t q = 0; q < world; q++)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long *>(push->dst[q]) + at + i), "l"(e) : "memory");
        }
    }
    if (!out) return;                                 // store only: the reader waits for the elements itself
    const uint32_t total = world * slice_len;
    for (uint32_t i = tid; i < total; i += nthreads) {
        unsigned long long t0 = 0, e;
        for (uint32_t spins = 0;; spins++) {
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(e) : "l"(local_vec + i) : "memory");
            if ((uint32_t)(e >> 32) == stamp) break;
            if ((spins & 31u) == 31u) {
                if (*reinterpret_cast<const volatile uint32_t *>(error) != 0u) break;
                const unsigned long long now = dev::global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > wait_ns) { atomicExch(error, 1u); break; }
            }
        }
        const uint32_t q = i / slice_len, rem = i - q * slice_len, r = rem / cols, c = rem - r * cols;
        out[(size_t)r * world * cols + (size_t)q * cols + c] = __uint_as_float((uint32_t)e);
    }
}

int launch_all_gather(const float *slice, const void *push_dev, const void *local_vec, float *out, uint32_t rows, uint32_t cols,
                      uint32_t pitch, uint32_t world, const unsigned long long *epoch, unsigned int *error, void *stream_v)
{
    const uint32_t threads = 256;
    uint32_t grid = ((out ? world : 1u) * rows * cols + threads - 1) / threads;
    if (grid > 148) grid = 148;
    if (grid < 1) grid = 1;
    all_gather_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream_v)>>>(
        slice, static_cast<const mgq_exchange_push *>(push_dev), static_cast<const float2 *>(local_vec), out, rows, cols, pitch, world,
        epoch, error, exchange_wait_ns());
    MGQ_CUDA(cudaGetLastError());
    return MGQ_OK;
}

bool gemv_streamable(const void *x, uint32_t k, uint32_t n)
{
    const uint32_t bpc = k / 32;
    return bpc >= 8 && bpc <= 1024 && (((unsigned long long)bpc * n) % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
}

int launch_gemv(int fmt, const float *x, const void *w, const float *addend, float *y,
                uint32_t m, uint32_t k, uint32_t n, void *stream_v, const GemvExchange *xchg)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const uint32_t bpc = k / 32;
    GemvParams p{};
    p.k = k; p.n = n; p.bpc = bpc;
    p.num_blocks = (unsigned long long)bpc * n;
    p.w = static_cast<const uint8_t *>(w);
    if (xchg) {
        p.push = static_cast<const dev::ExchangePush *>(xchg->push_dev);
        p.wait_vec = static_cast<const float2 *>(xchg->wait_vec);
        p.epoch = xchg->epoch;
        p.xerror = xchg->error;
        p.wait_ns = exchange_wait_ns();
    }

    if (!xchg && g_tuning.batch_mma && gemv_mma_eligible(m, k, n, x, w))
        return launch_gemv_mma(fmt, x, w, addend, y, m, k, n, stream_v);
    const bool streamable = gemv_streamable(x, k, n);
    if (!streamable) {
        if (xchg) return fail(MGQ_ERR_SHAPE, "this shape has no exchanging GEMV kernel (K=%u N=%u)", k, n);
        p.x = x; p.addend = addend; p.y = y;
        const uint32_t warps = 8, grid = (n + warps - 1) / warps;
        if (fmt == MGQ_FMT_Q4) gemv_generic_kernel<MGQ_FMT_Q4><<<grid, warps * 32, 0, stream>>>(p, m);
        else                   gemv_generic_kernel<MGQ_FMT_Q8><<<grid, warps * 32, 0, stream>>>(p, m);
        MGQ_CUDA(cudaGetLastError());
        return MGQ_OK;
    }

    DeviceInfo di;
    if (int rc = device_info(di)) return rc;

    // Rows are processed two at a time (their activations live in registers); more rows re-read W.
    for (uint32_t r0 = 0; r0 < m;) {
        const int mt = (m - r0 >= 2 && bpc <= 512) ? 2 : 1;
        const Config cfg = choose_config(fmt, bpc, n, mt, di.sms);
        p.cpi = cfg.cpi;
        p.active = cfg.cpi * bpc;
        p.red_shift = cfg.red_shift;
        p.red_chunk = cfg.red_chunk;
        p.total_iters = (n + cfg.cpi - 1) / cfg.cpi;
        KernelFn fn = pick_kernel(fmt, mt, cfg);
        if (!fn) return fail(MGQ_ERR_SHAPE, "no GEMV kernel for K=%u", k);
        const size_t smem = smem_bytes(fmt, cfg.threads, (int)cfg.cols_per_thread, mt);
        int occ = 0;
        if (int rc = kernel_occupancy(fn, cfg.threads, smem, occ)) return rc;
        const uint32_t stages_total = (p.total_iters + cfg.cols_per_thread - 1) / cfg.cols_per_thread;
        // 3 CTAs per SM leave room for the next GEMV's CTAs to become resident and prefetch while this
        // one drains; a long stream (>= 64 stages per CTA even at full occupancy) is better served by
        // every warp the SM can hold
        int per_sm = g_tuning.ctas_per_sm > 0 ? g_tuning.ctas_per_sm : 3;
        if (!g_tuning.ctas_per_sm && stages_total >= 64u * (uint32_t)di.sms * (uint32_t)occ) per_sm = occ;
        if (per_sm > occ) per_sm = occ;
        // wide CTAs (K >= 12288) with only a few stages each: one CTA per SM halves the per-CTA start-up
        // (activation fetch and preparation) and the partly filled last round
        if (!g_tuning.ctas_per_sm && cfg.threads >= 384 && stages_total < 8u * (uint32_t)di.sms * (uint32_t)per_sm) per_sm = 1;
        uint32_t grid = (uint32_t)di.sms * (uint32_t)per_sm;
        if (grid > stages_total) grid = stages_total;
        // With programmatic dependent launch the CTAs of the next kernel take whatever room is left on
        // an SM while this one still runs; the hardware packs them onto the first SMs that have room,
        // which leaves the other SMs short of work, and co-resident CTAs that only wait were measured
        // to cost more than their early prefetch gains.  So the shared-memory request is padded until
        // exactly per_sm CTAs fit: a successor's CTA starts when one of ours exits.
        size_t launch_smem = smem;
        if (overlap_allowed() && occ > per_sm) {
            const size_t share = di.smem_per_sm / (size_t)per_sm;
            if (share > di.smem_reserved + smem) launch_smem = (share - di.smem_reserved) & ~(size_t)127;
            if (launch_smem > di.smem_optin) launch_smem = di.smem_optin;
        }
        p.x = x + (size_t)r0 * k;
        p.addend = addend ? addend + (size_t)r0 * n : nullptr;
        p.y = y + (size_t)r0 * n;
        cudaLaunchConfig_t lc{};
        lc.gridDim = dim3(grid, 1, 1);
        lc.blockDim = dim3(cfg.threads, 1, 1);
        lc.dynamicSmemBytes = launch_smem;
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
