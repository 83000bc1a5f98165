// Dequantize-fused GEMM on the sm_100a tensor cores (tcgen05 + TMEM) for M >= 64 tokens:
//     C[m,n] = A[m,k] (bf16) . dequant(W)[k,n] (+ addend),   f32 accumulation, f32 out.
//
// Stands in for the MatMul / FusedMatMulAdd dispatch with a quantized weight_format
// (src/compile.rs:1408-1419, 1511-1522 of meganeura; kernel src/shaders/matmul.wgsl with
// dequant_q4 / dequant_q8 as the B-tile load).  The reference runs this shape on scalar FP32
// ALUs (its cooperative-matrix path excludes quantized weights, src/runtime.rs:1634).
//
// One CTA owns 112 weight columns for up to 512 tokens (four 128-token slabs, one TMEM
// accumulator of 112 columns each), so every weight is read and dequantized exactly once per
// 512 tokens and N = 14336 gives 128 CTAs: a single wave on 148 SMs.  K advances 64 per stage.
//   warp 0      TMA producer: one 128B-swizzled box [128 tokens x 64 k] of bf16 activations per
//               slab and stage (cp.async.bulk.tensor.2d, no multicast), completing on full_a.
//   warps 2-9   dequantizers: two threads per weight column n0+j, each converting one of the stage's
//               two 32-k blocks.  Every second stage a thread reads the column's next 4 blocks (Q8: 144 contiguous bytes, Q4: 16 B of headers + 64 B of
//               nibbles, all 16-byte aligned); per stage it forms w = code*scale(+min) in f32 for 64
//               k, splits it into hi = bf16(w), lo = bf16(w - hi)  (16 significant bits: a single
//               bf16 operand would cost ~1e-3 relative error, the target is 1e-4) and stores both
//               as K-major 128B-swizzled operand tiles; fence.proxy.async, then arrives on full_b.
//   warp 1      MMA issuer: per stage and slab 4 x (A.hi + A.lo) tcgen05.mma.kind::f16
//               (M=128, N=112, K=16) into the slab's TMEM accumulator, tcgen05.commit -> empty
//               (frees the stage); after the last stage tcgen05.commit -> acc_full.
//   warps 2-9   epilogue: tcgen05.ld 32 lanes x 16 columns at a time, + addend, store f32.
//
// Every mbarrier wait is bounded; when one runs out the CTA raises a device-wide error word
// (mgq_device_status reports MGQ_ERR_TIMEOUT), drains, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "mgq_internal.h"

namespace mgq {
namespace {

constexpr int TM = 128, TN = 112, TK = 64;         // slab rows, weight columns per CTA, K per pipeline stage
constexpr int kSlabs = 4;                          // token slabs per CTA (TMEM: 4 x 112 columns)
constexpr int kTcStages = 2;
constexpr uint32_t kSubA = 128 * 128;              // activation sub-tile: 128 rows x 64 bf16 (128 B), 16 KB
constexpr uint32_t kSubB = TN * 128;               // weight sub-tile: 112 rows x 128 B, 14 KB (a 1024-byte multiple)
constexpr uint32_t kStageBytes = kSlabs * kSubA + 2 * kSubB;   // A0..A3 | Bhi | Blo
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kWaitLimit = 1u << 20;          // try_wait calls before a wait gives up (each may sleep for a short hardware quantum)
constexpr int kThreads = 320;                      // TMA warp, MMA warp, 8 dequant/epilogue warps

__device__ unsigned int g_tc_error = 0;

struct TcParams {
    const uint8_t *w;
    const float *addend;
    float *c;
    uint32_t m, k, n, bpc, fmt;
    uint32_t vec;                 // rows of c / addend can be accessed as float4
    unsigned long long num_blocks;
};

struct __align__(8) TcShared {
    unsigned long long full_a[kTcStages], full_b[kTcStages], empty[kTcStages], acc_full;
    uint32_t tmem_base;
    volatile int failed;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role of this CTA already gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, uint32_t parity, TcShared *sh)
{
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (sh->failed) return false;
    }
    sh->failed = 1;
    atomicExch(&g_tc_error, 1u);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// K-major, 128-byte swizzle: rows are 128 B apart, 8-row groups 1024 B apart (SBO), version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset
    d |= (uint64_t)1 << 46;                                // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
    return d;
}
// kind::f16: D f32, A bf16, B bf16, both K-major, N = 112, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(addr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// words[off + 9*blk] for blk in 0..3 with compile-time off: register selects instead of a dynamic index.
__device__ __forceinline__ uint32_t pick4(const uint32_t *words, int off, uint32_t blk)
{
    return blk == 0 ? words[off] : blk == 1 ? words[off + 9] : blk == 2 ? words[off + 18] : words[off + 27];
}

// Splits two f32 weights into packed bf16 (hi, hi) and (lo, lo): hi = rn(w), lo = rn(w - hi).
__device__ __forceinline__ void split_pair(float w0, float w1, uint32_t &hi, uint32_t &lo)
{
    const __nv_bfloat162 h = __floats2bfloat162_rn(w0, w1);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    const float h0 = __uint_as_float(hi << 16), h1 = __uint_as_float(hi & 0xFFFF0000u);
    const __nv_bfloat162 l = __floats2bfloat162_rn(w0 - h0, w1 - h1);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

// Stores 8 consecutive k (one 16-byte chunk) of weight row `row` into a swizzled sub-tile.
__device__ __forceinline__ void store_chunk(uint8_t *sub, uint32_t row, uint32_t chunk, const uint32_t (&v)[4])
{
    uint4 q;
    q.x = v[0]; q.y = v[1]; q.z = v[2]; q.w = v[3];
    *reinterpret_cast<uint4 *>(sub + row * 128u + ((chunk ^ (row & 7u)) << 4)) = q;
}

__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcShared sh;
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t m0 = blockIdx.y * (TM * kSlabs), n0 = blockIdx.x * TN;
    const uint32_t nk = p.k / TK;
    const uint32_t slabs = min((uint32_t)kSlabs, (p.m - m0 + TM - 1) / TM);      // slabs that hold tokens

    if (tid == 0) {
        for (int s = 0; s < kTcStages; s++) {
            mbar_init(&sh.full_a[s], 1);
            mbar_init(&sh.full_b[s], 2 * TN);
            mbar_init(&sh.empty[s], 1);
        }
        mbar_init(&sh.acc_full, 1);
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {            // TMEM: 128 lanes x 512 columns of f32 (4 accumulators of 112 columns)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh.tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ activations by TMA
        if (lane == 0) {
            int armed = -1;
            for (uint32_t kc = 0; kc < nk; kc++) {
                const uint32_t s = kc % kTcStages, ph = (kc / kTcStages) & 1u;
                if (!mbar_wait(&sh.empty[s], ph ^ 1u, &sh)) break;
                uint8_t *st = tiles + s * kStageBytes;
                mbar_arrive_expect_tx(&sh.full_a[s], slabs * kSubA);
                for (uint32_t i = 0; i < slabs; i++)
                    tma_load_2d(st + i * kSubA, &tmap_a, (int)(kc * TK), (int)(m0 + i * TM), &sh.full_a[s]);
                armed = (int)kc;
            }
            if (sh.failed && armed >= 0) {      // let this thread's own copies land before the CTA exits
                const uint32_t s = (uint32_t)armed % kTcStages, ph = ((uint32_t)armed / kTcStages) & 1u;
                for (uint32_t i = 0; i < kWaitLimit && !mbar_try_wait(&sh.full_a[s], ph); i++) { }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issue
        if (lane == 0) {
            bool ok = true;
            for (uint32_t kc = 0; kc < nk && ok; kc++) {
                const uint32_t s = kc % kTcStages, ph = (kc / kTcStages) & 1u;
                ok = mbar_wait(&sh.full_a[s], ph, &sh) && mbar_wait(&sh.full_b[s], ph, &sh);
                if (!ok) break;
                tc_fence_after();
                const uint32_t base = smem_u32(tiles + s * kStageBytes);
                const uint32_t b_hi = base + kSlabs * kSubA, b_lo = b_hi + kSubB;
#pragma unroll
                for (uint32_t j = 0; j < 4; j++) {                        // four K=16 steps inside a 128-byte row
                    const uint64_t dh = umma_desc(b_hi + j * 32u), dl = umma_desc(b_lo + j * 32u);
                    for (uint32_t i = 0; i < slabs; i++) {
                        const uint64_t da = umma_desc(base + i * kSubA + j * 32u);
                        umma_f16(tmem + i * TN, da, dh, (kc | j) != 0 ? 1u : 0u);
                        umma_f16(tmem + i * TN, da, dl, 1u);
                    }
                }
                umma_commit(&sh.empty[s]);                               // stage reusable once these MMAs retire
            }
            if (ok) umma_commit(&sh.acc_full);
        }
    } else {
        // ------------------------------------------------------------ dequantize, then epilogue
        // two threads per weight column: thread (j, hb) converts block hb of each stage's two blocks
        const uint32_t d = tid - 64;
        const uint32_t j = d % TN, hb = d / TN;                          // operand row, block inside the stage
        const uint32_t col = n0 + j;
        const bool owner = d < 2 * TN, live = owner && col < p.n;
        const uint8_t *colq8 = p.w + (unsigned long long)col * p.bpc * 36ull;
        const uint8_t *colhdr = p.w + (unsigned long long)col * p.bpc * 4ull;
        const uint8_t *colnib = p.w + p.num_blocks * 4ull + (unsigned long long)col * p.bpc * 16ull;
        uint4 raw[9], raw_next[9];                                       // this pair of stages and the one after it
        auto fetch = [&](uint32_t pair, uint4 (&dst)[9]) {               // 4 blocks = 128 k = two stages
            if (!live || pair * 2 >= nk) return;
            if (p.fmt == MGQ_FMT_Q8) {
                const uint4 *src = reinterpret_cast<const uint4 *>(colq8 + (size_t)pair * 144);
#pragma unroll
                for (int i = 0; i < 9; i++) dst[i] = __ldg(src + i);
            } else {
                dst[0] = __ldg(reinterpret_cast<const uint4 *>(colhdr + (size_t)pair * 16));
                const uint4 *src = reinterpret_cast<const uint4 *>(colnib + (size_t)pair * 64);
#pragma unroll
                for (int i = 0; i < 4; i++) dst[1 + i] = __ldg(src + i);
            }
        };
        bool ok = true;
        if (owner) {
            fetch(0, raw);
            fetch(1, raw_next);
            for (uint32_t kc = 0; kc < nk; kc++) {
                const uint32_t s = kc % kTcStages, ph = (kc / kTcStages) & 1u;
                if (!mbar_wait(&sh.empty[s], ph ^ 1u, &sh)) { ok = false; break; }
                uint8_t *st = tiles + s * kStageBytes;
                uint8_t *sub_hi = st + kSlabs * kSubA, *sub_lo = sub_hi + kSubB;
                const uint32_t *words = reinterpret_cast<const uint32_t *>(raw);
                const uint32_t half = kc & 1u;                           // which half of the fetched 128 k
                const uint32_t blk = half * 2 + hb;                      // block inside the fetched four (registers: selected, not indexed)
                {
                    const uint32_t b2 = hb;                               // this thread's block of 32 k
#pragma unroll
                    for (uint32_t c8 = 0; c8 < 4; c8++) {                // 8 k at a time = one 16-byte chunk
                        float wv[8];
                        if (!live) {
#pragma unroll
                            for (int e = 0; e < 8; e++) wv[e] = 0.f;
                        } else if (p.fmt == MGQ_FMT_Q8) {
                            const uint32_t sw = pick4(words, 0, blk);
                            const uint32_t a = pick4(words, 1 + c8 * 2, blk);
                            const uint32_t b = pick4(words, 2 + c8 * 2, blk);
                            const float scale = __half2float(__ushort_as_half((unsigned short)(sw & 0xFFFFu)));
                            // (q + 128) placed in the mantissa of 2^23, then 2^23 + 128 taken off again: exact int8 -> f32
                            // without a conversion instruction (prmt issues at full rate, I2F at a quarter of it)
                            const uint32_t ua = a ^ 0x80808080u, ub = b ^ 0x80808080u;
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                wv[e] = (__uint_as_float(__byte_perm(ua, 0x4B000000u, 0x7650 + e)) - 8388736.f) * scale;
                                wv[4 + e] = (__uint_as_float(__byte_perm(ub, 0x4B000000u, 0x7650 + e)) - 8388736.f) * scale;
                            }
                        } else {
                            const uint32_t h = blk == 0 ? words[0] : blk == 1 ? words[1] : blk == 2 ? words[2] : words[3];
                            const uint32_t q = blk == 0 ? words[4 + c8] : blk == 1 ? words[8 + c8] : blk == 2 ? words[12 + c8] : words[16 + c8];
                            const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&h));
#pragma unroll
                            for (int e = 0; e < 8; e++) wv[e] = fmaf((float)((q >> (4 * e)) & 0xFu), dm.x, dm.y);
                        }
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) split_pair(wv[2 * e], wv[2 * e + 1], hi[e], lo[e]);
                        const uint32_t chunk = b2 * 4 + c8;              // 64 k per stage: 8 chunks
                        store_chunk(sub_hi, j, chunk, hi);
                        store_chunk(sub_lo, j, chunk, lo);
                    }
                }
                if (half) {                                               // a whole fetched pair is consumed: rotate, refill two pairs ahead
#pragma unroll
                    for (int i = 0; i < 9; i++) raw[i] = raw_next[i];
                    fetch(kc / 2 + 2, raw_next);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA's async proxy
                mbar_arrive(&sh.full_b[s]);
            }
        }
        // epilogue: TMEM lane = token row; this warp may touch lanes 32*(warp%4) .. +31
        ok = ok && mbar_wait(&sh.acc_full, 0, &sh);
        ok = __all_sync(0xffffffffu, ok);                                // tcgen05.ld is warp-collective
        if (ok) {
            tc_fence_after();
            const uint32_t quad = warp & 3u;
            // warps 2-5 take columns [0,64), warps 6-9 columns [64,112) of every accumulator
            const uint32_t c_begin = warp < 6 ? 0u : 64u, c_end = warp < 6 ? 64u : (uint32_t)TN;
            for (uint32_t i = 0; i < slabs; i++) {
                const uint32_t row = m0 + i * TM + quad * 32 + lane;
#pragma unroll 1
                for (uint32_t c0 = c_begin; c0 < c_end; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem + ((quad * 32u) << 16) + i * TN + c0, r);
                    if (row < p.m) {
                        const size_t o = (size_t)row * p.n + n0 + c0;
#pragma unroll
                        for (int e = 0; e < 16; e += 4) {
                            if (p.vec && n0 + c0 + e + 3 < p.n) {
                                float4 v = make_float4(__uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
                                if (p.addend) {
                                    const float4 a = *reinterpret_cast<const float4 *>(p.addend + o + e);
                                    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                                }
                                *reinterpret_cast<float4 *>(p.c + o + e) = v;
                            } else {
#pragma unroll
                                for (int t = 0; t < 4; t++)
                                    if (n0 + c0 + e + t < p.n) {
                                        const float v = __uint_as_float(r[e + t]);
                                        p.c[o + e + t] = p.addend ? v + p.addend[o + e + t] : v;
                                    }
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_fn(EncodeTiledFn &out)
{
    static std::mutex mu;
    static EncodeTiledFn cached = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        MGQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !fn) return fail(MGQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        cached = reinterpret_cast<EncodeTiledFn>(fn);
    }
    out = cached;
    return MGQ_OK;
}

}  // namespace

bool gemm_tc_eligible(int a_dtype, uint32_t m, uint32_t k, uint32_t n, const void *a)
{
    (void)n;
    return a_dtype == MGQ_A_BF16 && m >= 64 && k % 128 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0;
}

int launch_gemm_tc(int fmt, const void *a, const void *w, const float *addend, float *c,
                   uint32_t m, uint32_t k, uint32_t n, void *stream_v)
{
    EncodeTiledFn encode = nullptr;
    if (int rc = encode_fn(encode)) return rc;
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {k, m};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)TM};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(MGQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)cr);

    TcParams p{};
    p.w = static_cast<const uint8_t *>(w);
    p.addend = addend;
    p.c = c;
    p.m = m; p.k = k; p.n = n; p.bpc = k / 32; p.fmt = (uint32_t)fmt;
    p.num_blocks = (unsigned long long)p.bpc * n;
    p.vec = (n % 4 == 0) && reinterpret_cast<uintptr_t>(c) % 16 == 0 && reinterpret_cast<uintptr_t>(addend) % 16 == 0;
    const size_t smem = (size_t)kTcStages * kStageBytes + 1024;
    static std::mutex mu;
    static bool opted[64] = {};
    int dev = 0;
    MGQ_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && !opted[dev]) {
            MGQ_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            opted[dev] = true;
        }
    }
    const dim3 grid((n + TN - 1) / TN, (m + TM * kSlabs - 1) / (TM * kSlabs), 1);
    gemm_tc_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream_v)>>>(tmap, p);
    MGQ_CUDA(cudaGetLastError());
    return MGQ_OK;
}

int tc_device_status()
{
    unsigned int err = 0;
    MGQ_CUDA(cudaMemcpyFromSymbol(&err, g_tc_error, sizeof err));
    if (err) {
        const unsigned int zero = 0;
        MGQ_CUDA(cudaMemcpyToSymbol(g_tc_error, &zero, sizeof zero));
        return fail(MGQ_ERR_TIMEOUT, "a bounded wait inside the tensor-core GEMM ran out");
    }
    return MGQ_OK;
}

}  // namespace mgq
