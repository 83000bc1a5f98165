// Persistent plan kernel: a static list of dequantize-fused GEMVs executed by ONE cooperative
// launch, the B200 counterpart of meganeura's Session::step replaying ExecutionPlan.dispatches
// in barrier groups inside one submission (src/runtime.rs:2843-2959, groups 1202-1256).
//
// Why: a decode token is ~150 dependent GEMVs of 10-60 MB.  Launched one by one, each pays a
// dependency-release + activation-fetch + first-round latency during which HBM idles.  Here one
// CTA per SM walks the whole list, split into two roles:
//
//   * producer (one elected thread): streams this CTA's share of every op's packed weights into a
//     shared-memory ring with 1-D bulk copies (cp.async.bulk, completion counted on an mbarrier per
//     slot).  Weights are immutable, so the producer does not wait for any dependency: it runs
//     ahead across op boundaries until the ring is full, which keeps HBM streaming while the
//     consumers wait for the previous op's results.
//   * consumers (TC threads): thread t owns block-in-column b = t % bpc of column t / bpc of each
//     pass, holds that block's activations in registers as byte planes (dp4a block dot products,
//     mgq_gemv_device.cuh), takes tiles out of the ring, and finishes column sums through shared
//     memory and warp shuffles in an order that depends only on K.
//
// Dependencies between ops are data flow, not grid barriers.  An op publishes its leading columns
// as 8-byte {value, stamp} elements (stamp = token index + 1, one 64-bit store per element, so a
// reader that sees the stamp has the value and no fence is needed) into a vector that the consuming
// op polls: first two pieces of the block it needs (cheap), then the whole block, re-read until
// every stamp matches.  The same vector may live in every peer GPU's memory (mgq_exchange_push),
// which makes the column-sharded multi-GPU step the same code: remote data always lands in the
// consumer GPU's own memory.  Ops whose activations are an arbitrary plain vector use a per-op
// arrival counter instead (release: stores, __threadfence, atomicAdd; acquire: ld.acquire poll).
//
// Every wait (mbarrier, stamp, counter) has a deadline read from %globaltimer.  When one runs out
// the CTA raises the plan's error word and an abort flag that makes all later waits of the CTA fall
// through at once: the launch finishes with undefined results, nothing hangs, bulk copies still in
// flight are waited for, and the host reports MGQ_ERR_TIMEOUT.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "mgq_gemv_device.cuh"
#include "mgq_internal.h"

namespace mgq {
namespace {
using namespace dev;

constexpr uint32_t kConsumers = 768;           // consumer threads per CTA (the producer warp comes on top)
constexpr uint32_t kConsumerWarps = kConsumers / 32;
constexpr uint32_t kMaxOps = MGQ_PLAN_MAX_OPS;  // every op descriptor of a plan is kept in shared memory
constexpr uint32_t kStageWords = 32 * 33;      // per leader warp: 32 blocks x 32 activations, rows padded to 33 words
constexpr uint32_t kMaxSlots = 16;             // 2 groups of at most 8 slots
constexpr uint32_t kHeadBytes = 512;           // ring barriers (256 B), abort flag, two destination tables of kMaxPeers pointers (at 384)
constexpr uint32_t kMaxBpc = 384;              // K <= 12288: the prepared activations of one op must fit their shared-memory stage

struct ChainOp {                               // 128 bytes
    const uint8_t *w;
    const float *x;                            // plain activations (when xs is null)
    const unsigned long long *xs;              // k {value, stamp} elements this op consumes, or null
    const float *addend;
    float *y;
    unsigned long long *const *pub_tab;        // [pub_world] in global memory: rank p's gathered vector
    unsigned long long num_blocks;
    uint32_t k, n, bpc, fmt;
    uint32_t lanes;                            // columns per pass
    uint32_t active;                           // lanes * bpc threads carry a block
    uint32_t col_align;                        // CTA column ranges start on multiples of this (16-byte aligned copies)
    uint32_t hdr_off;                          // Q4: byte offset of the headers inside a ring slot
    uint32_t wait_for;                         // plain activations: ops [0, wait_for) must have arrived (0: none)
    uint32_t arrive;                           // 1: CTAs count themselves in done[op] when they finish the op
    uint32_t red_shift, red_chunk;
    uint32_t pub_cols, pub_world, pub_rank;    // leading columns published as {value, stamp}, to how many ranks, as which rank
    uint32_t units;                            // n / col_align: what the CTAs divide among themselves
    uint32_t group_sync;                       // 1: a column's bpc threads are whole warps and reduce behind a barrier of their own
    uint32_t pad[1];
};
static_assert(sizeof(ChainOp) == 128, "ChainOp is copied in 16-byte pieces");

struct ChainArgs {
    const ChainOp *ops;
    uint32_t n_ops;
    uint32_t slot_bytes;
    uint32_t xchg_bytes;
    unsigned long long *epoch;                 // token index; the CTA that finishes last adds one
    unsigned long long *done;                  // [n_ops] arrival counters (monotonic: G per token)
    unsigned int *error;
    unsigned int *finish;                      // CTAs that have finished the launch (returns to zero)
    const unsigned long long *final_vec;       // gathered vector whose stamps must all be in before the token ends, or null
    uint32_t final_len;
    unsigned long long deadline_ns;
};

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// The CTA's abort flag sits at a fixed place in dynamic shared memory (behind the ring barriers), so
// no function needs a pointer to it.
__device__ __forceinline__ volatile uint32_t *abort_flag_ptr()
{
    extern __shared__ __align__(128) uint8_t dyn_smem[];
    return reinterpret_cast<volatile uint32_t *>(dyn_smem + 2 * kMaxSlots * 8);
}

// Bounded waiting: expired() is called once per failed try; it looks at the abort flag and the
// clock every 32nd time.
struct Waiter {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    __device__ __forceinline__ bool expired(const ChainArgs &a)
    {
        volatile uint32_t *abort_flag = abort_flag_ptr();
        if ((++spins & 31u) != 0) return false;
        if (*abort_flag) return true;
        const unsigned long long now = global_ns();
        if (t0 == 0) { t0 = now; return false; }
        if (now - t0 <= a.deadline_ns) return false;
        *abort_flag = 1u;
        atomicExch(a.error, 1u);
        return true;
    }
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// 1-D bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// The common case (the phase has completed, or completes within try_wait's own suspend time) is two
// instructions; the bounded spin with its clock reads stays out of line so that it costs the callers
// neither registers nor instruction-cache space.
__device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, const ChainArgs &a)
{
    Waiter w;
    while (!mbar_try(bar, parity))
        if (w.expired(a)) break;
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, const ChainArgs &a)
{
    if (!mbar_try(bar, parity)) mbar_wait_slow(bar, parity, a);
}
// Arrival by lane 0 only, as one predicated instruction (no branch).
__device__ __forceinline__ void mbar_arrive_lane0(uint32_t bar, uint32_t lane)
{
    asm volatile("{\n .reg .pred p;\n setp.eq.u32 p, %1, 0;\n @p mbarrier.arrive.shared::cta.b64 _, [%0];\n}\n"
                 ::"r"(bar), "r"(lane) : "memory");
}
// Shared-memory loads by 32-bit shared address; volatile so that they stay between the barrier wait
// before them and the arrival after them.
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void consumer_sync(uint32_t threads)
{
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}
// Barrier 1 is all consumers; barriers 2..15 are the threads that share one column of every pass.
__device__ __forceinline__ void named_sync(uint32_t id, uint32_t threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ ulonglong2 ld_pair2(const ulonglong2 *p)
{
    ulonglong2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_elem(unsigned long long *p, float value, uint32_t stamp)
{
    const unsigned long long v = (unsigned long long)__float_as_uint(value) | ((unsigned long long)stamp << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// This CTA's share of an op: a contiguous column range, cut into passes of `lanes` columns; a ring
// tile holds one pass.  Producer and consumers derive it from the same numbers.
struct Share {
    uint32_t c0, ncols, passes;
};
__device__ __forceinline__ Share share_of(const ChainOp &o)
{
    // units * gridDim.x < 2^32 (checked when the plan is built): plain 32-bit divisions
    const uint32_t units = o.units;
    const uint32_t u0 = blockIdx.x * units / gridDim.x;
    const uint32_t u1 = (blockIdx.x + 1u) * units / gridDim.x;
    Share s;
    s.c0 = u0 * o.col_align;
    s.ncols = (u1 - u0) * o.col_align;
    s.passes = (s.ncols + o.lanes - 1) / o.lanes;
    return s;
}

__device__ __forceinline__ void wait_counter(const ChainOp &o, unsigned long long target, const ChainArgs &a)
{
    if (!o.wait_for) return;
    Waiter w;
    while (ld_acquire_u64(a.done + (o.wait_for - 1)) < target)
        if (w.expired(a)) break;
}

// One warp fetches the activations of its blocks [b0, b0 + nb), nb <= 32, together: consecutive lanes
// read consecutive 16-byte pieces (whole 128-byte lines per instruction instead of one line per lane),
// the values go through a shared-memory stage (rows of 33 words, free of bank conflicts both ways)
// and lane l leaves with the 32 activations of block b0 + l.  Stamped vectors are first polled at the
// first and last piece of each block (polling all of them from every CTA loads the L2 enough to
// slow the producers down), then fetched until every stamp matches.
__device__ __forceinline__ void warp_fetch_x(const ChainOp &o, uint32_t b0, uint32_t nb, uint32_t stamp, unsigned long long target,
                                             const ChainArgs &a, uint32_t *stage, float (&v)[32])
{
    const uint32_t lane = threadIdx.x & 31u;
    if (o.xs) {
        const ulonglong2 *src = reinterpret_cast<const ulonglong2 *>(o.xs + 32u * b0);     // 16 pieces of two elements per block
        Waiter w;
        for (;;) {
            uint32_t ok = 1;
            if (lane < nb) {
                const ulonglong2 p = ld_pair2(src + 16u * lane), q = ld_pair2(src + 16u * lane + 15u);
                ok = ((uint32_t)(p.x >> 32) == stamp) & ((uint32_t)(p.y >> 32) == stamp) & ((uint32_t)(q.x >> 32) == stamp) &
                     ((uint32_t)(q.y >> 32) == stamp);
            }
            if (__all_sync(0xffffffffu, ok)) break;
            if (__any_sync(0xffffffffu, w.expired(a))) break;
        }
        const uint32_t pieces = nb * 16u;
        for (;;) {
            uint32_t ok = 1;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t p = (uint32_t)j * 32u + lane;
                if (p < pieces) {
                    const ulonglong2 e = ld_pair2(src + p);
                    ok &= ((uint32_t)(e.x >> 32) == stamp) & ((uint32_t)(e.y >> 32) == stamp);
                    uint32_t *dst = stage + (p >> 4) * 33u + 2u * (p & 15u);
                    dst[0] = (uint32_t)e.x;
                    dst[1] = (uint32_t)e.y;
                }
            }
            if (__all_sync(0xffffffffu, ok)) break;
            if (__any_sync(0xffffffffu, w.expired(a))) break;
        }
    } else {
        if (lane == 0) wait_counter(o, target, a);
        __syncwarp();
        const float4 *src = reinterpret_cast<const float4 *>(o.x + 32u * b0);              // 8 pieces of four values per block
        const uint32_t pieces = nb * 8u;
        float4 e[8];                                 // all eight loads in flight before the first is used
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t p = (uint32_t)j * 32u + lane;
            e[j] = __ldcg(src + (p < pieces ? p : 0u));
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t p = (uint32_t)j * 32u + lane;
            if (p < pieces) {
                uint32_t *dst = stage + (p >> 3) * 33u + 4u * (p & 7u);
                dst[0] = __float_as_uint(e[j].x); dst[1] = __float_as_uint(e[j].y); dst[2] = __float_as_uint(e[j].z); dst[3] = __float_as_uint(e[j].w);
            }
        }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(stage[(lane < nb ? lane : 0u) * 33u + i]);
    __syncwarp();                                   // the stage may be overwritten (prepared planes go to the same place)
}

// Ring layout.  A round is R passes (R tiles) followed by one column reduction; the ring has two
// groups of R slots and round r (counted over all ops) uses group r & 1, its p-th pass slot
// R * (r & 1) + p, for the (r >> 1)-th time.  An op's last round may hold fewer than R passes: the
// slots it does not use are simply skipped that time.  So a slot's index and barrier parity follow
// from the round counter alone -- neither side keeps ring state or computes a wrap -- and every
// address inside a round is the round's base plus a compile-time multiple of the slot size.

// The producer: one thread streams this CTA's share of every op's weights into the ring.  Its own
// function (not inlined) so that its loop state is allocated apart from the consumers' registers.
template <int R>
__device__ __noinline__ void produce(const ChainArgs &a, const ChainOp *s_ops, uint32_t full0, uint32_t ring0)
{
    const uint32_t empty0 = full0 + 2u * R * 8u;
    uint32_t round = 0;
    for (uint32_t op = 0; op < a.n_ops; op++) {
        const ChainOp &o = s_ops[op];
        const Share sh = share_of(o);
        // per op: where this CTA's range starts and how large a full tile is; per tile only the
        // wait, the copies and a few additions remain (the loop is one thread's latency chain)
        const bool q4 = o.fmt == MGQ_FMT_Q4;
        const uint32_t bpc = o.bpc, hdr_off = o.hdr_off;
        const unsigned long long first = (unsigned long long)sh.c0 * bpc;
        const uint8_t *src_a = q4 ? o.w + o.num_blocks * 4ull + first * 16ull : o.w + first * 36ull;
        const uint8_t *src_h = o.w + first * 4ull;
        uint32_t blocks_left = sh.ncols * bpc;
        const uint32_t tile_blocks = o.lanes * bpc;
        for (uint32_t pass0 = 0; pass0 < sh.passes; pass0 += R, round++) {
            const uint32_t group = (round & 1u) * R, use = round >> 1;
            const uint32_t n = min((uint32_t)R, sh.passes - pass0);
            for (uint32_t p = 0; p < n; p++) {
                const uint32_t slot = group + p;
                if (use) mbar_wait(empty0 + 8u * slot, (use - 1u) & 1u, a);
                const uint32_t blocks = min(tile_blocks, blocks_left);
                blocks_left -= blocks;
                const uint32_t bar = full0 + 8u * slot, dst = ring0 + slot * a.slot_bytes;
                if (q4) {
                    mbar_expect(bar, blocks * 20u);
                    bulk_load(dst, src_a, blocks * 16u, bar);
                    bulk_load(dst + hdr_off, src_h, blocks * 4u, bar);
                    src_a += (size_t)tile_blocks * 16u;
                    src_h += (size_t)tile_blocks * 4u;
                } else {
                    mbar_expect(bar, blocks * 36u);
                    bulk_load(dst, src_a, blocks * 36u, bar);
                    src_a += (size_t)tile_blocks * 36u;
                }
            }
            // slots of the group that this round leaves out: nobody will wait for or release them this
            // time, so their barriers are stepped here to keep every slot's parity equal to use & 1
            for (uint32_t p = n; p < (uint32_t)R; p++) {
                const uint32_t slot = group + p;
                if (use) mbar_wait(empty0 + 8u * slot, (use - 1u) & 1u, a);
                mbar_arrive(full0 + 8u * slot);                       // completes the "full" phase with no bytes
                for (uint32_t w = 0; w < kConsumerWarps; w++) mbar_arrive(empty0 + 8u * slot);
            }
        }
    }
    // Copies still in flight must land before the CTA may exit (the consumers normally wait for
    // every tile themselves; after an abort they may not have).  Every slot's last use has been
    // issued above; wait for the phase each slot is in, with the same deadline.
    if (*abort_flag_ptr() && round) {
        const uint32_t last = round - 1u;
        for (uint32_t s = 0; s < 2u * R; s++) {
            const uint32_t g = s / R;
            if (g > last) continue;                                    // group never used
            const uint32_t r_last = ((last & 1u) == g) ? last : last - 1u;
            const unsigned long long t0 = global_ns();
            while (!mbar_try(full0 + 8u * s, (r_last >> 1) & 1u))
                if (global_ns() - t0 > a.deadline_ns) break;
        }
    }
}

// Once per op, by the first bpc threads a warp at a time: fetch 32 blocks of activations (with the
// dependency wait), turn them into byte planes and leave the planes in the warp's stage for
// everyone.  Not inlined: the raw activations and the conversion's temporaries stay in this
// function's own frame.
__device__ __noinline__ void fetch_prepare_shared(const ChainOp &o, uint32_t w0, uint32_t stamp, unsigned long long target,
                                                  const ChainArgs &a, uint32_t *stage)
{
    const uint32_t lane = threadIdx.x & 31u;
    float v[32];
    XBlock xb;
    warp_fetch_x(o, w0, min(32u, o.bpc - w0), stamp, target, a, stage, v);
    if (o.fmt == MGQ_FMT_Q4) prepare_x<1>(v, xb); else prepare_x<0>(v, xb);
    uint32_t *dst = stage + lane;
#pragma unroll
    for (int i = 0; i < 8; i++) { dst[i * 32] = xb.p0[i]; dst[(8 + i) * 32] = xb.p1[i]; dst[(16 + i) * 32] = xb.p2[i]; }
    dst[24 * 32] = __float_as_uint(xb.inv);
    dst[25 * 32] = __float_as_uint(xb.sum);
}

template <int R>
__global__ void __launch_bounds__(kConsumers + 32, 1) chain_kernel(const __grid_constant__ ChainArgs a)
{
    constexpr uint32_t TC = kConsumers;
    extern __shared__ __align__(128) uint8_t smem[];
    // [barriers, abort flag, destination tables: kHeadBytes][op descriptors][activation stages][reduction 2 x R x TC floats][ring 2 x R slots]
    ChainOp *s_ops = reinterpret_cast<ChainOp *>(smem + kHeadBytes);
    uint32_t *s_xchg = reinterpret_cast<uint32_t *>(smem + kHeadBytes + (size_t)a.n_ops * sizeof(ChainOp));
    float *s_red = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(s_xchg) + a.xchg_bytes);
    const uint32_t t = threadIdx.x, G = gridDim.x;
    const uint32_t full0 = smem_u32(smem), empty0 = full0 + 2u * R * 8u;
    const uint32_t ring0 = smem_u32(s_red) + 2u * R * TC * (uint32_t)sizeof(float);

    if (t == 0) {
        for (uint32_t s = 0; s < 2u * R; s++) {
            mbar_init(full0 + 8u * s, 1u);
            mbar_init(empty0 + 8u * s, kConsumerWarps);
        }
        *abort_flag_ptr() = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.ops);
        uint4 *dst = reinterpret_cast<uint4 *>(s_ops);
        for (uint32_t i = t; i < a.n_ops * (uint32_t)(sizeof(ChainOp) / 16); i += blockDim.x) dst[i] = __ldg(src + i);
    }
    const uint32_t stamp = (uint32_t)*reinterpret_cast<volatile const unsigned long long *>(a.epoch) + 1u;
    __syncthreads();

    if (t >= TC) {
        // ------------------------------------------------------------------ producer
        if (t == TC) produce<R>(a, s_ops, full0, ring0);
        __syncwarp();                               // the other lanes of the producer warp wait here for the elected one
    } else {
        // ------------------------------------------------------------------ consumers
        const uint32_t lane = t & 31u;
        uint32_t round = 0;
        for (uint32_t op = 0; op < a.n_ops; op++) {
            const ChainOp &o = s_ops[op];
            const Share sh = share_of(o);
            if (sh.ncols != 0) {
                // Little is held in registers across the pass loop (72 registers per thread are all that 25 warps
                // leave): the byte planes, two ring offsets, and a few packed words; everything else about the
                // op is read from its descriptor in shared memory where it is needed.
                const uint32_t bpc = o.bpc;
                const bool has_block = t < o.active;
                const bool q4 = o.fmt == MGQ_FMT_Q4;
                const uint32_t my_col = has_block ? t / bpc : 0x40000000u;      // column inside a pass; idle threads: never live

                // the ranks' gathered vectors this op publishes to: pointers into shared memory now (tables of
                // consecutive ops alternate), so that the finishing lanes do not wait for global memory later;
                // the barrier after the activation fetch orders these stores before their readers
                unsigned long long *s_tab = reinterpret_cast<unsigned long long *>(smem + 384) + (op & 1u) * kMaxPeers;
                if (t >= TC - 32u && lane < o.pub_world) s_tab[lane] = __ldg(reinterpret_cast<const unsigned long long *>(o.pub_tab + lane));

                // ---- which column sum this thread finishes after each round (same for every round), worked out
                //      before the activations are waited for and packed into one word:
                //      [0,12) float offset of its partials in the round's staging rows, [12,21) how many, 21: scalar
                //      reads, [22,31) column inside a round, 31: this lane stores the sum
                uint32_t fin;
                const bool group_sync = o.group_sync != 0u;
                {
                    const uint32_t o_lanes = o.lanes, o_shift = o.red_shift, chunk = o.red_chunk;
                    const uint32_t li = t & ((1u << o_shift) - 1u);
                    uint32_t fu, fj;
                    bool valid;
                    if (group_sync) {
                        // the j-th warp of a column's threads finishes that column of the round's j-th pass: it reads
                        // only what its own group wrote, so the group's barrier is all it needs
                        const uint32_t gw = bpc >> 5, w = t >> 5;
                        fj = w / gw;
                        fu = w % gw;
                        valid = fu < (uint32_t)R && fj < o_lanes;
                        if (!valid) fu = fj = 0u;
                    } else {
                        const uint32_t f = t >> o_shift;
                        valid = f < (uint32_t)R * o_lanes;
                        fu = valid ? f / o_lanes : 0u;
                        fj = valid ? f % o_lanes : 0u;
                    }
                    const uint32_t first = li * chunk;
                    const uint32_t cnt = (valid && first < bpc) ? min(chunk, bpc - first) : 0u;
                    const uint32_t scalar = ((bpc % 4u == 0u) && (chunk % 4u == 0u)) ? 0u : 1u;
                    fin = ((fu * TC + fj * bpc + first) & 4095u) | (cnt << 12) | (scalar << 21) | ((fu * o_lanes + fj) << 22) |
                          ((valid && li == 0u) ? 0x80000000u : 0u);
                }

                // the barrier between a round's partial sums and its column sums, as id | threads << 4: the column's
                // own threads where they are whole warps (idle threads then take no part: id 0), else all consumers
                const uint32_t sync = group_sync ? (has_block ? (my_col + 2u) | (bpc << 4) : 0u) : (1u | (TC << 4));

                // ---- activations of this thread's block, as byte planes in registers: the first bpc threads
                //      fetch and prepare (a warp at a time, 32 blocks each), everyone reads the planes
                XBlock xb;
                {
                    const uint32_t w0 = (t >> 5) * 32u;
                    if (w0 < bpc) fetch_prepare_shared(o, w0, stamp, (unsigned long long)G * stamp, a, s_xchg + (t >> 5) * kStageWords);
                    consumer_sync(TC);
                    const uint32_t b = t % bpc;
                    const uint32_t *src = s_xchg + (b >> 5) * kStageWords + (b & 31u);
#pragma unroll
                    for (int i = 0; i < 8; i++) { xb.p0[i] = src[i * 32]; xb.p1[i] = src[(8 + i) * 32]; xb.p2[i] = src[(16 + i) * 32]; }
                    xb.inv = __uint_as_float(src[24 * 32]);
                    xb.sum = __uint_as_float(src[25 * 32]);
                }

                // shared-memory offsets of this thread's block inside a ring slot; threads beyond `active`
                // shadow the last active thread in full rounds (nothing reads what they produce)
                const uint32_t tt = has_block ? t : o.active - 1u;
                const uint32_t off_a = q4 ? tt * 16u : tt * 36u, off_h = o.hdr_off + tt * 4u;
                const uint32_t cpr = (uint32_t)R * o.lanes;                     // columns per round

                for (uint32_t col0 = 0; col0 < sh.ncols; col0 += cpr, round++) {
                    const uint32_t group = (round & 1u) * R, parity = (round >> 1) & 1u;
                    const uint32_t tile0 = ring0 + group * a.slot_bytes, full_g = full0 + 8u * group, empty_g = empty0 + 8u * group;
                    // partial sums go straight to the staging buffer of this round (nothing is held across passes)
                    float *part = s_red + (size_t)(round & 1u) * R * TC + t;
                    if (col0 + cpr <= sh.ncols) {
                        // full round: R whole passes, no predicates.  The warp is converged, so the loads of all its
                        // lanes are one instruction that precedes the elected lane's arrival in program order.
                        if (q4) {
#pragma unroll
                            for (int u = 0; u < R; u++) {
                                mbar_wait(full_g + 8u * u, parity, a);
                                const uint32_t tile = tile0 + (uint32_t)u * a.slot_bytes;
                                const uint4 q = lds128(tile + off_a);
                                const uint32_t h = lds32(tile + off_h);
                                mbar_arrive_lane0(empty_g + 8u * u, lane);
                                const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&h));
                                part[u * TC] = fmaf(dm.x * xb.inv, dot_q4(q, xb), dm.y * xb.sum);
                            }
                        } else {
#pragma unroll
                            for (int u = 0; u < R; u++) {
                                mbar_wait(full_g + 8u * u, parity, a);
                                const uint32_t tile = tile0 + (uint32_t)u * a.slot_bytes + off_a;
                                uint32_t c[9];
#pragma unroll
                                for (int i = 0; i < 9; i++) c[i] = lds32(tile + 4u * i);
                                mbar_arrive_lane0(empty_g + 8u * u, lane);
                                const float scale = __half2float(__ushort_as_half((unsigned short)(c[0] & 0xFFFFu)));
                                part[u * TC] = scale * xb.inv * dot_q8(c + 1, xb);
                            }
                        }
                    } else {
                        // last round of the op: fewer than R passes, or a last pass with fewer columns
                        const uint32_t o_lanes = o.lanes;
#pragma unroll
                        for (int u = 0; u < R; u++) {
                            part[u * TC] = 0.f;
                            const uint32_t first_col = col0 + (uint32_t)u * o_lanes;
                            if (first_col < sh.ncols) {                           // CTA-uniform: the pass exists
                                mbar_wait(full_g + 8u * u, parity, a);
                                const uint32_t tile = tile0 + (uint32_t)u * a.slot_bytes;
                                const bool live = first_col + my_col < sh.ncols;
                                uint4 q = make_uint4(0, 0, 0, 0);
                                uint32_t c[9];
#pragma unroll
                                for (int i = 0; i < 9; i++) c[i] = 0;
                                if (live) {
                                    if (q4) {
                                        q = lds128(tile + off_a);
                                        c[0] = lds32(tile + off_h);
                                    } else {
#pragma unroll
                                        for (int i = 0; i < 9; i++) c[i] = lds32(tile + off_a + 4u * i);
                                    }
                                }
                                __syncwarp();                                     // every lane's data is in registers: hand the slot back
                                mbar_arrive_lane0(empty_g + 8u * u, lane);
                                if (live) {
                                    if (q4) {
                                        const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&c[0]));
                                        part[u * TC] = fmaf(dm.x * xb.inv, dot_q4(q, xb), dm.y * xb.sum);
                                    } else {
                                        const float scale = __half2float(__ushort_as_half((unsigned short)(c[0] & 0xFFFFu)));
                                        part[u * TC] = scale * xb.inv * dot_q8(c + 1, xb);
                                    }
                                }
                            }
                        }
                    }
                    // ---- finish the round's columns
                    if (sync) named_sync(sync & 15u, sync >> 4);
                    const uint32_t rel = col0 + ((fin >> 22) & 511u);                        // column inside this CTA's range
                    const bool store = (fin >> 31) != 0u && rel < sh.ncols;
                    float add = 0.f;
                    if (store && o.addend) add = __ldcg(o.addend + sh.c0 + rel);             // in flight during the sums below
                    float s = 0.f;
                    const float *src = s_red + (size_t)(round & 1u) * R * TC + (fin & 4095u);
                    const uint32_t cnt = (fin >> 12) & 511u;
                    if (!(fin & (1u << 21))) {
                        for (uint32_t j = 0; j < cnt; j += 4) {
                            const float4 q = *reinterpret_cast<const float4 *>(src + j);
                            s += (q.x + q.y) + (q.z + q.w);
                        }
                    } else {
                        for (uint32_t j = 0; j < cnt; j++) s += src[j];
                    }
                    const uint32_t o_shift = o.red_shift;
                    if (o_shift == 5) {                       // a whole warp per column
                        s += __shfl_xor_sync(0xffffffffu, s, 16);
                        s += __shfl_xor_sync(0xffffffffu, s, 8);
                        s += __shfl_xor_sync(0xffffffffu, s, 4);
                        s += __shfl_xor_sync(0xffffffffu, s, 2);
                        s += __shfl_xor_sync(0xffffffffu, s, 1);
                    } else {
                        if (o_shift > 3) s += __shfl_xor_sync(0xffffffffu, s, 8);
                        if (o_shift > 2) s += __shfl_xor_sync(0xffffffffu, s, 4);
                        if (o_shift > 1) s += __shfl_xor_sync(0xffffffffu, s, 2);
                        if (o_shift > 0) s += __shfl_xor_sync(0xffffffffu, s, 1);
                    }
                    if (store) {                           // the descriptor is in shared memory: nothing of it is held in registers
                        const uint32_t col = sh.c0 + rel;
                        const float v = o.addend ? s + add : s;
                        o.y[col] = v;
                        const uint32_t pub_cols = o.pub_cols;
                        // after a timeout nothing is published: peers must run into their own limit rather than
                        // consume results computed from incomplete inputs under a valid stamp
                        if (col < pub_cols && *abort_flag_ptr() == 0u) {
                            const size_t at = (size_t)o.pub_rank * pub_cols + col;
                            const unsigned long long *tab = reinterpret_cast<const unsigned long long *>(smem + 384) + (op & 1u) * kMaxPeers;
                            for (uint32_t q = 0; q < o.pub_world; q++)
                                st_elem(reinterpret_cast<unsigned long long *>(tab[q]) + at, v, stamp);
                        }
                    }
                }
            }
            if (o.arrive) {
                // publish this CTA's part of the op to readers of the plain vector: the barrier orders every
                // consumer's stores before thread 0's fence, which is cumulative, then the arrival
                consumer_sync(TC);
                if (t == 0) {
                    __threadfence();
                    atomicAdd(a.done + op, 1ull);
                }
            }
        }
        // ---- the token ends when the last gathered vector is complete on this GPU
        if (a.final_vec) {
            for (uint32_t i = blockIdx.x * TC + t; i < a.final_len; i += G * TC) {
                Waiter w;
                for (;;) {
                    unsigned long long e;
                    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(e) : "l"(a.final_vec + i) : "memory");
                    if ((uint32_t)(e >> 32) == stamp) break;
                    if (w.expired(a)) break;
                }
            }
        }
    }
    __syncthreads();
    if (t == 0) {
        __threadfence();
        if (atomicAdd(a.finish, 1u) == G - 1u) {
            atomicExch(a.finish, 0u);
            *reinterpret_cast<volatile unsigned long long *>(a.epoch) = *reinterpret_cast<volatile unsigned long long *>(a.epoch) + 1ull;
            __threadfence();
        }
    }
}

// ------------------------------------------------------------------------------- host side

struct PlanTuning {
    int dataflow = 0;           // "plan.dataflow": 1 = on one GPU, too, hand activations from op to op as {value, stamp} vectors
    long deadline_us = 0;       // "plan.deadline_us": limit of every device-side wait of a self-contained plan (0: 20000)
    long peer_deadline_us = 0;  // "plan.peer_deadline_us": the same for plans that wait for other GPUs (0: 2000000)
};
PlanTuning g_plan_tuning;

struct Layout {
    uint32_t tc = 0, round = 0, slot_bytes = 0, xchg_bytes = 0;     // round: passes per round (the ring holds 2 * round slots)
    size_t smem = 0;
};

inline uint32_t gcd_u32(uint32_t a, uint32_t b) { while (b) { const uint32_t r = a % b; a = b; b = r; } return a; }

// Fills the kernel-side fields of one op that depend only on its shape and the consumer count.
int shape_op(ChainOp &d, size_t i, uint32_t tc, uint32_t round)
{
    const uint32_t bpc = d.bpc;
    d.col_align = 4u / gcd_u32(bpc, 4u);
    uint32_t lanes = tc / bpc;
    lanes -= lanes % d.col_align;
    if (lanes == 0 || bpc > kMaxBpc)
        return fail(MGQ_ERR_SHAPE, "op %zu: K=%u is outside the plan kernel's range (256 <= K <= %u)", i, d.k,
                    (tc / d.col_align < kMaxBpc ? tc / d.col_align : kMaxBpc) * 32u);
    d.lanes = lanes;
    d.active = lanes * bpc;
    d.hdr_off = d.active * 16u;
    d.units = d.n / d.col_align;
    if ((unsigned long long)d.units * 1024ull >= (1ull << 32)) return fail(MGQ_ERR_SHAPE, "op %zu: N=%u is too large for the plan kernel", i, d.n);
    // finishing lanes per column: a power of two, at most 32, as many as a round leaves room for;
    // all of it follows from K and the consumer count, so a column's sum does not depend on N
    const uint32_t cols_per_round = round * lanes;
    d.red_shift = 0;
    while (d.red_shift < 5 && (cols_per_round << (d.red_shift + 1)) <= tc && (2u << d.red_shift) <= bpc) d.red_shift++;
    // whole warps per column and at least one of them per pass of a round: columns reduce on their own
    d.group_sync = (bpc % 32u == 0u && bpc / 32u >= round && lanes <= 14u && d.red_shift == 5u) ? 1u : 0u;
    const uint32_t fl = 1u << d.red_shift;
    d.red_chunk = (bpc + fl - 1) / fl;
    if (d.red_chunk % 4 != 0 && bpc % 4 == 0 && d.red_chunk > 4) d.red_chunk = (d.red_chunk + 3u) & ~3u;
    return MGQ_OK;
}

int check_op(const mgq_plan_op &o, size_t i)
{
    if (!o.w || !o.y) return fail(MGQ_ERR_NULL, "op %zu: null operand pointer", i);
    if (!is_quant(o.fmt)) return fail(MGQ_ERR_FORMAT, "op %zu: weight format %d is not Q4/Q8", i, o.fmt);
    if (o.m != 1) return fail(MGQ_ERR_SHAPE, "op %zu: the plan kernel takes single-row GEMVs (m=%u)", i, o.m);
    if (o.k == 0 || o.n == 0 || o.k % 32 != 0) return fail(MGQ_ERR_SHAPE, "op %zu: bad shape k=%u n=%u", i, o.k, o.n);
    const uint32_t bpc = o.k / 32;
    const unsigned long long nb = (unsigned long long)bpc * o.n;
    if (bpc < 8 || nb % 4 != 0)
        return fail(MGQ_ERR_SHAPE, "op %zu: K=%u N=%u is outside the plan kernel's range (K >= 256, K*N/32 %% 4 == 0)", i, o.k, o.n);
    if (reinterpret_cast<uintptr_t>(o.w) % 16 != 0 || reinterpret_cast<uintptr_t>(o.x) % 16 != 0)
        return fail(MGQ_ERR_ALIGN, "op %zu: weights and activations must be 16-byte aligned", i);
    return MGQ_OK;
}

void base_op(ChainOp &d, const mgq_plan_op &o)
{
    std::memset(&d, 0, sizeof d);
    d.w = static_cast<const uint8_t *>(o.w);
    d.x = o.x; d.addend = o.addend; d.y = o.y;
    d.k = o.k; d.n = o.n; d.bpc = o.k / 32; d.fmt = (uint32_t)o.fmt;
    d.num_blocks = (unsigned long long)d.bpc * o.n;
}

// Passes per round for a list of ops: 4 when every op is Q4 (15 KB tiles), 2 when Q8 tiles (27 KB)
// have to fit the ring as well.
uint32_t round_for(const mgq_plan_op *ops, size_t count)
{
    for (size_t i = 0; i < count; i++)
        if (ops[i].fmt == MGQ_FMT_Q8) return 2;
    return 4;
}

// Shared-memory layout for a list of shaped ops.
int layout_for(const ChainOp *ops, size_t count, uint32_t tc, uint32_t round, int optin, Layout &L)
{
    uint32_t slot = 0, xchg = 0;
    for (size_t i = 0; i < count; i++) {
        const ChainOp &d = ops[i];
        const uint32_t tile = d.active * (d.fmt == MGQ_FMT_Q4 ? 20u : 36u);
        slot = tile > slot ? tile : slot;
        const uint32_t need = (d.bpc + 31u) / 32u * kStageWords * 4u;
        xchg = need > xchg ? need : xchg;
    }
    L.tc = tc;
    L.round = round;
    L.slot_bytes = (slot + 127u) & ~127u;
    L.xchg_bytes = (xchg + 127u) & ~127u;
    L.smem = kHeadBytes + count * sizeof(ChainOp) + L.xchg_bytes + (size_t)2 * round * tc * sizeof(float) + (size_t)2 * round * L.slot_bytes;
    if (L.smem > (size_t)optin) return fail(MGQ_ERR_SHAPE, "plan needs %zu B of shared memory, device allows %d", L.smem, optin);
    return MGQ_OK;
}

// A plan whose waits only concern this GPU's own CTAs (all resident at once) can give up after
// milliseconds.  A plan that waits for other GPUs also waits for their host processes, which may
// launch seconds apart, so its limit is long by default.
unsigned long long deadline_ns(bool waits_for_peers)
{
    long us = g_plan_tuning.deadline_us > 0 ? g_plan_tuning.deadline_us : 20000;
    if (waits_for_peers) us = g_plan_tuning.peer_deadline_us > 0 ? g_plan_tuning.peer_deadline_us : 2000000;
    return (unsigned long long)us * 1000ull;
}

void *kernel_for(uint32_t round) { return round == 4 ? (void *)chain_kernel<4> : (void *)chain_kernel<2>; }

struct DeviceFacts { int device = 0, sms = 0, optin = 0; };
int device_facts(DeviceFacts &f)
{
    MGQ_CUDA(cudaGetDevice(&f.device));
    MGQ_CUDA(cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, f.device));
    MGQ_CUDA(cudaDeviceGetAttribute(&f.optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, f.device));
    return MGQ_OK;
}

uint32_t consumer_threads() { return 768u; }

}  // namespace

int set_plan_option(const char *name, long value)
{
    if (!std::strcmp(name, "plan.dataflow")) {
        g_plan_tuning.dataflow = value ? 1 : 0;
    } else if (!std::strcmp(name, "plan.deadline_us")) {
        if (value < 0 || value > 10000000) return fail(MGQ_ERR_SHAPE, "%s out of range", name);
        g_plan_tuning.deadline_us = value;
    } else if (!std::strcmp(name, "plan.peer_deadline_us")) {
        if (value < 0 || value > 600000000) return fail(MGQ_ERR_SHAPE, "%s out of range", name);
        g_plan_tuning.peer_deadline_us = value;
    } else {
        return fail(MGQ_ERR_NAME, "unknown option: %s", name);
    }
    return MGQ_OK;
}

}  // namespace mgq

using namespace mgq;

struct mgq_plan {
    size_t count = 0;
    uint8_t *dev_block = nullptr;             // one allocation: descriptors, push records, counters, state words, gathered vectors
    size_t dev_bytes = 0, state_off = 0, state_bytes = 0;
    ChainArgs args{};
    Layout layout;
    uint32_t grid = 0;
    int device = 0;
    void *kernel = nullptr;
    bool own_state = true;                    // epoch / error words live in dev_block
    uint64_t launches = 0;
};

namespace {

int create_plan(const mgq_plan_op *ops, const mgq_plan_link *links, size_t count, unsigned long long *epoch, unsigned int *error,
                const mgq_exchange_elem *final_vec, uint32_t final_len, mgq_plan **out)
{
    if (!ops || !out) return fail(MGQ_ERR_NULL, "null argument");
    *out = nullptr;
    if (count == 0 || count > kMaxOps)
        return fail(MGQ_ERR_SIZE, "a plan holds 1..%u ops (their descriptors live in shared memory), got %zu; split longer lists over several plans",
                    kMaxOps, count);
    const uint32_t tc = consumer_threads(), round = round_for(ops, count);
    std::vector<ChainOp> host(count);
    std::vector<uint32_t> publish(count, 0);        // columns op j publishes into a vector owned by the plan
    std::vector<unsigned long long> tables(count * kMaxPeers, 0ull);   // per op: the gathered vector of every rank
    std::vector<int> source(count, -1);
    std::vector<size_t> source_off(count, 0);
    for (size_t i = 0; i < count; i++) {
        const mgq_plan_op &o = ops[i];
        if (int rc = check_op(o, i)) return rc;
        const bool linked_x = links && links[i].wait_vec;
        if (!o.x && !linked_x) return fail(MGQ_ERR_NULL, "op %zu: null activation pointer", i);
        ChainOp &d = host[i];
        base_op(d, o);
        if (int rc = shape_op(d, i, tc, round)) return rc;
        d.wait_for = o.wait_for > i ? (uint32_t)i : o.wait_for;
        if (links) {
            if (links[i].push_dev) {
                // the caller's record lives in device memory: read it once, keep its contents in the descriptor
                ExchangePush rec;
                MGQ_CUDA(cudaMemcpy(&rec, links[i].push_dev, sizeof rec, cudaMemcpyDeviceToHost));
                if (rec.world < 1 || rec.world > (uint32_t)kMaxPeers || rec.rank >= rec.world || rec.gather_cols > o.n)
                    return fail(MGQ_ERR_SHAPE, "op %zu: bad exchange record (world=%u rank=%u gather_cols=%u)", i, rec.world, rec.rank, rec.gather_cols);
                d.pub_world = rec.world; d.pub_rank = rec.rank; d.pub_cols = rec.gather_cols;
                for (uint32_t q = 0; q < rec.world; q++) tables[i * kMaxPeers + q] = reinterpret_cast<unsigned long long>(rec.dst[q]);
            }
            d.xs = reinterpret_cast<const unsigned long long *>(links[i].wait_vec);
            if (d.xs) d.wait_for = 0;
            if (reinterpret_cast<uintptr_t>(d.xs) % 16 != 0) return fail(MGQ_ERR_ALIGN, "op %zu: the gathered vector must be 16-byte aligned", i);
        } else if (d.wait_for && g_plan_tuning.dataflow) {
            // activations that are a range of an earlier op's output travel as stamped elements
            for (size_t j = d.wait_for; j-- > 0;) {
                const float *y0 = ops[j].y, *y1 = ops[j].y + ops[j].n;
                if (o.x >= y0 && o.x + o.k <= y1) {
                    source[i] = (int)j;
                    source_off[i] = (size_t)(o.x - y0);
                    const uint32_t need = (uint32_t)source_off[i] + o.k;
                    publish[j] = need > publish[j] ? need : publish[j];
                    break;
                }
            }
        }
    }
    for (size_t i = 0; i < count; i++)
        if (!host[i].xs && source[i] < 0 && host[i].wait_for) host[host[i].wait_for - 1].arrive = 1;

    DeviceFacts df;
    if (int rc = device_facts(df)) return rc;
    Layout L;
    if (int rc = layout_for(host.data(), count, tc, round, df.optin, L)) return rc;

    // device block: [ChainOp x count][destination tables 8 x u64 x count][done u64 x count][epoch u64, error u32, finish u32][vectors]
    size_t off = 0;
    const size_t ops_off = off;      off += count * sizeof(ChainOp);
    const size_t tab_off = off;      off += count * kMaxPeers * sizeof(unsigned long long);
    const size_t done_off = off;     off += count * sizeof(unsigned long long);
    const size_t state_off = off;    off += 64;
    off = (off + 255) & ~(size_t)255;
    const size_t vec_off = off;
    std::vector<size_t> vec_at(count, 0);
    for (size_t j = 0; j < count; j++) {
        if (!publish[j]) continue;
        vec_at[j] = off;
        off += ((size_t)publish[j] * 8 + 255) & ~(size_t)255;
    }
    mgq_plan *pl = new mgq_plan();
    pl->count = count;
    pl->device = df.device;
    pl->layout = L;
    pl->grid = (uint32_t)df.sms;
    pl->kernel = kernel_for(round);
    pl->dev_bytes = off;
    pl->state_off = done_off;
    pl->state_bytes = off - done_off;
    pl->own_state = epoch == nullptr;
    int rc = cuda_check((int)cudaMalloc(&pl->dev_block, off), "cudaMalloc", __FILE__, __LINE__);
    if (!rc) rc = cuda_check((int)cudaMemset(pl->dev_block, 0, off), "cudaMemset", __FILE__, __LINE__);
    if (rc) { delete pl; return rc; }
    (void)vec_off;
    for (size_t j = 0; j < count; j++) {
        if (publish[j]) {
            host[j].pub_world = 1; host[j].pub_rank = 0; host[j].pub_cols = publish[j];
            tables[j * kMaxPeers] = reinterpret_cast<unsigned long long>(pl->dev_block + vec_at[j]);
        }
        host[j].pub_tab = reinterpret_cast<unsigned long long *const *>(pl->dev_block + tab_off) + j * kMaxPeers;
    }
    if (!rc) rc = cuda_check((int)cudaMemcpy(pl->dev_block + tab_off, tables.data(), tables.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice), "cudaMemcpy", __FILE__, __LINE__);
    for (size_t i = 0; i < count; i++)
        if (source[i] >= 0) {
            host[i].xs = reinterpret_cast<const unsigned long long *>(pl->dev_block + vec_at[source[i]]) + source_off[i];
            host[i].wait_for = 0;
        }
    for (size_t i = 0; i < count; i++)
        if (reinterpret_cast<uintptr_t>(host[i].xs) % 16 != 0) {
            // an odd element offset into the producer's vector: fall back to the arrival counter of the op before
            host[i].xs = nullptr;
            host[i].wait_for = ops[i].wait_for > i ? (uint32_t)i : ops[i].wait_for;
            if (host[i].wait_for) host[host[i].wait_for - 1].arrive = 1;
        }
    if (!rc) rc = cuda_check((int)cudaMemcpy(pl->dev_block + ops_off, host.data(), count * sizeof(ChainOp), cudaMemcpyHostToDevice), "cudaMemcpy", __FILE__, __LINE__);
    int occ = 0;
    if (!rc) rc = cuda_check((int)cudaFuncSetAttribute(pl->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, df.optin), "cudaFuncSetAttribute", __FILE__, __LINE__);
    if (!rc) rc = cuda_check((int)cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, pl->kernel, (int)tc + 32, L.smem), "occupancy", __FILE__, __LINE__);
    if (!rc && occ < 1) rc = fail(MGQ_ERR_CUDA, "plan kernel does not fit on an SM");
    if (rc) { mgq_plan_destroy(pl); return rc; }
    ChainArgs &a = pl->args;
    a.ops = reinterpret_cast<const ChainOp *>(pl->dev_block + ops_off);
    a.n_ops = (uint32_t)count;
    a.slot_bytes = L.slot_bytes; a.xchg_bytes = L.xchg_bytes;
    a.done = reinterpret_cast<unsigned long long *>(pl->dev_block + done_off);
    a.epoch = epoch ? epoch : reinterpret_cast<unsigned long long *>(pl->dev_block + state_off);
    a.error = error ? error : reinterpret_cast<unsigned int *>(pl->dev_block + state_off + 8);
    a.finish = reinterpret_cast<unsigned int *>(pl->dev_block + state_off + 12);
    a.final_vec = reinterpret_cast<const unsigned long long *>(final_vec);
    a.final_len = final_vec ? final_len : 0;
    a.deadline_ns = deadline_ns(!pl->own_state);
    *out = pl;
    return MGQ_OK;
}

}  // namespace

extern "C" {

int mgq_plan_create(const mgq_plan_op *ops, size_t count, mgq_plan **out)
{
    return create_plan(ops, nullptr, count, nullptr, nullptr, nullptr, 0, out);
}

int mgq_plan_create_linked(const mgq_plan_op *ops, const mgq_plan_link *links, size_t count, unsigned long long *epoch,
                           unsigned int *error, const mgq_exchange_elem *final_vec, uint32_t final_len, mgq_plan **out)
{
    if (!links || !epoch || !error) return fail(MGQ_ERR_NULL, "null argument");
    return create_plan(ops, links, count, epoch, error, final_vec, final_len, out);
}

int mgq_plan_launch(mgq_plan *pl, void *stream)
{
    if (!pl) return fail(MGQ_ERR_NULL, "null plan");
    pl->args.deadline_ns = deadline_ns(!pl->own_state);
    void *args[] = {&pl->args};
    MGQ_CUDA(cudaLaunchCooperativeKernel(pl->kernel, dim3(pl->grid), dim3(pl->layout.tc + 32), args, pl->layout.smem,
                                         static_cast<cudaStream_t>(stream)));
    pl->launches++;
    return MGQ_OK;
}

int mgq_plan_check(mgq_plan *pl, void *stream)
{
    if (!pl) return fail(MGQ_ERR_NULL, "null plan");
    unsigned int err = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MGQ_CUDA(cudaMemcpyAsync(&err, pl->args.error, sizeof err, cudaMemcpyDeviceToHost, s));
    MGQ_CUDA(cudaStreamSynchronize(s));
    if (err) {
        // rearm: a timed-out launch leaves counters and stamps that no longer match the token index
        MGQ_CUDA(cudaMemsetAsync(pl->args.error, 0, sizeof err, s));
        if (pl->own_state) MGQ_CUDA(cudaMemsetAsync(pl->dev_block + pl->state_off, 0, pl->state_bytes, s));
        MGQ_CUDA(cudaStreamSynchronize(s));
        return fail(MGQ_ERR_TIMEOUT, "a wait inside the plan kernel ran out of its time limit");
    }
    return MGQ_OK;
}

int mgq_plan_info(const mgq_plan *pl, uint32_t *grid, uint32_t *threads, uint32_t *ring_slots, size_t *smem_bytes)
{
    if (!pl) return fail(MGQ_ERR_NULL, "null plan");
    if (grid) *grid = pl->grid;
    if (threads) *threads = pl->layout.tc + 32;
    if (ring_slots) *ring_slots = 2 * pl->layout.round;
    if (smem_bytes) *smem_bytes = pl->layout.smem;
    return MGQ_OK;
}

void mgq_plan_destroy(mgq_plan *pl)
{
    if (!pl) return;
    if (pl->dev_block) cudaFree(pl->dev_block);
    delete pl;
}

}  // extern "C"

// ------------------------------------------------------------------ allocation-free variant
//
// mgq_plan_run_static runs a short list of GEMVs through the same persistent kernel without
// asking CUDA for memory.  It exists for hosts that are not allowed to allocate on their
// execution path: an inference loop that was given a fixed device-memory budget at start-up, or a
// plug-in host that forbids cudaMalloc/cudaFree after initialisation because those calls can
// synchronise the whole device and can fail late when memory is tight.  Such a caller cannot use
// mgq_plan_create (it allocates the descriptor table, the counters and the gathered vectors).
//
// The kernel's scratch (descriptors, one arrival counter per op, the token index, the error word
// and the exit counter) lives in the array below, which every GPU that loads this library carries
// until the process exits.  Dependent ops wait on the arrival counters here; stamped vectors would
// need memory that grows with the ops' widths.  In host code the array's name is only a stand-in;
// the device address comes from cudaGetSymbolAddress, looked up once per device while that device is
// current.
constexpr size_t kStaticMaxOps = MGQ_STATIC_PLAN_MAX_OPS;
constexpr size_t kStaticOpsBytes = kStaticMaxOps * sizeof(mgq::ChainOp);
constexpr size_t kStaticDoneBytes = kStaticMaxOps * sizeof(unsigned long long);
constexpr size_t kStaticScratchBytes = kStaticOpsBytes + kStaticDoneBytes + 256;     // + state words (own 256-byte line)
static __device__ __align__(256) unsigned char g_static_plan_scratch[kStaticScratchBytes];

namespace {

struct StaticSetup {
    bool ready = false;
    unsigned char *scratch = nullptr;     // device address of g_static_plan_scratch on this device
    int sms = 0, optin = 0;
};

// One-time, allocation-free preparation for the current device: symbol address, SM count and the
// shared-memory opt-in of the kernel variants.
int static_setup(StaticSetup *&out)
{
    static std::mutex mu;
    static StaticSetup per_device[64];
    int dev = 0;
    MGQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return mgq::fail(MGQ_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    StaticSetup &st = per_device[dev];
    if (!st.ready) {
        void *ptr = nullptr;
        MGQ_CUDA(cudaGetSymbolAddress(&ptr, g_static_plan_scratch));
        MGQ_CUDA(cudaDeviceGetAttribute(&st.sms, cudaDevAttrMultiProcessorCount, dev));
        MGQ_CUDA(cudaDeviceGetAttribute(&st.optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        MGQ_CUDA(cudaFuncSetAttribute(mgq::chain_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, st.optin));
        MGQ_CUDA(cudaFuncSetAttribute(mgq::chain_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, st.optin));
        st.scratch = static_cast<unsigned char *>(ptr);
        st.ready = true;
    }
    out = &st;
    return MGQ_OK;
}

}  // namespace

extern "C" int mgq_plan_run_static(const mgq_plan_op *ops, size_t count, void *stream_v)
{
    using namespace mgq;
    if (!ops) return fail(MGQ_ERR_NULL, "null op list");
    if (count == 0) return fail(MGQ_ERR_SHAPE, "empty op list");
    if (count > kStaticMaxOps)
        return fail(MGQ_ERR_SIZE, "mgq_plan_run_static takes at most %zu ops (its scratch is a fixed %zu-byte device array), got %zu; "
                                  "use mgq_plan_create for longer lists", kStaticMaxOps, kStaticScratchBytes, count);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    MGQ_CUDA(cudaStreamIsCapturing(stream, &capturing));
    if (capturing != cudaStreamCaptureStatusNone)
        return fail(MGQ_ERR_STATE, "mgq_plan_run_static synchronises its stream and cannot be part of a stream capture");
    const uint32_t tc = consumer_threads(), round = round_for(ops, count);
    static thread_local ChainOp host_ops[kStaticMaxOps];      // fixed host staging, no heap
    for (size_t i = 0; i < count; i++) {
        const mgq_plan_op &o = ops[i];
        if (int rc = check_op(o, i)) return rc;
        if (!o.x) return fail(MGQ_ERR_NULL, "op %zu: null activation pointer", i);
        ChainOp &d = host_ops[i];
        base_op(d, o);
        if (int rc = shape_op(d, i, tc, round)) return rc;
        d.wait_for = o.wait_for > i ? (uint32_t)i : o.wait_for;
    }
    for (size_t i = 0; i < count; i++)
        if (host_ops[i].wait_for) host_ops[host_ops[i].wait_for - 1].arrive = 1;
    StaticSetup *st = nullptr;
    if (int rc = static_setup(st)) return rc;
    Layout L;
    if (int rc = layout_for(host_ops, count, tc, round, st->optin, L)) return rc;      // depends on the list: worked out on every call
    void *kernel = kernel_for(round);
    int occ = 0;
    MGQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, (int)tc + 32, L.smem));
    if (occ < 1) return fail(MGQ_ERR_CUDA, "plan kernel does not fit on an SM");

    // The array still holds the previous call's descriptors, counters and state words: overwrite the
    // first, zero the others.  All of it is ordered on `stream` before the kernel.
    unsigned char *d_ops = st->scratch, *d_done = st->scratch + kStaticOpsBytes, *d_state = d_done + kStaticDoneBytes;
    MGQ_CUDA(cudaMemcpyAsync(d_ops, host_ops, count * sizeof(ChainOp), cudaMemcpyHostToDevice, stream));
    MGQ_CUDA(cudaMemsetAsync(d_done, 0, kStaticDoneBytes + 256, stream));
    ChainArgs a{};
    a.ops = reinterpret_cast<const ChainOp *>(d_ops);
    a.n_ops = (uint32_t)count;
    a.slot_bytes = L.slot_bytes; a.xchg_bytes = L.xchg_bytes;
    a.done = reinterpret_cast<unsigned long long *>(d_done);
    a.epoch = reinterpret_cast<unsigned long long *>(d_state);
    a.error = reinterpret_cast<unsigned int *>(d_state + 8);
    a.finish = reinterpret_cast<unsigned int *>(d_state + 12);
    a.deadline_ns = deadline_ns(false);
    void *args[] = {&a};
    MGQ_CUDA(cudaLaunchCooperativeKernel(kernel, dim3((unsigned)st->sms), dim3(tc + 32), args, L.smem, stream));
    unsigned int err = 0;
    MGQ_CUDA(cudaMemcpyAsync(&err, d_state + 8, sizeof err, cudaMemcpyDeviceToHost, stream));
    MGQ_CUDA(cudaStreamSynchronize(stream));
    if (err) return fail(MGQ_ERR_TIMEOUT, "a wait inside the plan kernel ran out of its time limit");
    return MGQ_OK;
}
