// Persistent plan kernel: a static list of dequantize-fused GEMVs executed by ONE cooperative
// launch, the B200 counterpart of meganeura's Session::step replaying ExecutionPlan.dispatches
// in barrier groups inside one submission (src/runtime.rs:2843-2959, groups 1202-1256).
//
// Why: a decode token is ~150 dependent GEMVs of 10-60 MB.  Launched one by one, each pays a
// dependency-release + activation-fetch + first-round latency of 2-5 us during which HBM idles.
// Here every CTA walks the whole list; the shared-memory weight ring is one continuous pipeline
// across ops (weights are immutable, so the ring keeps prefetching the next op's weights while
// the CTA waits at the barrier of the current one), and dependent ops are separated by a grid
// barrier built from per-op arrival counters in global memory:
//
//   writer side:  y stores -> __threadfence -> __syncthreads -> thread 0: atomicAdd(done[op])
//   reader side:  thread 0 spins (bounded) on ld.acquire(done[wait_for-1]) == gridDim.x
//                 -> __syncthreads -> activations are read with ld.global.cg (L2, never L1)
//
// Every spin has an iteration limit; when it runs out the CTA raises the plan's error word and
// carries on (results are then undefined, nothing hangs), and the host reports
// MGQ_ERR_TIMEOUT.  The CTA that arrives last at the final op zeroes the counters, so a launch
// can be replayed from a CUDA graph with no host-side reset.
//
// The arithmetic per block is the GEMV kernels' (mgq_gemv_device.cuh); the thread count is fixed
// for the whole plan and each op's column grouping is derived from it.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "mgq_gemv_device.cuh"
#include "mgq_internal.h"

struct mgq_plan {
    std::vector<mgq_plan_op> ops;
    void *dev_ops = nullptr;              // PlanOp[count]
    unsigned long long *dev_done = nullptr;   // arrival counters [count] + error word behind them
    unsigned int *dev_error = nullptr;
    uint32_t threads = 0, grid = 0, cols = 0, step_bytes = 0;
    size_t smem = 0;
    int device = 0;
    void *kernel = nullptr;
    uint64_t launches = 0;
};

namespace mgq {
namespace {
using namespace dev;

constexpr int kPlanStages = 4;
constexpr uint32_t kSpinLimit = 1u << 22;          // ~1 s of L2 round trips before a wait gives up

struct PlanOp {
    GemvParams p;
    uint32_t fmt;
    uint32_t wait_for;       // ops [0, wait_for) must be complete before this op reads or writes anything
};

__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Weight-side cursor: which step of which op this thread fetches next.  It runs kPlanStages-1
// steps ahead of the compute side through the same padded sequence (every op is padded to whole
// rounds, so ring slots stay compile-time constants).
struct FetchCursor {
    uint32_t op;
    uint32_t steps_left;        // padded steps of the current op still to issue
    uint32_t fmt;
    uint32_t g_next;            // next group inside this CTA's range
    uint32_t limit;             // Q4: groups in which this thread has a column; Q8: groups of this CTA
    uint32_t stride;            // elements (Q4) or bytes (Q8) between consecutive groups
    uint32_t full, last, last_group;   // Q8: blocks this warp owns per group / in the matrix's final group
    const uint4 *nib;
    const uint32_t *hdr;
    const uint8_t *src;
};

template <int C, int MINB>
__global__ void __launch_bounds__(384, MINB)
plan_kernel(const PlanOp *__restrict__ ops, uint32_t n_ops, uint32_t step_bytes,
            unsigned long long *done, unsigned int *error
#ifdef MGQ_PLAN_TRACE
            , unsigned long long *trace      // [n_ops][gridDim.x][6] globaltimer stamps
#endif
            )
{
#ifdef MGQ_PLAN_TRACE
#define PLAN_STAMP(op_, slot_) do { if (trace && threadIdx.x == 0) trace[((size_t)(op_) * gridDim.x + blockIdx.x) * 6 + (slot_)] = now_ns(); } while (0)
#else
#define PLAN_STAMP(op_, slot_) do { } while (0)
#endif
    constexpr int STAGES = kPlanStages, ROUND = STAGES * C;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t T = blockDim.x, t = threadIdx.x, lane = t & 31u, warp = t >> 5, G = gridDim.x;
    uint8_t *ring = smem;                                                        // [STAGES][step_bytes]
    float *s_red = reinterpret_cast<float *>(smem + (size_t)STAGES * step_bytes);  // [2][ROUND][T]
    // A step's slot is divided into one private area per warp (C*640 B used by Q4, C*1152 B by Q8),
    // so no warp ever writes where another one reads, whatever the formats of neighbouring ops.
    const uint32_t warp_bytes = step_bytes / (T >> 5);

    auto cta_range = [&](const GemvParams &p, uint32_t &g0, uint32_t &g1) {
        g0 = (uint32_t)((unsigned long long)blockIdx.x * p.total_iters / G);
        g1 = (uint32_t)((unsigned long long)(blockIdx.x + 1) * p.total_iters / G);
    };
    auto my_groups = [&](const GemvParams &p, uint32_t g1, uint32_t n_g) {
        const bool has_block = t < p.active;
        const uint32_t csub = t / p.bpc;
        uint32_t my_n = has_block ? n_g : 0u;
        if (has_block && g1 == p.total_iters && n_g > 0 && (p.total_iters - 1) * p.cpi + csub >= p.n) my_n = n_g - 1;
        return my_n;
    };

    // ------------------------------------------------------------------ weight side
    FetchCursor f{};
    f.op = 0xFFFFFFFFu;
    auto fetch_setup = [&]() {                      // advance to the next op in which this CTA has work
        for (;;) {
            f.op++;
            if (f.op >= n_ops) { f.steps_left = 0xFFFFFFFFu; f.fmt = 0; return; }
            const GemvParams p = ops[f.op].p;
            uint32_t g0, g1;
            cta_range(p, g0, g1);
            const uint32_t n_g = g1 - g0;
            if (n_g == 0) continue;
            const uint32_t steps = (n_g + C - 1) / C;
            f.steps_left = (steps + STAGES - 1) / STAGES * STAGES;
            f.fmt = ops[f.op].fmt;
            f.g_next = 0;
            if (f.fmt == MGQ_FMT_Q4) {
                const unsigned long long first = (unsigned long long)g0 * p.active + t;
                f.hdr = reinterpret_cast<const uint32_t *>(p.w) + first;
                f.nib = reinterpret_cast<const uint4 *>(p.w + p.num_blocks * 4) + first;
                f.stride = p.active;
                f.limit = my_groups(p, g1, n_g);
            } else {
                const uint32_t w0 = warp * 32u;
                f.full = p.active > w0 ? min(32u, p.active - w0) : 0u;
                const uint32_t last_live = (p.n - (p.total_iters - 1) * p.cpi) * p.bpc;
                f.last = last_live > w0 ? min(32u, last_live - w0) : 0u;
                f.last_group = g1 == p.total_iters ? n_g - 1 : 0xFFFFFFFFu;
                f.src = p.w + ((unsigned long long)g0 * p.active + w0) * 36ull + 16u * lane;
                f.stride = p.active * 36u;
                f.limit = n_g;
            }
            return;
        }
    };
    auto fetch_step = [&](int slot) {
        if (f.steps_left == 0) fetch_setup();
        uint8_t *base = ring + (size_t)slot * step_bytes;
        if (f.fmt == MGQ_FMT_Q4) {
            uint8_t *area = base + (size_t)warp * warp_bytes;          // only this warp touches its area
            uint4 *s_nib = reinterpret_cast<uint4 *>(area) + lane;
            uint32_t *s_hdr = reinterpret_cast<uint32_t *>(area + C * 512) + lane;
#pragma unroll
            for (int j = 0; j < C; j++) {
                if (f.g_next + j < f.limit) {
                    cp_async16(s_nib + j * 32, f.nib);
                    cp_async4(s_hdr + j * 32, f.hdr);
                }
                f.nib += f.stride;
                f.hdr += f.stride;
            }
        } else if (f.fmt == MGQ_FMT_Q8) {
            uint8_t *s_w = base + (size_t)warp * warp_bytes + 16u * lane;
#pragma unroll
            for (int j = 0; j < C; j++) {
                const uint32_t gi = f.g_next + j;
                if (gi < f.limit) {
                    const uint32_t cnt = gi == f.last_group ? f.last : f.full;
                    const uint32_t pieces = (cnt * 36u + 15u) >> 4;
                    uint8_t *dst = s_w + j * kQ8WarpStage;
                    if (lane < pieces) cp_async16(dst, f.src);
                    if (lane + 32u < pieces) cp_async16(dst + 512, f.src + 512);
                    if (lane + 64u < pieces) cp_async16(dst + 1024, f.src + 1024);
                }
                f.src += f.stride;
            }
        }
        f.g_next += C;
        if (f.steps_left != 0xFFFFFFFFu) f.steps_left--;
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) fetch_step(s);

    // ------------------------------------------------------------------ compute side
    uint32_t parity = 0;
    for (uint32_t op = 0; op < n_ops; op++) {
        const GemvParams p = ops[op].p;
        const uint32_t fmt = ops[op].fmt, wait_for = ops[op].wait_for;
        uint32_t g0, g1;
        cta_range(p, g0, g1);
        const uint32_t n_g = g1 - g0;
        PLAN_STAMP(op, 0);
        if (n_g > 0) {
            if (wait_for) {
                if (t == 0) {
                    uint32_t spins = 0;
                    while (ld_acquire(done + (wait_for - 1)) < (unsigned long long)G) {
                        if (++spins > kSpinLimit) { atomicExch(error, 1u); break; }
                    }
                }
                __syncthreads();
            }
            PLAN_STAMP(op, 1);
            const uint32_t b = t % p.bpc;
            const uint32_t my_n = my_groups(p, g1, n_g);
            XBlock xb;
            if (fmt == MGQ_FMT_Q4) load_x<1, true>(p.x, b, xb); else load_x<0, true>(p.x, b, xb);
            const ReduceSlot slot = make_slot<ROUND>(p);
            PLAN_STAMP(op, 2);

            // one copy of the round loop per format, so that only one format's block code is hot
            auto run_rounds = [&](auto fmt_tag) {
                constexpr int FMT = decltype(fmt_tag)::value;
                for (uint32_t g = 0; g < n_g; g += ROUND) {
                    float part[1][ROUND];
#pragma unroll
                    for (int u = 0; u < STAGES; u++) {
                        __syncwarp();                   // staging areas are per warp: all lanes left the slot refilled next
                        fetch_step((u + STAGES - 1) % STAGES);
                        cp_async_wait<STAGES - 1>();
                        __syncwarp();
                        const uint8_t *area = ring + (size_t)u * step_bytes + (size_t)warp * warp_bytes;
#pragma unroll
                        for (int j = 0; j < C; j++) {
                            float out = 0.f;
                            if (g + u * C + j < my_n) {
                                if (FMT == MGQ_FMT_Q4) {
                                    const uint4 q = (reinterpret_cast<const uint4 *>(area) + lane)[j * 32];
                                    const uint32_t h = (reinterpret_cast<const uint32_t *>(area + C * 512) + lane)[j * 32];
                                    const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&h));
                                    out = fmaf(dm.x * xb.inv, dot_q4(q, xb), dm.y * xb.sum);
                                } else {
                                    const uint32_t *bp = reinterpret_cast<const uint32_t *>(area + j * kQ8WarpStage + 36u * lane);
                                    const float scale = __half2float(__ushort_as_half((unsigned short)(bp[0] & 0xFFFFu)));
                                    out = scale * xb.inv * dot_q8(bp + 1, xb);
                                }
                            }
                            part[0][u * C + j] = out;
                        }
                    }
                    reduce_store<1, ROUND, true>(p, slot, s_red + (size_t)(parity & 1u) * ROUND * T, part, g0 + g, g1);
                    parity++;
                }
            };
            if (fmt == MGQ_FMT_Q4) run_rounds(std::integral_constant<int, MGQ_FMT_Q4>{});
            else                   run_rounds(std::integral_constant<int, MGQ_FMT_Q8>{});
        }
        // publish this CTA's part of op: results first, then the arrival
        PLAN_STAMP(op, 3);
        __threadfence();
        __syncthreads();
        PLAN_STAMP(op, 4);
        if (t == 0) {
            const unsigned long long prev = atomicAdd(done + op, 1ull);
            if (op == n_ops - 1 && prev == (unsigned long long)G - 1) {
                // every CTA has finished every op and reads no counter any more: rearm for the next launch
                for (uint32_t i = 0; i < n_ops; i++) done[i] = 0ull;
                __threadfence();
            }
        }
    }
    cp_async_wait<0>();
}

int g_plan_cols = 0;
int plan_cols_option() { return g_plan_cols; }

uint32_t columns_for(uint32_t threads, uint32_t bpc)
{
    uint32_t cpi = threads / bpc;
    const uint32_t need = bpc % 4 == 0 ? 1u : (bpc % 2 == 0 ? 2u : 4u);
    return cpi - cpi % need;
}

}  // namespace
}  // namespace mgq

using namespace mgq;

namespace mgq {
int set_plan_option(const char *name, long value)
{
    if (!std::strcmp(name, "plan.columns_per_thread")) {
        if (value != 0 && value != 1 && value != 2 && value != 4) return fail(MGQ_ERR_SHAPE, "%s must be 0, 1, 2 or 4", name);
        g_plan_cols = (int)value;
        return MGQ_OK;
    }
    return fail(MGQ_ERR_NAME, "unknown option: %s", name);
}
}  // namespace mgq

#ifdef MGQ_PLAN_TRACE
static unsigned long long *g_plan_trace = nullptr;
extern "C" void mgq_debug_set_plan_trace(unsigned long long *buf) { g_plan_trace = buf; }
#endif

extern "C" {

int mgq_plan_create(const mgq_plan_op *ops, size_t count, mgq_plan **out)
{
    if (!ops || !out) return fail(MGQ_ERR_NULL, "null argument");
    *out = nullptr;
    if (count == 0 || count > 65535) return fail(MGQ_ERR_SHAPE, "a plan holds 1..65535 ops, got %zu", count);
    const uint32_t threads = 384;
    bool any_q8 = false;
    std::vector<PlanOp> dev_ops(count);
    for (size_t i = 0; i < count; i++) {
        const mgq_plan_op &o = ops[i];
        if (!o.x || !o.w || !o.y) return fail(MGQ_ERR_NULL, "op %zu: null operand pointer", i);
        if (!is_quant(o.fmt)) return fail(MGQ_ERR_FORMAT, "op %zu: weight format %d is not Q4/Q8", i, o.fmt);
        if (o.m != 1) return fail(MGQ_ERR_SHAPE, "op %zu: the plan kernel takes single-row GEMVs (m=%u)", i, o.m);
        if (o.k == 0 || o.n == 0 || o.k % 32 != 0) return fail(MGQ_ERR_SHAPE, "op %zu: bad shape k=%u n=%u", i, o.k, o.n);
        const uint32_t bpc = o.k / 32;
        const unsigned long long nb = (unsigned long long)bpc * o.n;
        if (bpc < 8 || bpc > threads || nb % 4 != 0)
            return fail(MGQ_ERR_SHAPE, "op %zu: K=%u N=%u is outside the plan kernel's range (256 <= K <= %u, K*N/32 %% 4 == 0)",
                        i, o.k, o.n, threads * 32);
        if (reinterpret_cast<uintptr_t>(o.w) % 16 != 0 || reinterpret_cast<uintptr_t>(o.x) % 16 != 0)
            return fail(MGQ_ERR_ALIGN, "op %zu: weights and activations must be 16-byte aligned", i);
        any_q8 |= o.fmt == MGQ_FMT_Q8;
        PlanOp &d = dev_ops[i];
        std::memset(&d, 0, sizeof d);
        d.p.x = o.x; d.p.w = static_cast<const uint8_t *>(o.w); d.p.addend = o.addend; d.p.y = o.y;
        d.p.k = o.k; d.p.n = o.n; d.p.bpc = bpc;
        d.p.cpi = columns_for(threads, bpc);
        d.p.active = d.p.cpi * bpc;
        d.p.total_iters = (o.n + d.p.cpi - 1) / d.p.cpi;
        d.p.num_blocks = nb;
        const uint32_t slots = (uint32_t)(kPlanStages * 4) * d.p.cpi;       // sized for 4 columns per thread: order depends on K only
        d.p.red_shift = 0;
        while (d.p.red_shift < 5 && (slots << (d.p.red_shift + 1)) <= threads && (2u << d.p.red_shift) <= bpc) d.p.red_shift++;
        const uint32_t lanes = 1u << d.p.red_shift;
        d.p.red_chunk = (bpc + lanes - 1) / lanes;
        if (d.p.red_chunk % 4 != 0 && bpc % 4 == 0 && d.p.red_chunk > 4) d.p.red_chunk = (d.p.red_chunk + 3u) & ~3u;
        d.fmt = (uint32_t)o.fmt;
        d.wait_for = o.wait_for > i ? (uint32_t)i : o.wait_for;   // only earlier ops can be waited for
    }
    // columns per thread and step: 4 when the round still leaves a finishing lane per column and the
    // ring fits (Q8 blocks need 36 B per thread and column, Q4 20 B), else 2
    uint32_t max_cpi = 1;
    for (const PlanOp &d : dev_ops) max_cpi = d.p.cpi > max_cpi ? d.p.cpi : max_cpi;
    const uint32_t per_thread = any_q8 ? 36u : 20u;
    // Two CTAs per SM with 2 columns per thread and step by default (CTA-wide barriers of one CTA
    // overlap with the other's work); "plan.columns_per_thread" = 4 selects one wide CTA per SM.
    uint32_t cols = plan_cols_option() == 4 ? 4 : 2;
    auto smem_for = [&](uint32_t c) { return (size_t)kPlanStages * per_thread * threads * c + (size_t)2 * kPlanStages * c * threads * 4; };
    if (cols == 4 && ((uint32_t)(kPlanStages * 4) * max_cpi > threads || smem_for(4) > 200 * 1024)) cols = 2;
    if ((uint32_t)(kPlanStages * 2) * max_cpi > threads && cols == 2) cols = 1;
    if (plan_cols_option() == 1) cols = 1;

    mgq_plan *pl = new mgq_plan();
    pl->ops.assign(ops, ops + count);
    pl->threads = threads;
    pl->cols = cols;
    pl->step_bytes = per_thread * threads * cols;
    pl->smem = smem_for(cols);
    pl->kernel = cols == 4 ? (void *)plan_kernel<4, 1> : cols == 2 ? (void *)plan_kernel<2, 2> : (void *)plan_kernel<1, 2>;
    int rc = cuda_check((int)cudaGetDevice(&pl->device), "cudaGetDevice", __FILE__, __LINE__);
    int sms = 0, occ = 0, optin = 0;
    if (!rc) rc = cuda_check((int)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, pl->device), "attr", __FILE__, __LINE__);
    if (!rc) rc = cuda_check((int)cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, pl->device), "attr", __FILE__, __LINE__);
    if (!rc && pl->smem > (size_t)optin) rc = fail(MGQ_ERR_SHAPE, "plan needs %zu B of shared memory, device allows %d", pl->smem, optin);
    if (!rc) rc = cuda_check((int)cudaFuncSetAttribute(pl->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin), "cudaFuncSetAttribute", __FILE__, __LINE__);
    if (!rc) rc = cuda_check((int)cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, pl->kernel, (int)threads, pl->smem), "occupancy", __FILE__, __LINE__);
    if (!rc && occ < 1) rc = fail(MGQ_ERR_CUDA, "plan kernel does not fit on an SM");
    if (!rc) {
        pl->grid = (uint32_t)sms * (uint32_t)occ;
        rc = cuda_check((int)cudaMalloc(&pl->dev_ops, count * sizeof(PlanOp)), "cudaMalloc", __FILE__, __LINE__);
    }
    if (!rc) rc = cuda_check((int)cudaMemcpy(pl->dev_ops, dev_ops.data(), count * sizeof(PlanOp), cudaMemcpyHostToDevice), "cudaMemcpy", __FILE__, __LINE__);
    if (!rc) rc = cuda_check((int)cudaMalloc(&pl->dev_done, (count + 1) * sizeof(unsigned long long)), "cudaMalloc", __FILE__, __LINE__);
    if (!rc) rc = cuda_check((int)cudaMemset(pl->dev_done, 0, (count + 1) * sizeof(unsigned long long)), "cudaMemset", __FILE__, __LINE__);
    if (rc) { mgq_plan_destroy(pl); return rc; }
    pl->dev_error = reinterpret_cast<unsigned int *>(pl->dev_done + count);
    *out = pl;
    return MGQ_OK;
}

int mgq_plan_launch(mgq_plan *pl, void *stream)
{
    if (!pl) return fail(MGQ_ERR_NULL, "null plan");
    const PlanOp *ops = static_cast<const PlanOp *>(pl->dev_ops);
    uint32_t n_ops = (uint32_t)pl->ops.size(), step_bytes = pl->step_bytes;
    unsigned long long *done = pl->dev_done;
    unsigned int *error = pl->dev_error;
#ifdef MGQ_PLAN_TRACE
    unsigned long long *trace = g_plan_trace;
    void *args[] = {&ops, &n_ops, &step_bytes, &done, &error, &trace};
#else
    void *args[] = {&ops, &n_ops, &step_bytes, &done, &error};
#endif
    MGQ_CUDA(cudaLaunchCooperativeKernel(pl->kernel, dim3(pl->grid), dim3(pl->threads), args, pl->smem,
                                         static_cast<cudaStream_t>(stream)));
    pl->launches++;
    return MGQ_OK;
}

int mgq_plan_check(mgq_plan *pl, void *stream)
{
    if (!pl) return fail(MGQ_ERR_NULL, "null plan");
    unsigned int err = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MGQ_CUDA(cudaMemcpyAsync(&err, pl->dev_error, sizeof err, cudaMemcpyDeviceToHost, s));
    MGQ_CUDA(cudaStreamSynchronize(s));
    if (err) {
        // rearm: a timed-out run may have left counters behind
        MGQ_CUDA(cudaMemsetAsync(pl->dev_done, 0, (pl->ops.size() + 1) * sizeof(unsigned long long), s));
        MGQ_CUDA(cudaStreamSynchronize(s));
        return fail(MGQ_ERR_TIMEOUT, "a grid barrier of the plan kernel ran out of its wait limit");
    }
    return MGQ_OK;
}

int mgq_plan_info(const mgq_plan *pl, uint32_t *grid, uint32_t *threads, uint32_t *columns_per_thread, size_t *smem_bytes)
{
    if (!pl) return fail(MGQ_ERR_NULL, "null plan");
    if (grid) *grid = pl->grid;
    if (threads) *threads = pl->threads;
    if (columns_per_thread) *columns_per_thread = pl->cols;
    if (smem_bytes) *smem_bytes = pl->smem;
    return MGQ_OK;
}

void mgq_plan_destroy(mgq_plan *pl)
{
    if (!pl) return;
    if (pl->dev_ops) cudaFree(pl->dev_ops);
    if (pl->dev_done) cudaFree(pl->dev_done);
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
// mgq_plan_create (it allocates the descriptor table and the barrier counters).
//
// The kernel's scratch (descriptors, one arrival counter per op, the error word) lives in the
// array below, which every GPU that loads this library carries until the process exits.  In host
// code the array's name is only a stand-in; the device address comes from cudaGetSymbolAddress,
// looked up once per device while that device is current.
constexpr size_t kStaticMaxOps = MGQ_STATIC_PLAN_MAX_OPS;
constexpr size_t kStaticOpsBytes = kStaticMaxOps * sizeof(mgq::PlanOp);
constexpr size_t kStaticDoneBytes = kStaticMaxOps * sizeof(unsigned long long);
constexpr size_t kStaticScratchBytes = kStaticOpsBytes + kStaticDoneBytes + 256;     // + error word (own 256-byte line)
static __device__ __align__(256) unsigned char g_static_plan_scratch[kStaticScratchBytes];

namespace {

struct StaticSetup {
    bool ready = false;
    unsigned char *scratch = nullptr;     // device address of g_static_plan_scratch on this device
    int sms = 0, optin = 0;
    int occ[3] = {0, 0, 0};               // resident CTAs per SM for the 1-, 2- and 4-column kernels
};

// One-time, allocation-free preparation for the current device: symbol address, SM count, and the
// shared-memory opt-in of the three kernel variants.
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
        MGQ_CUDA(cudaFuncSetAttribute(mgq::plan_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, st.optin));
        MGQ_CUDA(cudaFuncSetAttribute(mgq::plan_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, st.optin));
        MGQ_CUDA(cudaFuncSetAttribute(mgq::plan_kernel<4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, st.optin));
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
    const uint32_t threads = 384;
    static thread_local PlanOp host_ops[kStaticMaxOps];      // fixed host staging, no heap
    bool any_q8 = false;
    uint32_t max_cpi = 1;
    for (size_t i = 0; i < count; i++) {
        const mgq_plan_op &o = ops[i];
        if (!o.x || !o.w || !o.y) return fail(MGQ_ERR_NULL, "op %zu: null operand pointer", i);
        if (!is_quant(o.fmt)) return fail(MGQ_ERR_FORMAT, "op %zu: weight format %d is not Q4/Q8", i, o.fmt);
        if (o.m != 1) return fail(MGQ_ERR_SHAPE, "op %zu: single-row GEMVs only (m=%u)", i, o.m);
        if (o.k == 0 || o.n == 0 || o.k % 32 != 0) return fail(MGQ_ERR_SHAPE, "op %zu: bad shape k=%u n=%u", i, o.k, o.n);
        const uint32_t bpc = o.k / 32;
        const unsigned long long nb = (unsigned long long)bpc * o.n;
        if (bpc < 8 || bpc > threads || nb % 4 != 0)
            return fail(MGQ_ERR_SHAPE, "op %zu: K=%u N=%u is outside the plan kernel's range (256 <= K <= %u, K*N/32 %% 4 == 0)",
                        i, o.k, o.n, threads * 32);
        if (reinterpret_cast<uintptr_t>(o.w) % 16 != 0 || reinterpret_cast<uintptr_t>(o.x) % 16 != 0)
            return fail(MGQ_ERR_ALIGN, "op %zu: weights and activations must be 16-byte aligned", i);
        any_q8 |= o.fmt == MGQ_FMT_Q8;
        PlanOp &d = host_ops[i];
        std::memset(&d, 0, sizeof d);
        d.p.x = o.x; d.p.w = static_cast<const uint8_t *>(o.w); d.p.addend = o.addend; d.p.y = o.y;
        d.p.k = o.k; d.p.n = o.n; d.p.bpc = bpc;
        d.p.cpi = columns_for(threads, bpc);
        d.p.active = d.p.cpi * bpc;
        d.p.total_iters = (o.n + d.p.cpi - 1) / d.p.cpi;
        d.p.num_blocks = nb;
        const uint32_t slots = (uint32_t)(kPlanStages * 4) * d.p.cpi;
        d.p.red_shift = 0;
        while (d.p.red_shift < 5 && (slots << (d.p.red_shift + 1)) <= threads && (2u << d.p.red_shift) <= bpc) d.p.red_shift++;
        const uint32_t lanes = 1u << d.p.red_shift;
        d.p.red_chunk = (bpc + lanes - 1) / lanes;
        if (d.p.red_chunk % 4 != 0 && bpc % 4 == 0 && d.p.red_chunk > 4) d.p.red_chunk = (d.p.red_chunk + 3u) & ~3u;
        d.fmt = (uint32_t)o.fmt;
        d.wait_for = o.wait_for > i ? (uint32_t)i : o.wait_for;
        max_cpi = d.p.cpi > max_cpi ? d.p.cpi : max_cpi;
    }
    StaticSetup *st = nullptr;
    if (int rc = static_setup(st)) return rc;

    // same kernel choice as mgq_plan_create's default: 2 columns per thread, 1 when a round would not fit
    const uint32_t per_thread = any_q8 ? 36u : 20u;
    const uint32_t cols = (uint32_t)(kPlanStages * 2) * max_cpi > threads ? 1u : 2u;
    void *kernel = cols == 2 ? (void *)plan_kernel<2, 2> : (void *)plan_kernel<1, 2>;
    const size_t smem = (size_t)kPlanStages * per_thread * threads * cols + (size_t)2 * kPlanStages * cols * threads * 4;
    if (smem > (size_t)st->optin) return fail(MGQ_ERR_SHAPE, "plan needs %zu B of shared memory, device allows %d", smem, st->optin);
    int &occ = st->occ[cols == 2 ? 1 : 0];
    if (occ == 0) MGQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, (int)threads, smem));
    if (occ < 1) return fail(MGQ_ERR_CUDA, "plan kernel does not fit on an SM");
    const uint32_t grid = (uint32_t)st->sms * (uint32_t)occ;

    // The array still holds the previous call's descriptors, counters and error word: overwrite the
    // first, zero the other two.  All of it is ordered on `stream` before the kernel.
    unsigned char *d_ops = st->scratch, *d_done = st->scratch + kStaticOpsBytes, *d_err = d_done + kStaticDoneBytes;
    MGQ_CUDA(cudaMemcpyAsync(d_ops, host_ops, count * sizeof(PlanOp), cudaMemcpyHostToDevice, stream));
    MGQ_CUDA(cudaMemsetAsync(d_done, 0, kStaticDoneBytes + 256, stream));
    const PlanOp *k_ops = reinterpret_cast<const PlanOp *>(d_ops);
    uint32_t n_ops = (uint32_t)count, step_bytes = per_thread * threads * cols;
    unsigned long long *k_done = reinterpret_cast<unsigned long long *>(d_done);
    unsigned int *k_err = reinterpret_cast<unsigned int *>(d_err);
#ifdef MGQ_PLAN_TRACE
    unsigned long long *trace = nullptr;
    void *args[] = {&k_ops, &n_ops, &step_bytes, &k_done, &k_err, &trace};
#else
    void *args[] = {&k_ops, &n_ops, &step_bytes, &k_done, &k_err};
#endif
    MGQ_CUDA(cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(threads), args, smem, stream));
    unsigned int err = 0;
    MGQ_CUDA(cudaMemcpyAsync(&err, d_err, sizeof err, cudaMemcpyDeviceToHost, stream));
    MGQ_CUDA(cudaStreamSynchronize(stream));
    if (err) return fail(MGQ_ERR_TIMEOUT, "a grid barrier of the plan kernel ran out of its wait limit");
    return MGQ_OK;
}
