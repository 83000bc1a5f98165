// Small-batch GEMV (3 <= M <= 16 rows) on the integer tensor-core path.
//
// With one or two rows the streaming kernels (mgq_gemv.cu) keep a row's activations in registers;
// more rows do not fit, and re-reading the weights once per pair of rows turns a batch-8 decode
// step into four passes over HBM.  Here the weights are read ONCE for up to 8 rows:
//
//   * Activations are turned into block-fixed-point integers exactly like in the streaming kernels
//     (X = round(x * 2^(21-E)), E from the block's largest magnitude), but as three SIGNED byte
//     digits, X = d2*65536 + d1*256 + d0.  A block of 32 activations of 8 rows is then three
//     32x8 int8 matrices -- the B operand of mma.m16n8k32.
//   * 16 weight columns x one block are a 16x32 matrix of codes (Q4 nibbles 0..15 as u8, Q8 codes as
//     s8) -- the A operand.  One mma per digit gives, exactly, the 16x8 integer dot products of
//     16 columns with 8 rows over that block; the block's f16 scale (and Q4 minimum) is applied in
//     f32 right after, per block, as the format demands.
//   * A warp owns a 16-column tile for the whole K slice, so column sums never leave its
//     registers: no shared-memory reduction and no CTA barrier after the activations are prepared.
//   * Weights stream through per-warp cp.async rings (16 columns x 8 blocks per stage); Q4 nibble
//     rows are fetched from shared memory with ldmatrix, which hands every lane exactly the word
//     the A fragment wants.
//
// This is the legacy mma.sync path on purpose: the work per weight byte is tiny (M <= 8), the kernel
// is bound by HBM and instruction issue, and tcgen05's 128-row tiles have no use for 8 rows.
// K slices of 4096 (the activations of one slice fill shared memory): K > 4096 runs one CTA
// column per slice and a small kernel adds the slices up in a fixed order.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "mgq_gemv_device.cuh"
#include "mgq_internal.h"

namespace mgq {
namespace {

// 16 warps share one copy of the activation planes (104 KB).  Four consecutive warps form a group
// that works on one 16-column tile at a time, each warp on a quarter of the slice's blocks, so
// that even a matrix with few columns keeps every warp of every SM busy; the four partial tiles
// are added in a fixed order through shared memory (two named barriers per tile).  Every warp has
// its own cp.async ring; a stage is 16 columns x 4 blocks: Q4 1024 B of nibbles + 256 B of headers,
// Q8 144 B per column (rows 36 words apart fall into distinct banks).
constexpr int kWarps = 16;
constexpr int kGroupWarps = 4;
constexpr int kGroups = kWarps / kGroupWarps;
constexpr int kSliceBlocks = 128;                 // blocks of K per slice (4096 activations)
constexpr int kTileCols = 16;
constexpr int kStageBlocks = 4;
constexpr int kNibStage = kTileCols * kStageBlocks * 16;      // 1024 B
constexpr int kHdrStage = kTileCols * kStageBlocks * 4;       //  256 B
constexpr int kQ8ColStride = kStageBlocks * 36;               //  144 B
constexpr int kQ8Stage = kTileCols * kQ8ColStride;            // 2304 B

struct MmaParams {
    const float *x;            // [m, k]
    const uint8_t *w;
    const float *addend;       // [m, n] or null (applied by the kernel when there is one slice)
    float *y;                  // [m, n], or partial sums [slices][m][n] when slices > 1
    uint32_t m, k, n, bpc;
    uint32_t tiles;            // ceil(n / 16)
    uint32_t slices;
    unsigned long long num_blocks;
};

__device__ __forceinline__ void cp16(void *smem, const void *gmem)
{
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Shared-memory map (dynamic):
//   planes  [kSliceBlocks][3 digits][32 lanes][2 words]   B fragments, ready to load       98304 B
//   scale   [kSliceBlocks][8 rows][2]  (2^(E-21), sum of the 32 activations)               8192 B
//   red     [kGroups][kGroupWarps][128]  partial tiles of a group                           8192 B
//   rings   [kWarps][stages][stage bytes]
constexpr int kPlaneBytes = kSliceBlocks * 3 * 32 * 8;
constexpr int kScaleBytes = kSliceBlocks * 8 * 2 * 4;
constexpr int kRedBytes = kGroups * kGroupWarps * 128 * 4;

template <int FMT>
__host__ __device__ constexpr int stage_bytes() { return FMT == MGQ_FMT_Q4 ? kNibStage + kHdrStage : kQ8Stage; }
template <int FMT>
__host__ __device__ constexpr int ring_stages() { return FMT == MGQ_FMT_Q4 ? 4 : 3; }

__device__ __forceinline__ void group_barrier(uint32_t grp)
{
    asm volatile("bar.sync %0, %1;\n" ::"r"(1u + grp), "r"(kGroupWarps * 32) : "memory");
}

template <int FMT>
__global__ void __launch_bounds__(kWarps * 32) gemv_mma_kernel(const MmaParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t *s_planes = reinterpret_cast<uint32_t *>(smem);
    float *s_scale = reinterpret_cast<float *>(smem + kPlaneBytes);
    const uint32_t t = threadIdx.x, lane = t & 31u, warp = t >> 5, grp = warp / kGroupWarps, q = warp % kGroupWarps;
    float *s_red = reinterpret_cast<float *>(smem + kPlaneBytes + kScaleBytes) + grp * (kGroupWarps * 128);
    constexpr int STAGES = ring_stages<FMT>();
    uint8_t *ring = smem + kPlaneBytes + kScaleBytes + kRedBytes + warp * (STAGES * stage_bytes<FMT>());
    const uint32_t g = lane >> 2, tq = lane & 3u;

    // this CTA's K slice and column tiles; a group takes every kGroups-th tile of the CTA's range,
    // and warp q of the group the q-th quarter of the slice's stages
    const uint32_t slice = blockIdx.y;
    const uint32_t b_first = slice * kSliceBlocks;
    const uint32_t nb = min((uint32_t)kSliceBlocks, p.bpc - b_first);          // blocks in this slice (a multiple of 8)
    const uint32_t t0 = (uint32_t)((unsigned long long)blockIdx.x * p.tiles / gridDim.x);
    const uint32_t t1 = (uint32_t)((unsigned long long)(blockIdx.x + 1) * p.tiles / gridDim.x);
    const uint32_t my_tiles = t1 > t0 + grp ? (t1 - t0 - grp + kGroups - 1) / kGroups : 0u;
    const uint32_t stages_per_tile = nb / kStageBlocks;
    const uint32_t s_lo = q * stages_per_tile / kGroupWarps, s_hi = (q + 1) * stages_per_tile / kGroupWarps;
    const uint32_t cnt = s_hi - s_lo;                                           // stages of a tile that are this warp's
    const uint32_t items = my_tiles * cnt;

    const uint32_t *hdr_base = reinterpret_cast<const uint32_t *>(p.w);
    const uint8_t *nib_base = p.w + p.num_blocks * 4;

    auto issue = [&](uint32_t item) {
        if (item < items) {
            const uint32_t tile = t0 + grp + (item / cnt) * kGroups, stg = s_lo + item % cnt;
            const uint32_t col0 = tile * kTileCols, blk0 = b_first + stg * kStageBlocks;
            uint8_t *dst = ring + (item % STAGES) * stage_bytes<FMT>();
            if (FMT == MGQ_FMT_Q4) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const uint32_t piece = lane + 32u * j, c = piece >> 2, bb = piece & 3u;
                    const uint32_t col = min(col0 + c, p.n - 1u);
                    cp16(dst + (c * 4u + (bb ^ ((c >> 1) & 3u))) * 16u, nib_base + ((size_t)col * p.bpc + blk0 + bb) * 16u);
                }
                if (lane < 16u) {
                    const uint32_t col = min(col0 + lane, p.n - 1u);
                    cp16(dst + kNibStage + lane * 16u, hdr_base + (size_t)col * p.bpc + blk0);
                }
            } else {
                // 16 columns x 144 contiguous bytes (4 blocks of 36): 9 pieces of 16 B per column
                for (uint32_t i = lane; i < 16u * 9u; i += 32u) {
                    const uint32_t c = i / 9u, piece = i % 9u;
                    const uint32_t col = min(col0 + c, p.n - 1u);
                    cp16(dst + c * kQ8ColStride + piece * 16u, p.w + ((size_t)col * p.bpc + blk0) * 36u + piece * 16u);
                }
            }
        }
        cp_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) issue(s);                               // weights depend on nothing
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // ---- activations of this slice -> signed byte digits in B-fragment order, scale and sum per (block, row)
    for (uint32_t job = t; job < nb * 8u; job += kWarps * 32) {
        const uint32_t bl = job >> 3, row = job & 7u;
        float v[32];
        if (row < p.m) {
            const float4 *xp = reinterpret_cast<const float4 *>(p.x + (size_t)row * p.k + (size_t)(b_first + bl) * 32u);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float4 qv = __ldg(xp + j);
                v[4 * j] = qv.x; v[4 * j + 1] = qv.y; v[4 * j + 2] = qv.z; v[4 * j + 3] = qv.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = 0.f;
        }
        // the streaming kernels' word orders are the fragment's: Q4 word 2c+wd = elements 8c+2e+wd
        // (low / high nibbles of nibble word c), Q8 word 4wd+c = elements 16wd+4c+e
        dev::XBlock xb;
        dev::prepare_x<FMT == MGQ_FMT_Q4 ? 1 : 0, true>(v, xb);
        s_scale[(bl * 8u + row) * 2u] = xb.inv;
        s_scale[(bl * 8u + row) * 2u + 1u] = xb.sum;
#pragma unroll
        for (int c = 0; c < 4; c++) {
#pragma unroll
            for (int wd = 0; wd < 2; wd++) {
                const int wi = FMT == MGQ_FMT_Q4 ? 2 * c + wd : 4 * wd + c;
                const uint32_t at = (row * 4u + c) * 2u + wd;                                      // lane = row*4 + c
                s_planes[(bl * 3u + 0u) * 64u + at] = xb.p0[wi];
                s_planes[(bl * 3u + 1u) * 64u + at] = xb.p1[wi];
                s_planes[(bl * 3u + 2u) * 64u + at] = xb.p2[wi];
            }
        }
    }
    __syncthreads();

    // ---- main loop: a tile at a time; one stage = 16 columns x 4 blocks
    uint32_t item = 0;
    for (uint32_t j = 0; j < my_tiles; j++) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};                // (col g, row 2t), (col g, row 2t+1), (col g+8, row 2t), (col g+8, row 2t+1)
        for (uint32_t stg = s_lo; stg < s_hi; stg++, item++) {
            issue(item + STAGES - 1);
            cp_wait<STAGES - 1>();
            __syncwarp();
            const uint8_t *st = ring + (item % STAGES) * stage_bytes<FMT>();
#pragma unroll
            for (int pair = 0; pair < kStageBlocks / 2; pair++) {
                uint32_t frag[4];                            // Q4: nibble words of (cols 0-7, b), (cols 8-15, b), (cols 0-7, b+1), (cols 8-15, b+1)
                if (FMT == MGQ_FMT_Q4) {
                    const uint32_t mi = lane >> 3, r = lane & 7u;
                    const uint32_t c = (mi & 1u) * 8u + r, bb = 2u * pair + (mi >> 1);
                    const unsigned addr = (unsigned)__cvta_generic_to_shared(st + (c * 4u + (bb ^ ((c >> 1) & 3u))) * 16u);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(frag[0]), "=r"(frag[1]), "=r"(frag[2]), "=r"(frag[3]) : "r"(addr));
                }
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t bb = 2u * pair + h, bl = stg * kStageBlocks + bb;
                    uint32_t a[4];
                    float2 hd0, hd1;                          // (d, m) of columns g and g+8 (Q8: m unused)
                    if (FMT == MGQ_FMT_Q4) {
                        const uint32_t w0 = frag[2 * h], w1 = frag[2 * h + 1];
                        a[0] = w0 & 0x0F0F0F0Fu; a[2] = (w0 >> 4) & 0x0F0F0F0Fu;
                        a[1] = w1 & 0x0F0F0F0Fu; a[3] = (w1 >> 4) & 0x0F0F0F0Fu;
                        const uint32_t *hdr = reinterpret_cast<const uint32_t *>(st + kNibStage);
                        const uint32_t h0 = hdr[g * 4u + bb], h1 = hdr[(g + 8u) * 4u + bb];
                        hd0 = __half22float2(*reinterpret_cast<const __half2 *>(&h0));
                        hd1 = __half22float2(*reinterpret_cast<const __half2 *>(&h1));
                    } else {
                        const uint32_t *r0 = reinterpret_cast<const uint32_t *>(st + g * kQ8ColStride + bb * 36u);
                        const uint32_t *r1 = reinterpret_cast<const uint32_t *>(st + (g + 8u) * kQ8ColStride + bb * 36u);
                        a[0] = r0[1 + tq]; a[2] = r0[5 + tq];
                        a[1] = r1[1 + tq]; a[3] = r1[5 + tq];
                        hd0 = make_float2(__half2float(__ushort_as_half((unsigned short)(r0[0] & 0xFFFFu))), 0.f);
                        hd1 = make_float2(__half2float(__ushort_as_half((unsigned short)(r1[0] & 0xFFFFu))), 0.f);
                    }
                    const uint2 b0 = *reinterpret_cast<const uint2 *>(s_planes + (bl * 3u + 0u) * 64u + lane * 2u);
                    const uint2 b1 = *reinterpret_cast<const uint2 *>(s_planes + (bl * 3u + 1u) * 64u + lane * 2u);
                    const uint2 b2 = *reinterpret_cast<const uint2 *>(s_planes + (bl * 3u + 2u) * 64u + lane * 2u);
                    // (2^(E-21), sum) of batch rows 2t and 2t+1 for this block
                    const float4 sc = *reinterpret_cast<const float4 *>(s_scale + (bl * 8u + 2u * tq) * 2u);
                    float dot[4];
                    if (FMT == MGQ_FMT_Q4) {
                        // |sum of nibble * X| <= 32 * 15 * 2^22 < 2^31: the three digits share ONE integer
                        // accumulator, shifted by a byte between the MMAs (top digit first)
                        int c[4] = {0, 0, 0, 0};
                        mma_u8s8(c, a, b2.x, b2.y);
#pragma unroll
                        for (int i = 0; i < 4; i++) c[i] *= 256;
                        mma_u8s8(c, a, b1.x, b1.y);
#pragma unroll
                        for (int i = 0; i < 4; i++) c[i] *= 256;
                        mma_u8s8(c, a, b0.x, b0.y);
#pragma unroll
                        for (int i = 0; i < 4; i++) dot[i] = (float)c[i];
                    } else {
                        // int8 codes: the two upper digits fit one accumulator (32 * 128 * (64 * 256 + 128) < 2^27)
                        int ch[4] = {0, 0, 0, 0}, cl[4] = {0, 0, 0, 0};
                        mma_s8s8(ch, a, b2.x, b2.y);
                        mma_s8s8(cl, a, b0.x, b0.y);
#pragma unroll
                        for (int i = 0; i < 4; i++) ch[i] *= 256;
                        mma_s8s8(ch, a, b1.x, b1.y);
#pragma unroll
                        for (int i = 0; i < 4; i++) dot[i] = fmaf((float)ch[i], 256.f, (float)cl[i]);
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 hd = i < 2 ? hd0 : hd1;
                        const float inv = (i & 1) ? sc.z : sc.x, sm = (i & 1) ? sc.w : sc.y;
                        acc[i] = FMT == MGQ_FMT_Q4 ? fmaf(hd.x * inv, dot[i], fmaf(hd.y, sm, acc[i])) : fmaf(hd.x * inv, dot[i], acc[i]);
                    }
                }
            }
            __syncwarp();                                     // all lanes are done with this stage before it is refilled
        }
        // the group's four partial tiles, added in warp order by warp 0 of the group
        *reinterpret_cast<float4 *>(s_red + q * 128u + lane * 4u) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        group_barrier(grp);
        if (q == 0) {
            const uint32_t tile = t0 + grp + j * kGroups;
            float4 sum = *reinterpret_cast<const float4 *>(s_red + lane * 4u);
#pragma unroll
            for (int w = 1; w < kGroupWarps; w++) {
                const float4 o = *reinterpret_cast<const float4 *>(s_red + w * 128u + lane * 4u);
                sum.x += o.x; sum.y += o.y; sum.z += o.z; sum.w += o.w;
            }
            const float out[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t col = tile * kTileCols + g + (i >= 2 ? 8u : 0u), row = 2u * tq + (i & 1);
                if (col < p.n && row < p.m) {
                    const size_t o = (size_t)row * p.n + col;
                    if (p.slices == 1) p.y[o] = p.addend ? out[i] + p.addend[o] : out[i];
                    else               p.y[(size_t)slice * p.m * p.n + o] = out[i];
                }
            }
        }
        group_barrier(grp);                                   // the partials may be overwritten by the next tile
    }
    cp_wait<0>();
}

// y = sum over slices of the partial sums (+ addend), in slice order.
__global__ void sum_slices_kernel(const float *part, const float *addend, float *y, uint32_t len, uint32_t slices)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (i >= len) return;
    float s = 0.f;
    for (uint32_t sl = 0; sl < slices; sl++) s += part[(size_t)sl * len + i];
    y[i] = addend ? s + addend[i] : s;
}

// Partial sums of sliced launches (K > 4096): one buffer per device.  A buffer that has been handed
// to a launch is never freed or moved -- a CUDA graph may have captured its address -- so when a
// larger request arrives a new, larger buffer is allocated and the old one is kept until the process
// exits.  The first call of a given size must therefore come before any stream capture (cudaMalloc is
// not allowed while capturing), and launches that use the buffer must be ordered on one stream per
// device: two streams running sliced GEMVs at the same time would mix their partial sums.
struct Scratch {
    float *ptr = nullptr;
    size_t bytes = 0;
};
Scratch g_scratch[64];
std::mutex g_scratch_mu;

}  // namespace

bool gemv_mma_eligible(uint32_t m, uint32_t k, uint32_t n, const void *x, const void *w)
{
    return m >= 3 && m <= MGQ_GEMV_MAX_M && k % 256 == 0 && k >= 256 && n >= 1 &&
           reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
           ((unsigned long long)(k / 32) * n) % 4 == 0;
}

int launch_gemv_mma(int fmt, const float *x, const void *w, const float *addend, float *y,
                    uint32_t m, uint32_t k, uint32_t n, void *stream_v)
{
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    int dev = 0, sms = 0;
    MGQ_CUDA(cudaGetDevice(&dev));
    MGQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const size_t ring = fmt == MGQ_FMT_Q4 ? (size_t)ring_stages<MGQ_FMT_Q4>() * stage_bytes<MGQ_FMT_Q4>()
                                          : (size_t)ring_stages<MGQ_FMT_Q8>() * stage_bytes<MGQ_FMT_Q8>();
    const size_t smem = kPlaneBytes + kScaleBytes + kRedBytes + (size_t)kWarps * ring;
    static bool opted[64][2] = {};
    auto kernel = fmt == MGQ_FMT_Q4 ? gemv_mma_kernel<MGQ_FMT_Q4> : gemv_mma_kernel<MGQ_FMT_Q8>;
    if (dev >= 0 && dev < 64 && !opted[dev][fmt == MGQ_FMT_Q4]) {
        MGQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        opted[dev][fmt == MGQ_FMT_Q4] = true;
    }
    for (uint32_t r0 = 0; r0 < m; r0 += 8) {
        MmaParams p{};
        p.m = m - r0 < 8 ? m - r0 : 8;
        p.x = x + (size_t)r0 * k;
        p.w = static_cast<const uint8_t *>(w);
        p.addend = addend ? addend + (size_t)r0 * n : nullptr;
        p.k = k; p.n = n; p.bpc = k / 32;
        p.tiles = (n + kTileCols - 1) / kTileCols;
        p.slices = (p.bpc + kSliceBlocks - 1) / kSliceBlocks;
        p.num_blocks = (unsigned long long)p.bpc * n;
        float *out = y + (size_t)r0 * n;
        p.y = out;
        if (p.slices > 1) {
            const size_t need = (size_t)p.slices * p.m * n * sizeof(float);
            std::lock_guard<std::mutex> lock(g_scratch_mu);
            if (dev < 0 || dev >= 64) return fail(MGQ_ERR_CUDA, "device index %d out of range", dev);
            if (g_scratch[dev].bytes < need) {
                // reserve for the widest batch (16 rows run as two launches of 8) so that a later,
                // larger batch of the same shape does not need a second buffer
                const size_t want = (size_t)p.slices * 8 * n * sizeof(float);
                float *fresh = nullptr;
                MGQ_CUDA(cudaMalloc(&fresh, want));
                g_scratch[dev].ptr = fresh;               // the previous buffer stays allocated (see above)
                g_scratch[dev].bytes = want;
            }
            p.y = g_scratch[dev].ptr;
        }
        uint32_t gx = (uint32_t)sms / p.slices;
        if (gx < 1) gx = 1;
        if (gx > p.tiles) gx = p.tiles;
        cudaLaunchConfig_t lc{};
        lc.gridDim = dim3(gx, p.slices, 1);
        lc.blockDim = dim3(kWarps * 32, 1, 1);
        lc.dynamicSmemBytes = smem;
        lc.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
        MGQ_CUDA(cudaLaunchKernelEx(&lc, kernel, p));
        if (p.slices > 1) {
            const uint32_t len = p.m * n;
            cudaLaunchConfig_t ls = lc;
            ls.gridDim = dim3((len + 255) / 256, 1, 1);
            ls.blockDim = dim3(256, 1, 1);
            ls.dynamicSmemBytes = 0;
            MGQ_CUDA(cudaLaunchKernelEx(&ls, sum_slices_kernel, (const float *)p.y, p.addend, out, len, p.slices));
        }
    }
    return MGQ_OK;
}

}  // namespace mgq
