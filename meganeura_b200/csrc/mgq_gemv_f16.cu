// GEMV over f16 weights: y[m, n] = x[m, k] . W[k, n] (+ addend), W row-major binary16, f32 accumulate.
//
// meganeura keeps `parameter_f16` weights as plain row-major f16 and runs its f32 GEMV shader with
// the matrix_b loads widened (src/codegen.rs:1065-1101, gen_matmul_gemv_f16; shader
// src/shaders/matmul_gemv.wgsl).  Rows of W are contiguous along N, so a thread owns 8 consecutive
// columns (one 16-byte load per row of W) and a strided set of rows; the K-slices of a CTA are
// added in slice order through shared memory.  HBM-bound: algorithmic bytes 2*K*N + 4*M*(K+N).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "mgq_internal.h"

namespace mgq {
namespace {

constexpr int kF16Threads = 256;
constexpr int kF16Rows = 4;                 // activation rows per pass

// LANES column lanes (8 columns each) x (256 / LANES) K-slices per CTA.
template <int LANES>
__global__ void __launch_bounds__(kF16Threads) gemv_f16_kernel(const float *x, const __half *w, const float *addend, float *y,
                                                              uint32_t m, uint32_t k, uint32_t n)
{
    constexpr int SLICES = kF16Threads / LANES, TILE = LANES * 8;
    __shared__ float s_part[SLICES][TILE + 1];
    const uint32_t t = threadIdx.x, lane = t % LANES, slice = t / LANES;
    const uint32_t col0 = blockIdx.x * TILE + lane * 8;
    const bool live = col0 < n;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    float acc[kF16Rows][8];
#pragma unroll
    for (int r = 0; r < kF16Rows; r++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[r][j] = 0.f;
    if (live) {
        const uint4 *wp = reinterpret_cast<const uint4 *>(w + (size_t)slice * n + col0);
        const size_t step = (size_t)SLICES * n / 8;                     // uint4 elements between this thread's rows
#pragma unroll 8
        for (uint32_t kk = slice; kk < k; kk += SLICES, wp += step) {
            const uint4 q = __ldg(wp);
            const __half2 *h = reinterpret_cast<const __half2 *>(&q);
            float wv[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(h[j]);
                wv[2 * j] = f.x;
                wv[2 * j + 1] = f.y;
            }
#pragma unroll
            for (int r = 0; r < kF16Rows; r++) {
                if (r < (int)m) {
                    const float xv = __ldg(x + (size_t)r * k + kk);
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[r][j] = fmaf(xv, wv[j], acc[r][j]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kF16Rows; r++) {
        if (r >= (int)m) break;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 8; j++) s_part[slice][lane * 8 + j] = acc[r][j];
        __syncthreads();
        if (t < TILE) {
            const uint32_t col = blockIdx.x * TILE + t;
            if (col < n) {
                float s = 0.f;
                for (int sl = 0; sl < SLICES; sl++) s += s_part[sl][t];
                const size_t o = (size_t)r * n + col;
                y[o] = addend ? s + addend[o] : s;
            }
        }
    }
}

}  // namespace

int launch_gemv_f16(const float *x, const void *w, const float *addend, float *y, uint32_t m, uint32_t k, uint32_t n, void *stream_v)
{
    if (n % 8 != 0) return fail(MGQ_ERR_SHAPE, "f16 GEMV needs N to be a multiple of 8, got %u", n);
    if (reinterpret_cast<uintptr_t>(w) % 16 != 0) return fail(MGQ_ERR_ALIGN, "f16 weight pointer must be 16-byte aligned");
    int dev = 0, sms = 0;
    MGQ_CUDA(cudaGetDevice(&dev));
    MGQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    // Narrow column tiles win: 32 columns (64-byte row segments, 64 K-slices per CTA); 16 columns when
    // even that gives an SM fewer than eight CTAs.
    const int lanes = (n + 31) / 32 >= 8u * (uint32_t)sms ? 4 : 2;
    for (uint32_t r0 = 0; r0 < m; r0 += kF16Rows) {
        const uint32_t rows = m - r0 < (uint32_t)kF16Rows ? m - r0 : (uint32_t)kF16Rows;
        cudaLaunchConfig_t lc{};
        lc.gridDim = dim3((n + lanes * 8 - 1) / (lanes * 8), 1, 1);
        lc.blockDim = dim3(kF16Threads, 1, 1);
        lc.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        lc.attrs = attr;
        lc.numAttrs = 1;
        const float *xr = x + (size_t)r0 * k;
        const float *ar = addend ? addend + (size_t)r0 * n : nullptr;
        float *yr = y + (size_t)r0 * n;
        const __half *wh = static_cast<const __half *>(w);
        if (lanes == 2) MGQ_CUDA(cudaLaunchKernelEx(&lc, gemv_f16_kernel<2>, xr, wh, ar, yr, rows, k, n));
        else            MGQ_CUDA(cudaLaunchKernelEx(&lc, gemv_f16_kernel<4>, xr, wh, ar, yr, rows, k, n));
    }
    return MGQ_OK;
}

}  // namespace mgq

// ---------------------------------------------------------------------------------------------
// Transposed f32 GEMV: y[n] = sum_k x[k] * B[n, k], B row-major [N, K] -- the reference's
// MatMulGemvBT (src/shaders/matmul_gemv_bt.wgsl:34-65; lowering src/compile.rs:1447-1469), which a
// model with tied embeddings uses for its lm_head (B is the embedding table).  A row of B is
// contiguous along K, so a warp owns a row at a time and its lanes read consecutive float4 pieces
// (the reference's K-split); two rows are in flight per warp.  HBM-bound: 4*K*N + 4*(K+N) bytes.
namespace mgq {
namespace {

__global__ void __launch_bounds__(256) gemv_bt_kernel(const float *x, const float *b, float *y, uint32_t k, uint32_t n)
{
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nwarps = gridDim.x * (blockDim.x >> 5);
    const uint32_t k4 = k / 4;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    for (uint32_t row = 2u * warp; row < n; row += 2u * nwarps) {
        const bool two = row + 1u < n;
        const float4 *r0 = reinterpret_cast<const float4 *>(b + (size_t)row * k);
        const float4 *r1 = reinterpret_cast<const float4 *>(b + (size_t)(two ? row + 1u : row) * k);
        float a0 = 0.f, a1 = 0.f;
        for (uint32_t i = lane; i < k4; i += 32u) {
            const float4 xv = __ldg(x4 + i), p = __ldcs(r0 + i), q = __ldcs(r1 + i);
            a0 += xv.x * p.x + xv.y * p.y + xv.z * p.z + xv.w * p.w;
            a1 += xv.x * q.x + xv.y * q.y + xv.z * q.z + xv.w * q.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a0 += __shfl_xor_sync(0xffffffffu, a0, o);
            a1 += __shfl_xor_sync(0xffffffffu, a1, o);
        }
        if (lane == 0) {
            y[row] = a0;
            if (two) y[row + 1u] = a1;
        }
    }
}

}  // namespace

int launch_gemv_bt(const float *x, const float *b, float *y, uint32_t k, uint32_t n, void *stream_v)
{
    const uint32_t warps_needed = (n + 1) / 2;
    uint32_t grid = (warps_needed + 7) / 8;
    if (grid > 148u * 8u) grid = 148u * 8u;
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3(grid);
    lc.blockDim = dim3(256);
    lc.stream = static_cast<cudaStream_t>(stream_v);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    MGQ_CUDA(cudaLaunchKernelEx(&lc, gemv_bt_kernel, x, b, y, k, n));
    return MGQ_OK;
}

}  // namespace mgq
