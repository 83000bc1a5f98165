// Dequantize-fused GEMM for Q4/Q8 weights:  C[m,n] = A[m,k] . dequant(W)[k,n] (+ addend).
//
// Stands in for meganeura's MatMul / FusedMatMulAdd dispatches with a quantized weight_format
// (src/compile.rs:1408-1419, 1511-1522; kernel src/shaders/matmul.wgsl:28-109 with
// dequant_q4 / dequant_q8 as the B-tile load, src/codegen.rs:702-713).
//
// gemm_tiled_kernel is the general kernel (any M, any N, f32 or bf16 activations): a 64x64x32
// register-tiled f32 contraction on the CUDA cores in which each K-tile is exactly one
// quantization block per column, so a block header is decoded once per 32 weights (the
// reference decodes it once per weight).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>

#include "mgq_internal.h"

namespace mgq {
namespace {

constexpr int BM = 64, BN = 64, BK = 32, PAD = 4;

template <int FMT, bool A_BF16>
__global__ void __launch_bounds__(256) gemm_tiled_kernel(const void *__restrict__ a_v, const uint8_t *__restrict__ w,
                                                         const float *__restrict__ addend, float *__restrict__ c,
                                                         uint32_t m, uint32_t k, uint32_t n)
{
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Bs[BK][BN + PAD];
    const uint32_t tid = threadIdx.x, tx = tid & 15u, ty = tid >> 4;
    const uint32_t row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const uint32_t bpc = k / 32;
    const unsigned long long num_blocks = (unsigned long long)bpc * n;
    const uint32_t *w32 = reinterpret_cast<const uint32_t *>(w);

    float acc[4][4] = {};
    for (uint32_t kb = 0; kb < bpc; kb++) {
        // A tile: 64 rows x 32 k, 8 values per thread
        {
            const uint32_t r = tid >> 2, kq = (tid & 3u) * 8u;
            const uint32_t row = row0 + r;
            float v[8] = {};
            if (row < m) {
                if (A_BF16) {
                    const __nv_bfloat16 *ap = static_cast<const __nv_bfloat16 *>(a_v) + (size_t)row * k + kb * 32u + kq;
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = __bfloat162float(ap[e]);
                } else {
                    const float *ap = static_cast<const float *>(a_v) + (size_t)row * k + kb * 32u + kq;
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = ap[e];
                }
            }
#pragma unroll
            for (int e = 0; e < 8; e++) As[kq + e][r] = v[e];
        }
        // W tile: 64 columns x one block, 8 weights per thread
        {
            const uint32_t cl = tid >> 2, part = tid & 3u;
            const uint32_t col = col0 + cl;
            float v[8] = {};
            if (col < n) {
                const unsigned long long g = (unsigned long long)col * bpc + kb;
                if (FMT == MGQ_FMT_Q4) {
                    const uint32_t h = w32[g];
                    const float2 dm = __half22float2(*reinterpret_cast<const __half2 *>(&h));
                    const uint32_t wv = w32[num_blocks + g * 4 + part];
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = (float)((wv >> (4 * e)) & 0xFu) * dm.x + dm.y;
                } else {
                    const uint32_t *bp = w32 + g * 9;
                    const float scale = __half2float(__ushort_as_half((unsigned short)(bp[0] & 0xFFFFu)));
#pragma unroll
                    for (int h2 = 0; h2 < 2; h2++) {
                        const uint32_t wv = bp[1 + part * 2 + h2];
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            v[h2 * 4 + e] = (float)(int)(signed char)((wv >> (8 * e)) & 0xFFu) * scale;
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < 8; e++) Bs[part * 8 + e][cl] = v[e];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            const float4 av = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t row = row0 + ty * 4 + i;
        if (row >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t col = col0 + tx * 4 + j;
            if (col >= n) continue;
            const size_t o = (size_t)row * n + col;
            c[o] = addend ? acc[i][j] + addend[o] : acc[i][j];
        }
    }
}

}  // namespace

static int g_force_tiled = 0;
bool force_tiled() { return g_force_tiled != 0; }
int set_gemm_option(const char *name, long value)
{
    if (!std::strcmp(name, "gemm.force_tiled")) { g_force_tiled = value ? 1 : 0; return MGQ_OK; }
    return fail(MGQ_ERR_NAME, "unknown option: %s", name);
}

int launch_gemm(int fmt, const void *a, int a_dtype, const void *w, const float *addend, float *c,
                uint32_t m, uint32_t k, uint32_t n, void *stream_v)
{
    if (gemm_tc_eligible(a_dtype, m, k, n, a) && !force_tiled()) return launch_gemm_tc(fmt, a, w, addend, c, m, k, n, stream_v);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM, 1), block(256, 1, 1);
    const uint8_t *w8 = static_cast<const uint8_t *>(w);
    const bool bf = a_dtype == MGQ_A_BF16;
    if (fmt == MGQ_FMT_Q4) {
        if (bf) gemm_tiled_kernel<MGQ_FMT_Q4, true><<<grid, block, 0, stream>>>(a, w8, addend, c, m, k, n);
        else    gemm_tiled_kernel<MGQ_FMT_Q4, false><<<grid, block, 0, stream>>>(a, w8, addend, c, m, k, n);
    } else {
        if (bf) gemm_tiled_kernel<MGQ_FMT_Q8, true><<<grid, block, 0, stream>>>(a, w8, addend, c, m, k, n);
        else    gemm_tiled_kernel<MGQ_FMT_Q8, false><<<grid, block, 0, stream>>>(a, w8, addend, c, m, k, n);
    }
    MGQ_CUDA(cudaGetLastError());
    return MGQ_OK;
}

}  // namespace mgq
