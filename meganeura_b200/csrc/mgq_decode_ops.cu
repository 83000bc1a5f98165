// The operators that sit between the quantized GEMVs of a decode step, as plain CUDA kernels:
// embedding lookup, RMSNorm, RoPE with a device-side position, KV-cache write, single-token cached
// attention, SwiGLU, and a device-side greedy pick.  Semantics follow meganeura's shaders
//   src/shaders/embedding.wgsl, rms_norm.wgsl, rope_dynamic.wgsl, cache_write.wgsl,
//   cached_attention.wgsl, swiglu_concat.wgsl (forward), binary.wgsl (swiglu)
// and their lowering in src/compile.rs (Op::Embedding, Op::RmsNorm, Op::RoPE with a dynamic offset,
// Op::CacheWrite, Op::CachedAttention, Op::SwiGLU, Op::SwiGLUConcat).
//
// All of them are tiny next to the GEMVs (a few KB to a few MB per launch), so the design goal is
// latency: every kernel is launched with programmatic stream serialization, does its index
// arithmetic, then waits for its predecessor (griddepcontrol.wait) right before the first load.
// The position / token inputs live in device memory (like the reference's kv_pos_buf), so a whole
// decode step is a fixed launch sequence that can be replayed from a CUDA graph.
#include <cuda_runtime.h>

#include <cfloat>
#include <cstdint>

#include "mgq_internal.h"

namespace mgq {
namespace {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

template <typename... Args>
int launch(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t lc{};
    lc.gridDim = grid;
    lc.blockDim = block;
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    MGQ_CUDA(cudaLaunchKernelEx(&lc, kernel, args...));
    return MGQ_OK;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------- embedding (embedding.wgsl)
__global__ void embedding_kernel(const uint32_t *ids, const float *table, float *out, uint32_t seq, uint32_t hidden,
                                 uint32_t vocab)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;          // float4 index
    const uint32_t per_row = hidden / 4;
    pdl_launch_dependents();
    pdl_wait();
    if (i >= seq * per_row) return;
    const uint32_t row = i / per_row, col = i - row * per_row;
    uint32_t tok = ids[row];
    if (tok >= vocab) tok = vocab - 1;                                  // the reference would read out of bounds
    reinterpret_cast<float4 *>(out)[i] = reinterpret_cast<const float4 *>(table)[(size_t)tok * per_row + col];
}

// ---------------------------------------------------------------- RMSNorm (rms_norm.wgsl)
// One CTA per row: dst = src * rsqrt(mean(src^2) + eps) * weight.  The weight vector is a constant
// of the model, so it is fetched before the wait on the predecessor; a row of up to 16384 floats
// stays in registers between the two passes, so the kernel costs one global round trip after the wait.
__global__ void __launch_bounds__(256) rms_norm_kernel(const float *src, const float *weight, float *dst, uint32_t cols, float eps)
{
    constexpr int kHold = 16;                       // float4 values a thread keeps
    __shared__ float s_part[8];
    const uint32_t row = blockIdx.x, t = threadIdx.x;
    const float4 *x4 = reinterpret_cast<const float4 *>(src + (size_t)row * cols);
    const float4 *w4 = reinterpret_cast<const float4 *>(weight);
    float4 *y4 = reinterpret_cast<float4 *>(dst + (size_t)row * cols);
    const uint32_t n4 = cols / 4;
    const bool held = n4 <= 256u * kHold;
    float4 w[kHold], v[kHold];
    pdl_launch_dependents();
    if (held) {
#pragma unroll
        for (int i = 0; i < kHold; i++) w[i] = t + 256u * i < n4 ? __ldg(w4 + t + 256u * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    float ss = 0.f;
    if (held) {
#pragma unroll
        for (int i = 0; i < kHold; i++) {
            v[i] = t + 256u * i < n4 ? x4[t + 256u * i] : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    } else {
        for (uint32_t j = t; j < n4; j += 256) {
            const float4 q = x4[j];
            ss += q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
        }
    }
    ss = warp_sum(ss);
    if ((t & 31u) == 0) s_part[t >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) total += s_part[i];
    const float r = rsqrtf(total / (float)cols + eps);
    if (held) {
#pragma unroll
        for (int i = 0; i < kHold; i++)
            if (t + 256u * i < n4) y4[t + 256u * i] = make_float4(v[i].x * r * w[i].x, v[i].y * r * w[i].y, v[i].z * r * w[i].z, v[i].w * r * w[i].w);
    } else {
        for (uint32_t j = t; j < n4; j += 256) {
            const float4 q = x4[j], u = w4[j];
            y4[j] = make_float4(q.x * r * u.x, q.y * r * u.y, q.z * r * u.z, q.w * r * u.w);
        }
    }
}

// ---------------------------------------------------------------- RoPE, dynamic offset (rope_dynamic.wgsl)
// HF half-split pairs inside each head; position = row + *pos_offset.
__global__ void rope_kernel(const float *src, float *dst, const uint32_t *pos_offset, uint32_t seq, uint32_t dim,
                            uint32_t head_dim, float theta)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t half_dim = dim / 2, half_head = head_dim / 2;
    pdl_launch_dependents();
    if (i >= seq * half_dim) { pdl_wait(); return; }
    const uint32_t row = i / half_dim, pair_in_row = i - row * half_dim;
    const uint32_t head = pair_in_row / half_head, pair_in_head = pair_in_row - head * half_head;
    const float inv_freq = powf(theta, -2.0f * (float)pair_in_head / (float)head_dim);
    pdl_wait();
    const float angle = (float)(row + pos_offset[0]) * inv_freq;
    float s, c;
    sincosf(angle, &s, &c);
    const uint32_t idx0 = row * dim + head * head_dim + pair_in_head, idx1 = idx0 + half_head;
    const float v0 = src[idx0], v1 = src[idx1];
    dst[idx0] = v0 * c - v1 * s;
    dst[idx1] = v0 * s + v1 * c;
}

// ---------------------------------------------------------------- RoPE(q), RoPE(k) and both cache writes in one launch
// The four dispatches that follow the q|k|v projection of a decode layer (rope_dynamic.wgsl twice,
// cache_write.wgsl twice) touch a few KB; one launch instead of four saves three kernel boundaries
// per layer.  Thread ranges: q pairs, then k pairs (rotated k also goes to its cache row), then v.
__global__ void rope_cache_kernel(const float *q_src, float *q_dst, const float *k_src, float *k_dst, const float *v_src,
                                  float *k_cache, float *v_cache, const uint32_t *pos_buf, uint32_t q_dim, uint32_t kv_dim,
                                  uint32_t head_dim, float theta, uint32_t max_seq)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t half_head = head_dim / 2, q_pairs = q_dim / 2, k_pairs = kv_dim / 2;
    pdl_launch_dependents();
    if (i >= q_pairs + k_pairs + kv_dim) { pdl_wait(); return; }
    const bool is_v = i >= q_pairs + k_pairs, is_k = !is_v && i >= q_pairs;
    const uint32_t pair = is_k ? i - q_pairs : i;
    const uint32_t head = pair / half_head, pair_in_head = pair - head * half_head;
    const float inv_freq = is_v ? 0.f : powf(theta, -2.0f * (float)pair_in_head / (float)head_dim);
    pdl_wait();
    const uint32_t pos = pos_buf[0];
    if (is_v) {
        const uint32_t j = i - q_pairs - k_pairs;
        if (pos < max_seq) v_cache[(size_t)pos * kv_dim + j] = v_src[j];
        return;
    }
    float s, c;
    sincosf((float)pos * inv_freq, &s, &c);
    const uint32_t idx0 = head * head_dim + pair_in_head, idx1 = idx0 + half_head;
    const float *src = is_k ? k_src : q_src;
    float *dst = is_k ? k_dst : q_dst;
    const float v0 = src[idx0], v1 = src[idx1];
    const float r0 = v0 * c - v1 * s, r1 = v0 * s + v1 * c;
    dst[idx0] = r0;
    dst[idx1] = r1;
    if (is_k && pos < max_seq) {
        k_cache[(size_t)pos * kv_dim + idx0] = r0;
        k_cache[(size_t)pos * kv_dim + idx1] = r1;
    }
}

// ---------------------------------------------------------------- KV-cache write (cache_write.wgsl)
__global__ void cache_write_kernel(const float *src, float *cache, const uint32_t *kv_pos, uint32_t dim, uint32_t max_seq)
{
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t pos = kv_pos[0];
    if (j < dim && pos < max_seq) cache[(size_t)pos * dim + j] = src[j];
}

// ---------------------------------------------------------------- SwiGLU (binary.wgsl swiglu, swiglu_concat.wgsl)
// out[r, c] = silu(gate[r, c]) * up[r, c]; gate and up are rows of pitch `pitch` floats (for the
// concatenated form both point into the same [rows, 2*half_n] matrix).
__global__ void swiglu_kernel(const float *gate, const float *up, float *out, uint32_t rows, uint32_t half_n, uint32_t pitch)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (i >= rows * half_n) return;
    const uint32_t row = i / half_n, col = i - row * half_n;
    const float g = gate[(size_t)row * pitch + col], u = up[(size_t)row * pitch + col];
    const float sig = 1.0f / (1.0f + expf(-g));
    out[i] = g * sig * u;
}

// ---------------------------------------------------------------- cached attention (cached_attention.wgsl)
// One query token against positions 0..kv_pos of the cache.  The reference runs one 64-thread
// workgroup per query head over the whole context with an online softmax; here the context is cut
// into chunks of kChunk positions and a CTA takes one chunk for ALL query heads of one KV head
// (grouped-query attention reads each K/V row once, not once per query head).  Every CTA leaves an
// unnormalised partial (max, sum, weighted V) in the workspace; the CTA of a KV head that finishes
// last merges the partials -- the same online-softmax algebra, applied across chunks.
constexpr int kChunk = 64;
constexpr int kMaxGroup = 8;          // query heads per KV head

// The last CTA of a KV head merges the chunk partials: out[g, d] = sum_c w_c acc_c[g, d] / sum_c w_c l_c
// with w_c = exp(m_c - max_c m_c).  Every global round trip costs ~1 us here (the partials sit in
// L2, written by other SMs), so the loads are arranged to need few of them: the first batch of
// accumulator loads is issued before the maxima and sums are even known, and each thread keeps
// NOUT x BATCH independent loads in flight (thread t owns outputs t + 128 j).
template <int D, int NOUT, int BATCH>
__device__ __forceinline__ void merge_partials(const float *base, uint32_t live, uint32_t group, float *s_w, float *out)
{
    __shared__ float s_inv[kMaxGroup];
    constexpr size_t cstride = (size_t)kMaxGroup * (D + 2);
    const uint32_t t = threadIdx.x, lane = t & 31u, warp = t >> 5, total = group * D;
    float acc[NOUT], v[NOUT][BATCH];
    auto fetch = [&](uint32_t c0) {
#pragma unroll
        for (int j = 0; j < NOUT; j++) {
            const uint32_t i = t + 128u * j;
            const float *col = base + (size_t)(i / D) * (D + 2) + i % D;
#pragma unroll
            for (int u = 0; u < BATCH; u++) v[j][u] = (i < total && c0 + u < live) ? __ldcg(col + (c0 + u) * cstride) : 0.f;
        }
    };
#pragma unroll
    for (int j = 0; j < NOUT; j++) acc[j] = 0.f;
    fetch(0);
    // chunk weights into shared memory ([group][kChunk]; at most kChunk chunks, checked at launch)
    for (uint32_t g = warp; g < group; g += 4) {
        float mc[2], lc[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t c = lane + 32u * h;
            const float *pc = base + ((size_t)c * kMaxGroup + g) * (D + 2);
            mc[h] = c < live ? __ldcg(pc + D) : -FLT_MAX;
            lc[h] = c < live ? __ldcg(pc + D + 1) : 0.f;
        }
        float m = fmaxf(mc[0], mc[1]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const float w = lane + 32u * h < live ? expf(mc[h] - m) : 0.f;
            s_w[g * kChunk + lane + 32u * h] = w;
            l = fmaf(lc[h], w, l);
        }
        l = warp_sum(l);
        if (lane == 0) s_inv[g] = 1.0f / (l == 0.f ? 1.f : l);
    }
    __syncthreads();
    for (uint32_t c0 = 0; c0 < live; c0 += BATCH) {
        if (c0) fetch(c0);
#pragma unroll
        for (int j = 0; j < NOUT; j++) {
            const uint32_t g = min((t + 128u * j) / D, (uint32_t)kMaxGroup - 1u);
#pragma unroll
            for (int u = 0; u < BATCH; u++) acc[j] = fmaf(v[j][u], c0 + u < live ? s_w[g * kChunk + c0 + u] : 0.f, acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < NOUT; j++) {
        const uint32_t i = t + 128u * j;
        if (i < total) out[i] = acc[j] * s_inv[i / D];
    }
}

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem)
{
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Dynamic shared memory: the chunk's K rows, then its V rows ([kChunk][D] floats each).  Both tiles
// are requested with cp.async up front, so a CTA has its whole 64 KB (D = 128) in flight at once
// instead of paying a memory round trip per position.
template <int D, int G2>              // head_dim: 64 or 128; G2: query heads per KV head rounded up to 4 or 8; blockDim.x == 128
__global__ void __launch_bounds__(128) cached_attention_kernel(const float *q, const float *k_cache, const float *v_cache,
                                                               const uint32_t *kv_pos, float *out, uint32_t num_heads,
                                                               uint32_t num_kv_heads, uint32_t max_seq, float *workspace,
                                                               unsigned int *counters)
{
    constexpr int LPP = D / 4;                    // lanes per position (each lane holds a float4 of the row)
    constexpr int PPW = 32 / LPP;                 // positions per warp step
    extern __shared__ __align__(16) float s_tiles[];
    float *s_k = s_tiles, *s_v = s_tiles + kChunk * D;
    __shared__ float s_score[kMaxGroup][kChunk];
    __shared__ float s_q[kMaxGroup][D];
    __shared__ float s_acc[128 / D][kMaxGroup][D];
    __shared__ bool s_last;
    const uint32_t kvh = blockIdx.x, chunk = blockIdx.y, splits = gridDim.y;
    const uint32_t t = threadIdx.x, lane = t & 31u, warp = t >> 5;
    const uint32_t group = num_heads / num_kv_heads, kv_dim = num_kv_heads * D;
    const float scale = rsqrtf((float)D);
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t kv_len = min(kv_pos[0] + 1u, max_seq);
    const uint32_t p0 = chunk * kChunk, p1 = min(p0 + kChunk, kv_len);
    float *part = workspace + ((size_t)kvh * splits + chunk) * kMaxGroup * (D + 2);      // [group][D + 2]: acc, max, sum

    if (p0 < kv_len) {
        const uint32_t rows = p1 - p0;
        for (uint32_t i = t; i < rows * LPP; i += 128) {
            const uint32_t r = i / LPP, c = i % LPP;
            cp_async16(s_k + r * D + c * 4, k_cache + (size_t)(p0 + r) * kv_dim + kvh * D + c * 4);
        }
        cp_async_commit();
        for (uint32_t i = t; i < rows * LPP; i += 128) {
            const uint32_t r = i / LPP, c = i % LPP;
            cp_async16(s_v + r * D + c * 4, v_cache + (size_t)(p0 + r) * kv_dim + kvh * D + c * 4);
        }
        cp_async_commit();
        for (uint32_t i = t; i < group * D; i += 128) s_q[i / D][i % D] = q[(size_t)kvh * group * D + i];
        cp_async_wait<1>();
        __syncthreads();
        // scores: PPW positions per warp step, LPP lanes per position.  The query slices stay in
        // registers; the G2 partial dot products of a row are reduced together: every exchange with
        // the lane `off` away halves the number of heads a lane is still responsible for, so a row
        // costs G2 - 1 + log2(LPP / G2) shuffles instead of one full reduction per head.
        const uint32_t sub = lane / LPP, li = lane % LPP;
        float4 qreg[G2];
#pragma unroll
        for (int h = 0; h < G2; h++)
            qreg[h] = h < (int)group ? *reinterpret_cast<const float4 *>(&s_q[h][li * 4]) : make_float4(0.f, 0.f, 0.f, 0.f);
        // the head this lane ends up with: one bit per halving step, taken from the lane's position
        uint32_t my_head = 0;
#pragma unroll
        for (int keep = G2 / 2, off = LPP / 2; keep >= 1; keep >>= 1, off >>= 1) my_head = my_head * 2u + ((li & off) ? 1u : 0u);
        for (uint32_t r = warp * PPW + sub; r < (uint32_t)kChunk; r += 4 * PPW) {
            float v[G2];
            if (r < rows) {
                const float4 kv = *reinterpret_cast<const float4 *>(s_k + r * D + li * 4);
#pragma unroll
                for (int h = 0; h < G2; h++) v[h] = kv.x * qreg[h].x + kv.y * qreg[h].y + kv.z * qreg[h].z + kv.w * qreg[h].w;
            } else {
#pragma unroll
                for (int h = 0; h < G2; h++) v[h] = 0.f;
            }
#pragma unroll
            for (int keep = G2 / 2, off = LPP / 2; keep >= 1; keep >>= 1, off >>= 1) {
                const bool upper = (li & off) != 0;
#pragma unroll
                for (int i = 0; i < keep; i++) {
                    const float send = upper ? v[i] : v[i + keep];
                    const float mine = upper ? v[i + keep] : v[i];
                    v[i] = mine + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
#pragma unroll
            for (int off = LPP / (2 * G2); off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
            if ((li & (LPP / G2 - 1)) == 0 && my_head < group) s_score[my_head][r] = r < rows ? v[0] * scale : -FLT_MAX;
        }
        __syncthreads();
        // per head: chunk maximum and exponentials (warp w takes heads w, w+4)
        for (uint32_t g = warp; g < group; g += 4) {
            float m = fmaxf(s_score[g][lane], s_score[g][lane + 32]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const float e0 = lane < rows ? expf(s_score[g][lane] - m) : 0.f;
            const float e1 = lane + 32 < rows ? expf(s_score[g][lane + 32] - m) : 0.f;
            s_score[g][lane] = e0;
            s_score[g][lane + 32] = e1;
            const float l = warp_sum(e0 + e1);
            if (lane == 0) { part[g * (D + 2) + D] = m; part[g * (D + 2) + D + 1] = l; }
        }
        cp_async_wait<0>();
        __syncthreads();
        // weighted V: thread <-> (position slice, dim); 128 / D slices
        const uint32_t d = t % D, slice = t / D;
        constexpr uint32_t SL = 128 / D;
        float acc[kMaxGroup];
#pragma unroll
        for (int g = 0; g < kMaxGroup; g++) acc[g] = 0.f;
        for (uint32_t r = slice; r < rows; r += SL) {
            const float v = s_v[r * D + d];
#pragma unroll
            for (int g = 0; g < kMaxGroup; g++)
                if (g < (int)group) acc[g] = fmaf(s_score[g][r], v, acc[g]);
        }
#pragma unroll
        for (int g = 0; g < kMaxGroup; g++)
            if (g < (int)group) s_acc[slice][g][d] = acc[g];
        __syncthreads();
        if (slice == 0) {
            for (uint32_t g = 0; g < group; g++) {
                float a = s_acc[0][g][d];
                if (SL > 1) a += s_acc[SL - 1][g][d];
                part[g * (D + 2) + d] = a;
            }
        }
    }
    // the last CTA of this KV head merges
    __threadfence();
    __syncthreads();
    if (t == 0) {
        const unsigned int done = atomicAdd(&counters[kvh], 1u);
        s_last = done == splits - 1;
        if (s_last) counters[kvh] = 0;                       // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const uint32_t live = (kv_len + kChunk - 1) / kChunk;
    const float *base = workspace + (size_t)kvh * splits * kMaxGroup * (D + 2);
    if (group * D <= 4 * 128) merge_partials<D, 4, 16>(base, live, group, &s_score[0][0], out + (size_t)kvh * group * D);
    else                      merge_partials<D, kMaxGroup, 8>(base, live, group, &s_score[0][0], out + (size_t)kvh * group * D);
}

// ---------------------------------------------------------------- greedy pick
// argmax over the logits (lowest index wins ties, like a sequential host scan); the CTA that
// finishes last writes the winner to *out_token, appends it to the history and, when asked,
// feeds it back: *next_token = winner, *kv_pos += 1.
__global__ void __launch_bounds__(256) argmax_kernel(const float *logits, uint32_t n, float *part_val, uint32_t *part_idx,
                                                     unsigned int *counter, uint32_t *out_token, uint32_t *next_token,
                                                     uint32_t *kv_pos, uint32_t *history, uint32_t history_cap)
{
    __shared__ float s_val[8];
    __shared__ uint32_t s_idx[8];
    __shared__ bool s_last;
    const uint32_t t = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    float best = -FLT_MAX;
    uint32_t best_i = 0xFFFFFFFFu;
    for (uint32_t i = blockIdx.x * 256 + t; i < n; i += gridDim.x * 256) {
        const float v = logits[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    auto merge = [](float &bv, uint32_t &bi, float ov, uint32_t oi) {
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        merge(best, best_i, ov, oi);
    }
    if ((t & 31u) == 0) { s_val[t >> 5] = best; s_idx[t >> 5] = best_i; }
    __syncthreads();
    if (t == 0) {
        for (int w = 1; w < 8; w++) merge(best, best_i, s_val[w], s_idx[w]);
        part_val[blockIdx.x] = best;
        part_idx[blockIdx.x] = best_i;
        __threadfence();
        const unsigned int done = atomicAdd(counter, 1u);
        s_last = done == gridDim.x - 1;
        if (s_last) *counter = 0;
    }
    __syncthreads();
    if (!s_last || t >= 32) return;
    __threadfence();
    best = -FLT_MAX;
    best_i = 0xFFFFFFFFu;
    for (uint32_t b = t; b < gridDim.x; b += 32) merge(best, best_i, __ldcg(part_val + b), __ldcg(part_idx + b));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        merge(best, best_i, ov, oi);
    }
    if (t != 0) return;
    if (best_i == 0xFFFFFFFFu) best_i = 0;                   // every logit was NaN
    *out_token = best_i;
    if (history && kv_pos && kv_pos[0] < history_cap) history[kv_pos[0]] = best_i;
    if (next_token) *next_token = best_i;
    if (kv_pos && next_token) kv_pos[0] += 1;
}

}  // namespace

int launch_embedding(const uint32_t *ids, const float *table, float *out, uint32_t seq, uint32_t hidden, uint32_t vocab, void *stream)
{
    if (hidden % 4 != 0) return fail(MGQ_ERR_SHAPE, "embedding width %u must be a multiple of 4", hidden);
    const uint32_t total = seq * (hidden / 4);
    return launch(embedding_kernel, dim3((total + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), ids, table, out, seq,
                  hidden, vocab);
}

int launch_rms_norm(const float *x, const float *weight, float *out, uint32_t rows, uint32_t cols, float eps, void *stream)
{
    if (cols % 4 != 0) return fail(MGQ_ERR_SHAPE, "rms_norm width %u must be a multiple of 4", cols);
    return launch(rms_norm_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), x, weight, out, cols, eps);
}

int launch_rope(const float *x, float *out, const uint32_t *pos_offset, uint32_t seq, uint32_t dim, uint32_t head_dim, float theta,
                void *stream)
{
    if (dim % 2 || head_dim % 2 || dim % head_dim) return fail(MGQ_ERR_SHAPE, "rope: dim %u / head_dim %u", dim, head_dim);
    const uint32_t total = seq * (dim / 2);
    return launch(rope_kernel, dim3((total + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), x, out, pos_offset, seq, dim,
                  head_dim, theta);
}

int launch_rope_cache(const float *q_src, float *q_dst, const float *k_src, float *k_dst, const float *v_src, float *k_cache,
                      float *v_cache, const uint32_t *pos, uint32_t q_dim, uint32_t kv_dim, uint32_t head_dim, float theta,
                      uint32_t max_seq, void *stream)
{
    if (q_dim % head_dim || kv_dim % head_dim || head_dim % 2) return fail(MGQ_ERR_SHAPE, "rope: dims %u / %u, head_dim %u", q_dim, kv_dim, head_dim);
    const uint32_t total = q_dim / 2 + kv_dim / 2 + kv_dim;
    return launch(rope_cache_kernel, dim3((total + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), q_src, q_dst, k_src, k_dst,
                  v_src, k_cache, v_cache, pos, q_dim, kv_dim, head_dim, theta, max_seq);
}

int launch_cache_write(const float *src, float *cache, const uint32_t *kv_pos, uint32_t dim, uint32_t max_seq, void *stream)
{
    return launch(cache_write_kernel, dim3((dim + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), src, cache, kv_pos, dim,
                  max_seq);
}

int launch_swiglu(const float *gate, const float *up, float *out, uint32_t rows, uint32_t half_n, uint32_t pitch, void *stream)
{
    const uint32_t total = rows * half_n;
    return launch(swiglu_kernel, dim3((total + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), gate, up, out, rows, half_n,
                  pitch);
}

size_t attention_workspace_bytes(uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq)
{
    const size_t splits = (max_seq + kChunk - 1) / kChunk;
    return 256 + (size_t)num_kv_heads * splits * kMaxGroup * (head_dim + 2) * sizeof(float);   // 256 B of counters first
}

int launch_cached_attention(const float *q, const float *k_cache, const float *v_cache, const uint32_t *kv_pos, float *out,
                            uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq, void *workspace,
                            void *stream)
{
    if (num_kv_heads == 0 || num_heads % num_kv_heads != 0) return fail(MGQ_ERR_SHAPE, "attention: %u heads over %u KV heads", num_heads, num_kv_heads);
    if (num_heads / num_kv_heads > (uint32_t)kMaxGroup) return fail(MGQ_ERR_SHAPE, "attention: at most %d query heads per KV head", kMaxGroup);
    if (num_kv_heads > 64) return fail(MGQ_ERR_SHAPE, "attention: at most 64 KV heads");
    if (max_seq > (uint32_t)(kChunk * kChunk)) return fail(MGQ_ERR_SHAPE, "attention: cache of %u rows (at most %d)", max_seq, kChunk * kChunk);
    if (!workspace) return fail(MGQ_ERR_NULL, "attention needs its workspace");
    unsigned int *counters = static_cast<unsigned int *>(workspace);
    float *partials = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + 256);
    const dim3 grid(num_kv_heads, (max_seq + kChunk - 1) / kChunk);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t tiles = (size_t)2 * kChunk * head_dim * sizeof(float);
    const bool small_group = num_heads / num_kv_heads <= 4;
    if (head_dim == 64)
        return launch(small_group ? cached_attention_kernel<64, 4> : cached_attention_kernel<64, 8>, grid, dim3(128), tiles, st, q, k_cache,
                      v_cache, kv_pos, out, num_heads, num_kv_heads, max_seq, partials, counters);
    if (head_dim == 128) {
        static bool opted_in[64] = {};
        int dev = 0;
        MGQ_CUDA(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !opted_in[dev]) {                  // 64 KB of dynamic shared memory needs the opt-in, once per device
            MGQ_CUDA(cudaFuncSetAttribute(cached_attention_kernel<128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tiles));
            MGQ_CUDA(cudaFuncSetAttribute(cached_attention_kernel<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tiles));
            opted_in[dev] = true;
        }
        return launch(small_group ? cached_attention_kernel<128, 4> : cached_attention_kernel<128, 8>, grid, dim3(128), tiles, st, q, k_cache,
                      v_cache, kv_pos, out, num_heads, num_kv_heads, max_seq, partials, counters);
    }
    return fail(MGQ_ERR_SHAPE, "attention: head_dim %u (64 and 128 are built)", head_dim);
}

size_t argmax_workspace_bytes() { return 256 + 2 * 256 * sizeof(float); }

int launch_argmax(const float *logits, uint32_t n, void *workspace, uint32_t *out_token, uint32_t *next_token, uint32_t *kv_pos,
                  uint32_t *history, uint32_t history_cap, void *stream)
{
    if (!workspace) return fail(MGQ_ERR_NULL, "argmax needs its workspace");
    unsigned int *counter = static_cast<unsigned int *>(workspace);
    float *part_val = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + 256);
    uint32_t *part_idx = reinterpret_cast<uint32_t *>(part_val + 256);
    uint32_t grid = (n + 256 * 8 - 1) / (256 * 8);
    if (grid > 256) grid = 256;
    if (grid < 1) grid = 1;
    return launch(argmax_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), logits, n, part_val, part_idx, counter,
                  out_token, next_token, kv_pos, history, history_cap);
}

}  // namespace mgq
