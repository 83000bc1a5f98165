// C ABI entry points that touch the device: buffers, argument checking and kernel routing.
#include <cuda_runtime.h>

#include <cstring>

#include "mgq_internal.h"

namespace mgq {

int cuda_check(int cuda_err, const char *what, const char *file, int line)
{
    if (cuda_err == (int)cudaSuccess) return MGQ_OK;
    return fail(MGQ_ERR_CUDA, "%s failed at %s:%d: %s", what, file, line,
                cudaGetErrorString(static_cast<cudaError_t>(cuda_err)));
}

static int check_matmul_args(int fmt, const void *a, const void *w, const float *c, uint32_t m, uint32_t k, uint32_t n)
{
    if (!a || !w || !c) return fail(MGQ_ERR_NULL, "null operand pointer");
    if (!is_quant(fmt)) return fail(MGQ_ERR_FORMAT, "weight format %d is not handled (only Q4=%d, Q8=%d)", fmt, MGQ_FMT_Q4, MGQ_FMT_Q8);
    if (m == 0 || k == 0 || n == 0) return fail(MGQ_ERR_SHAPE, "empty matmul %ux%ux%u", m, k, n);
    if (k % 32 != 0) return fail(MGQ_ERR_SHAPE, "K must be a multiple of 32 (quantization block), got %u", k);
    if (reinterpret_cast<uintptr_t>(w) % 16 != 0) return fail(MGQ_ERR_ALIGN, "packed weight pointer must be 16-byte aligned");
    return MGQ_OK;
}

}  // namespace mgq

using namespace mgq;

extern "C" {

int mgq_buffer_create(size_t bytes, void **out_dev)
{
    if (!out_dev) return fail(MGQ_ERR_NULL, "null out pointer");
    *out_dev = nullptr;
    if (bytes == 0) return fail(MGQ_ERR_SHAPE, "zero-sized buffer");
    void *p = nullptr;
    MGQ_CUDA(cudaMalloc(&p, bytes));
    const int rc = cuda_check((int)cudaMemset(p, 0, bytes), "cudaMemset", __FILE__, __LINE__);
    if (rc != MGQ_OK) { cudaFree(p); return rc; }
    *out_dev = p;
    return MGQ_OK;
}

int mgq_buffer_destroy(void *dev)
{
    if (!dev) return MGQ_OK;
    MGQ_CUDA(cudaFree(dev));
    return MGQ_OK;
}

int mgq_buffer_upload(void *dev, const void *host, size_t bytes, void *stream)
{
    if (!dev || !host) return fail(MGQ_ERR_NULL, "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MGQ_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, s));
    MGQ_CUDA(cudaStreamSynchronize(s));          // the reference's upload is synchronous
    return MGQ_OK;
}

int mgq_buffer_download(const void *dev, void *host, size_t bytes, void *stream)
{
    if (!dev || !host) return fail(MGQ_ERR_NULL, "null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MGQ_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, s));
    MGQ_CUDA(cudaStreamSynchronize(s));
    return MGQ_OK;
}

int mgq_set_option(const char *name, long value)
{
    if (!name) return fail(MGQ_ERR_NULL, "null option name");
    if (!std::strncmp(name, "plan.", 5)) return set_plan_option(name, value);
    if (!std::strncmp(name, "gemm.", 5)) return set_gemm_option(name, value);
    if (!std::strncmp(name, "session.", 8)) return set_session_option(name, value);
    return set_gemv_option(name, value);
}

int mgq_device_status(void) { return tc_device_status(); }

int mgq_gemv(int fmt, const float *x, const void *w, const float *addend, float *y,
             uint32_t m, uint32_t k, uint32_t n, void *stream)
{
    if (int rc = check_matmul_args(fmt, x, w, y, m, k, n)) return rc;
    if (m > MGQ_GEMV_MAX_M) return fail(MGQ_ERR_SHAPE, "gemv takes at most %d rows, got %u", MGQ_GEMV_MAX_M, m);
    return launch_gemv(fmt, x, w, addend, y, m, k, n, stream);
}

// ---- decode-step operators: argument checks, then the launchers of mgq_decode_ops.cu
int mgq_embedding(const uint32_t *ids, const float *table, float *out, uint32_t seq, uint32_t hidden, uint32_t vocab, void *stream)
{
    if (!ids || !table || !out) return fail(MGQ_ERR_NULL, "embedding: null pointer");
    if (seq == 0 || hidden == 0 || vocab == 0) return fail(MGQ_ERR_SHAPE, "embedding: empty shape");
    return launch_embedding(ids, table, out, seq, hidden, vocab, stream);
}

int mgq_rms_norm(const float *x, const float *weight, float *out, uint32_t rows, uint32_t cols, float eps, void *stream)
{
    if (!x || !weight || !out) return fail(MGQ_ERR_NULL, "rms_norm: null pointer");
    if (rows == 0 || cols == 0) return fail(MGQ_ERR_SHAPE, "rms_norm: empty shape");
    return launch_rms_norm(x, weight, out, rows, cols, eps, stream);
}

int mgq_rope_dynamic(const float *x, float *out, const uint32_t *pos_offset, uint32_t seq, uint32_t dim, uint32_t head_dim,
                     float theta, void *stream)
{
    if (!x || !out || !pos_offset) return fail(MGQ_ERR_NULL, "rope: null pointer");
    if (seq == 0 || dim == 0 || head_dim == 0) return fail(MGQ_ERR_SHAPE, "rope: empty shape");
    return launch_rope(x, out, pos_offset, seq, dim, head_dim, theta, stream);
}

int mgq_rope_cache_write(const float *q_src, float *q_dst, const float *k_src, float *k_dst, const float *v_src, float *k_cache,
                         float *v_cache, const uint32_t *kv_pos, uint32_t q_dim, uint32_t kv_dim, uint32_t head_dim, float theta,
                         uint32_t max_seq, void *stream)
{
    if (!q_src || !q_dst || !k_src || !k_dst || !v_src || !k_cache || !v_cache || !kv_pos) return fail(MGQ_ERR_NULL, "rope_cache_write: null pointer");
    if (q_dim == 0 || kv_dim == 0 || head_dim == 0 || max_seq == 0) return fail(MGQ_ERR_SHAPE, "rope_cache_write: empty shape");
    return launch_rope_cache(q_src, q_dst, k_src, k_dst, v_src, k_cache, v_cache, kv_pos, q_dim, kv_dim, head_dim, theta, max_seq, stream);
}

int mgq_cache_write(const float *src, float *cache, const uint32_t *kv_pos, uint32_t dim, uint32_t max_seq, void *stream)
{
    if (!src || !cache || !kv_pos) return fail(MGQ_ERR_NULL, "cache_write: null pointer");
    if (dim == 0 || max_seq == 0) return fail(MGQ_ERR_SHAPE, "cache_write: empty shape");
    return launch_cache_write(src, cache, kv_pos, dim, max_seq, stream);
}

int mgq_swiglu(const float *gate, const float *up, float *out, uint32_t rows, uint32_t half_n, uint32_t pitch, void *stream)
{
    if (!gate || !up || !out) return fail(MGQ_ERR_NULL, "swiglu: null pointer");
    if (rows == 0 || half_n == 0 || pitch < half_n) return fail(MGQ_ERR_SHAPE, "swiglu: bad shape");
    return launch_swiglu(gate, up, out, rows, half_n, pitch, stream);
}

size_t mgq_cached_attention_workspace(uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq)
{
    return attention_workspace_bytes(num_kv_heads, head_dim, max_seq);
}

int mgq_cached_attention(const float *q, const float *k_cache, const float *v_cache, const uint32_t *kv_pos, float *out,
                         uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq, void *workspace,
                         void *stream)
{
    if (!q || !k_cache || !v_cache || !kv_pos || !out) return fail(MGQ_ERR_NULL, "cached_attention: null pointer");
    if (max_seq == 0) return fail(MGQ_ERR_SHAPE, "cached_attention: empty cache");
    return launch_cached_attention(q, k_cache, v_cache, kv_pos, out, num_heads, num_kv_heads, head_dim, max_seq, workspace, stream);
}

size_t mgq_argmax_workspace(void) { return argmax_workspace_bytes(); }

int mgq_argmax(const float *logits, uint32_t n, void *workspace, uint32_t *out_token, uint32_t *next_token, uint32_t *kv_pos,
               uint32_t *history, uint32_t history_cap, void *stream)
{
    if (!logits || !out_token) return fail(MGQ_ERR_NULL, "argmax: null pointer");
    if (n == 0) return fail(MGQ_ERR_SHAPE, "argmax: empty vector");
    return launch_argmax(logits, n, workspace, out_token, next_token, kv_pos, history, history_cap, stream);
}

int mgq_gemv_f16(const float *x, const void *w_f16, const float *addend, float *y, uint32_t m, uint32_t k, uint32_t n, void *stream)
{
    if (!x || !w_f16 || !y) return fail(MGQ_ERR_NULL, "null operand pointer");
    if (m == 0 || k == 0 || n == 0) return fail(MGQ_ERR_SHAPE, "empty matmul %ux%ux%u", m, k, n);
    if (m > MGQ_GEMV_MAX_M) return fail(MGQ_ERR_SHAPE, "gemv takes at most %d rows, got %u", MGQ_GEMV_MAX_M, m);
    return launch_gemv_f16(x, w_f16, addend, y, m, k, n, stream);
}

int mgq_gemv_bt(const float *x, const float *b, float *y, uint32_t k, uint32_t n, void *stream)
{
    if (!x || !b || !y) return fail(MGQ_ERR_NULL, "null operand pointer");
    if (k == 0 || n == 0 || k % 4 != 0) return fail(MGQ_ERR_SHAPE, "gemv_bt: K=%u must be a positive multiple of 4 (N=%u)", k, n);
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(b) % 16 != 0)
        return fail(MGQ_ERR_ALIGN, "gemv_bt: activations and weights must be 16-byte aligned");
    return launch_gemv_bt(x, b, y, k, n, stream);
}

int mgq_gemv_exchange(int fmt, const float *x, const void *w, const float *addend, float *y, uint32_t k, uint32_t n,
                      const mgq_exchange_push *push_dev, const mgq_exchange_elem *wait_vec,
                      const unsigned long long *epoch, unsigned int *error, void *stream)
{
    if (!x && !wait_vec) return fail(MGQ_ERR_NULL, "x may only be null when the gathered vector is consumed (wait_vec)");
    if (int rc = check_matmul_args(fmt, x ? static_cast<const void *>(x) : static_cast<const void *>(wait_vec), w, y, 1, k, n)) return rc;
    if (!epoch || !error) return fail(MGQ_ERR_NULL, "exchange needs the epoch and error words");
    if (reinterpret_cast<uintptr_t>(wait_vec) % 16 != 0) return fail(MGQ_ERR_ALIGN, "the gathered vector must be 16-byte aligned");
    GemvExchange xc{push_dev, wait_vec, epoch, error};
    return launch_gemv(fmt, x, w, addend, y, 1, k, n, stream, &xc);
}

int mgq_exchange_finish(const mgq_exchange_elem *last_vec, uint32_t length, unsigned long long *epoch,
                        unsigned int *error, unsigned int *blocks_done, void *stream)
{
    if (!epoch || !error || !blocks_done) return fail(MGQ_ERR_NULL, "exchange needs the epoch, error and blocks_done words");
    return launch_exchange_finish(last_vec, length, epoch, error, blocks_done, stream);
}

int mgq_exchange_all_gather_rows(const float *slice, uint32_t slice_pitch, uint32_t rows, uint32_t cols, uint32_t world,
                                 const mgq_exchange_push *push_dev, const mgq_exchange_elem *local_vec, float *out,
                                 const unsigned long long *epoch, unsigned int *error, void *stream)
{
    if (!local_vec || !epoch || !error) return fail(MGQ_ERR_NULL, "all_gather needs the local gathered vector and the epoch and error words");
    if (!out && !slice) return fail(MGQ_ERR_NULL, "all_gather: nothing to store and nothing to wait for");
    if (slice && !push_dev) return fail(MGQ_ERR_NULL, "all_gather: a slice to push needs its push record");
    if (rows == 0 || cols == 0 || world == 0 || world > MGQ_MAX_PEERS || (slice && slice_pitch < cols) ||
        (unsigned long long)rows * cols * world >= (1ull << 31))
        return fail(MGQ_ERR_SHAPE, "all_gather: bad shape (rows %u, cols %u, pitch %u, world %u)", rows, cols, slice_pitch, world);
    if (reinterpret_cast<uintptr_t>(local_vec) % 8 != 0) return fail(MGQ_ERR_ALIGN, "the gathered vector must be 8-byte aligned");
    return launch_all_gather(slice, push_dev, local_vec, out, rows, cols, slice_pitch, world, epoch, error, stream);
}

int mgq_exchange_all_gather(const float *slice, const mgq_exchange_push *push_dev, const mgq_exchange_elem *local_vec, float *out,
                            uint32_t slice_len, uint32_t total, const unsigned long long *epoch, unsigned int *error, void *stream)
{
    if (slice_len == 0 || total % slice_len != 0) return fail(MGQ_ERR_SHAPE, "all_gather: bad lengths (slice %u, total %u)", slice_len, total);
    return mgq_exchange_all_gather_rows(slice, slice_len, 1, slice_len, total / slice_len, push_dev, local_vec, out, epoch, error, stream);
}

int mgq_gemm(int fmt, const void *a, int a_dtype, const void *w, const float *addend, float *c,
             uint32_t m, uint32_t k, uint32_t n, void *stream)
{
    if (int rc = check_matmul_args(fmt, a, w, c, m, k, n)) return rc;
    if (a_dtype != MGQ_A_F32 && a_dtype != MGQ_A_BF16) return fail(MGQ_ERR_FORMAT, "activation dtype %d is not f32/bf16", a_dtype);
    return launch_gemm(fmt, a, a_dtype, w, addend, c, m, k, n, stream);
}

int mgq_matmul(int fmt, const void *a, int a_dtype, const void *w, const float *addend, float *c,
               uint32_t m, uint32_t k, uint32_t n, void *stream)
{
    if (a_dtype == MGQ_A_F32 && m <= MGQ_GEMV_MAX_M)
        return mgq_gemv(fmt, static_cast<const float *>(a), w, addend, c, m, k, n, stream);
    return mgq_gemm(fmt, a, a_dtype, w, addend, c, m, k, n, stream);
}

int mgq_matmul_host(int fmt, const void *a_host, int a_dtype, const void *w_dev, const float *addend_host,
                    float *c_host, uint32_t m, uint32_t k, uint32_t n)
{
    if (int rc = check_matmul_args(fmt, a_host, w_dev, c_host, m, k, n)) return rc;
    if (a_dtype != MGQ_A_F32 && a_dtype != MGQ_A_BF16) return fail(MGQ_ERR_FORMAT, "activation dtype %d is not f32/bf16", a_dtype);
    const size_t a_bytes = (size_t)m * k * (a_dtype == MGQ_A_BF16 ? 2 : 4), c_bytes = (size_t)m * n * 4;
    void *a_dev = nullptr, *c_dev = nullptr, *d_dev = nullptr;
    int rc = MGQ_OK;
    auto cleanup = [&] { cudaFree(a_dev); cudaFree(c_dev); cudaFree(d_dev); };
    if ((rc = cuda_check((int)cudaMalloc(&a_dev, a_bytes), "cudaMalloc", __FILE__, __LINE__))) { cleanup(); return rc; }
    if ((rc = cuda_check((int)cudaMalloc(&c_dev, c_bytes), "cudaMalloc", __FILE__, __LINE__))) { cleanup(); return rc; }
    if (addend_host && (rc = cuda_check((int)cudaMalloc(&d_dev, c_bytes), "cudaMalloc", __FILE__, __LINE__))) { cleanup(); return rc; }
    rc = cuda_check((int)cudaMemcpyAsync(a_dev, a_host, a_bytes, cudaMemcpyHostToDevice, 0), "H2D", __FILE__, __LINE__);
    if (!rc && addend_host)
        rc = cuda_check((int)cudaMemcpyAsync(d_dev, addend_host, c_bytes, cudaMemcpyHostToDevice, 0), "H2D", __FILE__, __LINE__);
    if (!rc) rc = mgq_matmul(fmt, a_dev, a_dtype, w_dev, static_cast<const float *>(d_dev), static_cast<float *>(c_dev), m, k, n, nullptr);
    if (!rc) rc = cuda_check((int)cudaMemcpyAsync(c_host, c_dev, c_bytes, cudaMemcpyDeviceToHost, 0), "D2H", __FILE__, __LINE__);
    if (!rc) rc = cuda_check((int)cudaStreamSynchronize(0), "sync", __FILE__, __LINE__);
    cleanup();
    return rc;
}

}  // extern "C"
