// Internal helpers shared by the libmgq translation units (not part of the C ABI).
#pragma once
#include <cstdarg>
#include <cstddef>
#include <cstdint>

#include "../../include/mgq.h"

namespace mgq {

// Records a printf-style message for mgq_last_error() on this thread and returns `code`.
int fail(int code, const char *fmt, ...);

// cudaError_t -> status; records file/line and the CUDA error string on failure.
int cuda_check(int cuda_err, const char *what, const char *file, int line);

inline bool is_quant(int fmt) { return fmt == MGQ_FMT_Q4 || fmt == MGQ_FMT_Q8; }

// Multi-GPU exchange arguments of one GEMV launch (device pointers; see mgq_gemv_exchange).
struct GemvExchange {
    const void *push_dev;                     // mgq_exchange_push in device memory, or null
    const void *wait_vec;                     // gathered {value, stamp} vector this GEMV consumes, or null
    const unsigned long long *epoch;
    unsigned int *error;
};

// Launchers implemented in the .cu files (all pointers are device pointers).
int launch_gemv(int fmt, const float *x, const void *w, const float *addend, float *y,
                uint32_t m, uint32_t k, uint32_t n, void *stream, const GemvExchange *xchg = nullptr);
// Tensor-core (mma, int8 digit planes) GEMV for 3..16 rows (mgq_gemv_mma.cu).
bool gemv_mma_eligible(uint32_t m, uint32_t k, uint32_t n, const void *x, const void *w);
int launch_gemv_mma(int fmt, const float *x, const void *w, const float *addend, float *y,
                    uint32_t m, uint32_t k, uint32_t n, void *stream);
// f16-weight GEMV (mgq_gemv_f16.cu).
int launch_gemv_f16(const float *x, const void *w, const float *addend, float *y, uint32_t m, uint32_t k, uint32_t n, void *stream);
int launch_gemv_bt(const float *x, const float *b, float *y, uint32_t k, uint32_t n, void *stream);
bool gemv_streamable(const void *x, uint32_t k, uint32_t n);   // the streaming kernels take this shape (else the generic kernel runs)
int launch_exchange_finish(const void *last_vec, uint32_t length, unsigned long long *epoch,
                           unsigned int *error, unsigned int *blocks_done, void *stream);
int launch_all_gather(const float *slice, const void *push_dev, const void *local_vec, float *out, uint32_t rows, uint32_t cols,
                      uint32_t pitch, uint32_t world, const unsigned long long *epoch, unsigned int *error, void *stream);
int set_gemv_option(const char *name, long value);
int set_plan_option(const char *name, long value);
int set_gemm_option(const char *name, long value);
int set_session_option(const char *name, long value);
bool force_tiled();
int launch_gemm(int fmt, const void *a, int a_dtype, const void *w, const float *addend, float *c,
                uint32_t m, uint32_t k, uint32_t n, void *stream);

// Tensor-core GEMM (mgq_gemm_tc.cu): bf16 activations, M >= 64, K % 128 == 0.
bool gemm_tc_eligible(int a_dtype, uint32_t m, uint32_t k, uint32_t n, const void *a);
int launch_gemm_tc(int fmt, const void *a, const void *w, const float *addend, float *c,
                   uint32_t m, uint32_t k, uint32_t n, void *stream);
int tc_device_status();

// Decode-step operators (mgq_decode_ops.cu).
int launch_embedding(const uint32_t *ids, const float *table, float *out, uint32_t seq, uint32_t hidden, uint32_t vocab, void *stream);
int launch_rms_norm(const float *x, const float *weight, float *out, uint32_t rows, uint32_t cols, float eps, void *stream);
int launch_rope(const float *x, float *out, const uint32_t *pos_offset, uint32_t seq, uint32_t dim, uint32_t head_dim, float theta,
                void *stream);
int launch_rope_cache(const float *q_src, float *q_dst, const float *k_src, float *k_dst, const float *v_src, float *k_cache,
                      float *v_cache, const uint32_t *pos, uint32_t q_dim, uint32_t kv_dim, uint32_t head_dim, float theta,
                      uint32_t max_seq, void *stream);
int launch_cache_write(const float *src, float *cache, const uint32_t *kv_pos, uint32_t dim, uint32_t max_seq, void *stream);
int launch_swiglu(const float *gate, const float *up, float *out, uint32_t rows, uint32_t half_n, uint32_t pitch, void *stream);
size_t attention_workspace_bytes(uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq);
int launch_cached_attention(const float *q, const float *k_cache, const float *v_cache, const uint32_t *kv_pos, float *out,
                            uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq, void *workspace,
                            void *stream);
size_t argmax_workspace_bytes();
int launch_argmax(const float *logits, uint32_t n, void *workspace, uint32_t *out_token, uint32_t *next_token, uint32_t *kv_pos,
                  uint32_t *history, uint32_t history_cap, void *stream);

}  // namespace mgq

#define MGQ_CUDA(expr)                                                                 \
    do {                                                                               \
        int _rc = ::mgq::cuda_check((int)(expr), #expr, __FILE__, __LINE__);           \
        if (_rc != MGQ_OK) return _rc;                                                 \
    } while (0)
