/*
 * mgq -- B200 (sm_100a) CUDA implementation of meganeura's Q4/Q8 dequantize-fused matmul.
 *
 * C ABI of libmgq.  Plain pointers and sizes only; no C++ or framework types.
 * Every function returns an mgq_status (0 = ok) unless stated; the message of the
 * last failure on the calling thread is available from mgq_last_error().
 * Nothing in this library falls back to the CPU: a call that needs a GPU and finds
 * none returns MGQ_ERR_CUDA.
 *
 * Each group cites the meganeura interface it stands in for (paths inside the
 * meganeura source tree).  Packed weight layouts are byte-for-byte the reference's:
 *
 *   Q8: 36 B per 32-element block: f16 scale, 2 zero bytes, 32 int8 codes;
 *       block index = n * (K/32) + k/32                       (src/codegen.rs:785-805)
 *   Q4: all block headers first (u32 = f16 d | f16 m << 16), then 16 nibble bytes per
 *       block (element 2j low nibble, 2j+1 high nibble); value = nibble * d + m
 *                                                            (src/codegen.rs:748-769)
 */
#ifndef MGQ_H
#define MGQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* WeightFormat, same order as meganeura's enum (src/compile.rs:6-13). */
#define MGQ_FMT_F32 0
#define MGQ_FMT_F16 1
#define MGQ_FMT_Q4  2
#define MGQ_FMT_Q8  3

/* Activation dtype of the A operand. */
#define MGQ_A_F32  0
#define MGQ_A_BF16 1

typedef enum mgq_status {
    MGQ_OK = 0,
    MGQ_ERR_NULL = 1,        /* a required pointer was null */
    MGQ_ERR_SHAPE = 2,       /* K % 32 != 0, zero-sized or out-of-range dimension (replaces the
                                reference's assert!, src/runtime.rs:2037-2040, 2145-2148) */
    MGQ_ERR_FORMAT = 3,      /* weight format or dtype not handled by this library */
    MGQ_ERR_CUDA = 4,        /* a CUDA runtime call failed (no device, launch error, ...) */
    MGQ_ERR_NAME = 5,        /* unknown parameter / input name (reference panics, src/runtime.rs:2492) */
    MGQ_ERR_SIZE = 6,        /* host slice length does not match the tensor */
    MGQ_ERR_ALIGN = 7,       /* device pointer not aligned as the kernel requires (16 B for weights) */
    MGQ_ERR_STATE = 8,       /* call not valid in the object's current state */
    MGQ_ERR_TIMEOUT = 9      /* a bounded device-side wait ran out */
} mgq_status;

const char *mgq_last_error(void);
const char *mgq_version(void);

/* Runtime options, the counterpart of meganeura's ad-hoc environment switches
 * (MEGANEURA_SERIAL_DISPATCH, src/runtime.rs:1703-1707).  0 means "automatic" for the tunables.
 *   "gemv.serial_dispatch"      1: every GEMV starts only after its predecessor has finished
 *                               (no programmatic dependent launch); also MGQ_SERIAL_DISPATCH=1
 *   "gemv.columns_per_thread"   1 or 2 columns per thread and pipeline stage
 *   "gemv.ctas_per_sm"          CTAs per SM a GEMV grid is sized for (default 3)
 *   "gemv.batch_mma"            1 (default): 3..16 rows run on the integer tensor-core kernel that reads
 *                               the weights once per 8 rows; 0: two rows at a time on the streaming kernels
 *   "gemv.wait_us"              time limit of the stamp polls of mgq_gemv_exchange / mgq_exchange_finish
 *                               (default 2000000: the other ranks' processes may launch seconds apart)
 *   "plan.window_tiles"         ring tiles the producer keeps in flight (default: about 64 KB per SM)
 *   "plan.dataflow"             how a plan made by mgq_plan_create hands activations from op to op: 0 (default)
 *                               plain vectors, the consumer waits for the producer's arrival counter; 1 the
 *                               {value, stamp} vectors that multi-GPU plans use, consumers wait per block
 *   "plan.deadline_us"          time limit of every wait inside the plan kernel (default 20000)
 *   "plan.peer_deadline_us"     the same for plans created with mgq_plan_create_linked, whose waits also
 *                               depend on other GPUs' host processes (default 2000000)
 *   "gemm.force_tiled"          1: never use the tcgen05 kernel (CUDA-core tiled kernel only)
 *   "session.horizontal_fusion" sessions built afterwards merge single-row matmuls that read the same
 *                               activation into one GEMV over the concatenated weight: 0 never,
 *                               1 gate|up under a SwiGLU only (the reference's rule,
 *                               src/optimize.rs:776-879), 2 every such group, e.g. q|k|v (default)
 *   "session.fuse_rope_cache"   1 (default): RoPE(q), RoPE(k), CacheWrite(k), CacheWrite(v) of a decode
 *                               layer run as one launch; 0: four dispatches like the reference
 *   "session.fuse_exchange"     1 (default): in a column-sharded session a single-row GEMV whose output
 *                               feeds an all_gather stores its columns into the ranks' gathered vectors
 *                               itself; 0: the all_gather does */
int mgq_set_option(const char *name, long value);

/* ---- format: TensorType::size_bytes for quantized dtypes (src/graph.rs:52-68) ---------- */
size_t mgq_packed_bytes(int fmt, size_t k, size_t n);

/* ---- host quantizers: quantize_q4_0 / dequantize_q4_0 / quantize_q8_0 / dequantize_q8_0
 *      (src/runtime.rs:2035-2215).  w and out are row-major [k, n] f32 on the host. ------- */
int mgq_quantize_q4(const float *w, size_t k, size_t n, uint8_t *out);
int mgq_quantize_q8(const float *w, size_t k, size_t n, uint8_t *out);
int mgq_dequantize_q4(const uint8_t *packed, size_t k, size_t n, float *out);
int mgq_dequantize_q8(const uint8_t *packed, size_t k, size_t n, float *out);

/* Columns [n0, n1) of a packed [k, n] weight as a self-contained packed [k, n1-n0] weight
 * (host memory).  No reference counterpart: the reference is single-device; a block never
 * spans columns (block = n*(K/32)+b, src/codegen.rs:753, 788), so a column range is itself a
 * valid weight.  out must hold mgq_packed_bytes(fmt, k, n1-n0). */
int mgq_shard_columns(int fmt, const uint8_t *packed, size_t k, size_t n, size_t n0, size_t n1, uint8_t *out);

/* ---- device buffers: Session buffer allocation (zero-filled, src/runtime.rs:1737-1755),
 *      upload_buffer (2552-2558) and read-back (2612-2629). ------------------------------- */
int mgq_buffer_create(size_t bytes, void **out_dev);
int mgq_buffer_destroy(void *dev);
int mgq_buffer_upload(void *dev, const void *host, size_t bytes, void *stream);
int mgq_buffer_download(const void *dev, void *host, size_t bytes, void *stream);

/* ---- kernels.  All pointers are device pointers; stream is a cudaStream_t (NULL = default).
 *
 * y[m,n] = x[m,k] . dequant(w)[k,n] (+ addend[m,n]),  f32 in, f32 accumulate, f32 out.
 * Stands in for the MatMulGemv / MatMulGemvAdd dispatches (src/compile.rs:1390-1406,
 * 1498-1509; bindings matrix_a, matrix_b, matrix_c[, src], params=[m,k,n,0]) with the
 * quantized weight semantics of dequant_q4 / dequant_q8.  The reference has no working
 * quantized GEMV (src/codegen.rs:1065-1073 falls back to the f32 shader), so the result is
 * defined by the tiled kernel's math.  1 <= m <= MGQ_GEMV_MAX_M; w must be 16-byte aligned. */
#define MGQ_GEMV_MAX_M 16
int mgq_gemv(int fmt, const float *x, const void *w, const float *addend, float *y,
             uint32_t m, uint32_t k, uint32_t n, void *stream);

/* GEMV over f16 weights (WeightFormat::F16): y = x . W (+ addend), W row-major [k, n] binary16 as
 * the reference stores parameter_f16 weights, f32 accumulation -- the reference's f16 variant of
 * matmul_gemv.wgsl (src/codegen.rs:1065-1101).  1 <= m <= MGQ_GEMV_MAX_M, n % 8 == 0, W 16-byte
 * aligned.  mgq_convert_f16 is the host conversion (round to nearest even, like half::f16::from_f32). */
int mgq_gemv_f16(const float *x, const void *w_f16, const float *addend, float *y, uint32_t m, uint32_t k, uint32_t n, void *stream);
int mgq_convert_f16(const float *src, size_t len, uint16_t *dst);
/* MatMulGemvBT (src/shaders/matmul_gemv_bt.wgsl:34-65; src/compile.rs:1447-1469): y[n] = sum_k x[k] * b[n, k]
 * with b an f32 [N, K] row-major matrix -- the lm_head of a model with tied embeddings, b being the
 * embedding table.  K % 4 == 0; x and b 16-byte aligned. */
int mgq_gemv_bt(const float *x, const float *b, float *y, uint32_t k, uint32_t n, void *stream);

/* ---- column-sharded GEMV with a fused all-gather over peer memory (no reference counterpart: the
 * reference is single-device, src/runtime.rs:1513-1531).
 *
 * Each rank runs the unchanged GEMV on its column slice.  With `push_dev` set, the lane that
 * finishes a column also stores it into every rank's copy of the gathered vector (plain peer
 * stores over NVLink into memory the caller made peer-accessible, e.g. CUDA IPC or symmetric
 * memory).  An element travels as one 8-byte {value, stamp} pair, stamp = *epoch + 1, written by a
 * single 64-bit store, so data and validity arrive together and no fence, counter or atomic is
 * needed.  With `wait_vec` set (the local gathered vector of length k that this GEMV consumes),
 * every thread first polls -- with a time limit ("gemv.wait_us"), after which *error is raised --
 * the stamps of the 32 elements of its block.  mgq_exchange_finish ends a token: it polls all `length` stamps
 * of the last gathered vector and then increments *epoch.  Stamps only grow; nothing is reset
 * between tokens, so a token can be replayed from a CUDA graph.  m = 1 only.
 * Reuse rule: a gathered vector may be pushed again (next token) only after every rank's consumers
 * of it have finished.  mgq_exchange_finish on one rank says nothing about the other ranks' readers;
 * a token of three or more exchanging ops satisfies the rule by construction (a rank can finish the
 * token only after every rank has pushed the last op, which each rank does after consuming all the
 * vectors before it); a shorter chain needs a host-side barrier between tokens.
 * x may be NULL when wait_vec is set: the GEMV then takes its activations from the gathered vector
 * itself (the values it has just found valid), which is how a sharded model chains its layers.  A
 * non-NULL x must be data of this GPU's own stream (it is read through the read-only cache). */
#define MGQ_MAX_PEERS 8
typedef struct mgq_exchange_elem { float value; uint32_t stamp; } mgq_exchange_elem;
typedef struct mgq_exchange_push {            /* must live in device memory */
    uint32_t world, rank;
    uint32_t gather_cols;                     /* leading columns of this rank's y that every rank needs */
    uint32_t reserved;
    mgq_exchange_elem *dst[MGQ_MAX_PEERS];    /* rank p's gathered vector; this rank fills [rank*gather_cols, +gather_cols) */
} mgq_exchange_push;

int mgq_gemv_exchange(int fmt, const float *x, const void *w, const float *addend, float *y, uint32_t k, uint32_t n,
                      const mgq_exchange_push *push_dev, const mgq_exchange_elem *wait_vec,
                      const unsigned long long *epoch, unsigned int *error, void *stream);
/* blocks_done: a zero-initialised word in local device memory (returns to zero). */
int mgq_exchange_finish(const mgq_exchange_elem *last_vec, uint32_t length, unsigned long long *epoch,
                        unsigned int *error, unsigned int *blocks_done, void *stream);

/* The same exchange for the operators between the GEMVs of a sharded model: stores `slice`
 * (slice_len plain floats: this rank's part, e.g. its heads' attention output) into every rank's
 * gathered vector as {value, stamp} elements -- with slice == NULL nothing is stored, because the
 * producing GEMV has pushed already -- then waits, bounded like mgq_gemv_exchange, until all `total`
 * elements of the local gathered vector carry this token's stamp and writes their values to `out`
 * as a plain vector; with out == NULL it only stores (the reader, a GEMV given the vector as its
 * wait_vec, waits itself).  The epoch is not changed (mgq_exchange_finish with last_vec == NULL adds one). */
int mgq_exchange_all_gather(const float *slice, const mgq_exchange_push *push_dev, const mgq_exchange_elem *local_vec, float *out,
                            uint32_t slice_len, uint32_t total, const unsigned long long *epoch, unsigned int *error, void *stream);
/* The same for several rows (a batch of tokens): this rank's slice is `rows` rows of `cols` columns,
 * `slice_pitch` floats apart (e.g. the leading columns of a wider GEMV output); the push record's
 * gather_cols is rows * cols; `out` is the whole row-major [rows, world * cols] matrix. */
int mgq_exchange_all_gather_rows(const float *slice, uint32_t slice_pitch, uint32_t rows, uint32_t cols, uint32_t world,
                                 const mgq_exchange_push *push_dev, const mgq_exchange_elem *local_vec, float *out,
                                 const unsigned long long *epoch, unsigned int *error, void *stream);

/* c[m,n] = a[m,k] . dequant(w)[k,n] (+ addend[m,n]); a is f32 or bf16 row-major, c is f32.
 * Stands in for the MatMul / FusedMatMulAdd dispatches with a quantized weight_format
 * (src/compile.rs:1408-1419, 1511-1522; src/shaders/matmul.wgsl:28-109).
 * bf16 activations with m >= 64 and k % 128 == 0 run on the tensor cores (tcgen05, TMEM
 * accumulator, TMA-fed activations, weights dequantized into bf16 hi+lo operand tiles); every
 * other case runs the register-tiled CUDA-core kernel. */
int mgq_gemm(int fmt, const void *a, int a_dtype, const void *w, const float *addend, float *c,
             uint32_t m, uint32_t k, uint32_t n, void *stream);

/* Reports (and clears) a device-side timeout: every wait inside the tensor-core GEMM is bounded and
 * raises a device error word when it runs out instead of hanging.  Synchronises the device. */
int mgq_device_status(void);

/* ---- the operators between the GEMVs of a decode step (all pointers are device pointers, f32
 * row-major; positions and token ids are u32 words in device memory, like the reference's
 * kv_pos_buf / token_ids inputs, so that a whole step is a fixed launch sequence).
 *
 * mgq_embedding:        out[r, :] = table[ids[r], :]                 src/shaders/embedding.wgsl
 * mgq_rms_norm:         out = x * rsqrt(mean(x^2) + eps) * weight     src/shaders/rms_norm.wgsl
 * mgq_rope_dynamic:     HF half-split RoPE per head, position = row + *pos_offset
 *                                                                    src/shaders/rope_dynamic.wgsl
 * mgq_cache_write:      cache[*kv_pos, :] = src[0, :]                 src/shaders/cache_write.wgsl
 * mgq_swiglu:           out = silu(gate) * up; gate/up are rows of `pitch` floats, so the
 *                       concatenated [rows, 2*half_n] form passes gate = in, up = in + half_n,
 *                       pitch = 2*half_n       src/shaders/swiglu_concat.wgsl, binary.wgsl (swiglu)
 * mgq_cached_attention: one query token over cache rows 0..*kv_pos, grouped-query heads, scale
 *                       1/sqrt(head_dim), softmax in f32; head_dim 64 or 128 (the reference's
 *                       shader is fixed at 64), at most 8 query heads per KV head, max_seq at
 *                       most 4096 rows (MGQ_ERR_SHAPE beyond; a session checks it when it is
 *                       built).  `workspace`
 *                       is mgq_cached_attention_workspace(...) bytes of zero-initialised device
 *                       memory owned by the caller (split-context partials and counters; it
 *                       returns to its initial state).  Calls that share a workspace must be
 *                       ordered on one stream.                       src/shaders/cached_attention.wgsl
 * mgq_argmax:           greedy pick on the device (the reference picks on the host,
 *                       bench/bench_meganeura.rs:255-273): *out_token = argmax(logits), lowest
 *                       index on ties; history[*kv_pos] = token when history != NULL; when
 *                       next_token != NULL the token is fed back (*next_token = token,
 *                       *kv_pos += 1) so that steps can be replayed without a host round trip.
 *                       `workspace`: mgq_argmax_workspace() bytes, zero-initialised. */
int mgq_embedding(const uint32_t *ids, const float *table, float *out, uint32_t seq, uint32_t hidden, uint32_t vocab, void *stream);
int mgq_rms_norm(const float *x, const float *weight, float *out, uint32_t rows, uint32_t cols, float eps, void *stream);
int mgq_rope_dynamic(const float *x, float *out, const uint32_t *pos_offset, uint32_t seq, uint32_t dim, uint32_t head_dim,
                     float theta, void *stream);
/* The four dispatches after a decode layer's q|k|v projection in one launch (no reference
 * counterpart as a single shader): q_dst = rope(q_src), k_dst = rope(k_src),
 * k_cache[*kv_pos] = k_dst, v_cache[*kv_pos] = v_src; q is [1, q_dim], k and v are [1, kv_dim]. */
int mgq_rope_cache_write(const float *q_src, float *q_dst, const float *k_src, float *k_dst, const float *v_src, float *k_cache,
                         float *v_cache, const uint32_t *kv_pos, uint32_t q_dim, uint32_t kv_dim, uint32_t head_dim, float theta,
                         uint32_t max_seq, void *stream);
int mgq_cache_write(const float *src, float *cache, const uint32_t *kv_pos, uint32_t dim, uint32_t max_seq, void *stream);
int mgq_swiglu(const float *gate, const float *up, float *out, uint32_t rows, uint32_t half_n, uint32_t pitch, void *stream);
size_t mgq_cached_attention_workspace(uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq);
int mgq_cached_attention(const float *q, const float *k_cache, const float *v_cache, const uint32_t *kv_pos, float *out,
                         uint32_t num_heads, uint32_t num_kv_heads, uint32_t head_dim, uint32_t max_seq, void *workspace,
                         void *stream);
size_t mgq_argmax_workspace(void);
int mgq_argmax(const float *logits, uint32_t n, void *workspace, uint32_t *out_token, uint32_t *next_token, uint32_t *kv_pos,
               uint32_t *history, uint32_t history_cap, void *stream);

/* Routing wrapper: mgq_gemv when m <= MGQ_GEMV_MAX_M (f32 activations), else mgq_gemm. */
int mgq_matmul(int fmt, const void *a, int a_dtype, const void *w, const float *addend, float *c,
               uint32_t m, uint32_t k, uint32_t n, void *stream);

/* Same contraction with HOST activations/outputs and a resident device weight: copies
 * a (and addend) to the device, runs mgq_matmul, copies c back and synchronises.  This is
 * the set_input -> step -> wait -> read_output round trip of a one-node session. */
int mgq_matmul_host(int fmt, const void *a_host, int a_dtype, const void *w_dev, const float *addend_host,
                    float *c_host, uint32_t m, uint32_t k, uint32_t n);

/* ---- plan kernel: a static list of single-row GEMVs run by ONE persistent cooperative launch
 * (one CTA per SM).  Stands in for Session::step replaying ExecutionPlan.dispatches in barrier
 * groups inside one submission (src/runtime.rs:2843-2959; barrier groups 1202-1256).  A producer
 * thread per CTA streams the packed weights of all ops through a shared-memory ring with bulk
 * copies and runs ahead across op boundaries; op i starts reading its activations only after
 * ops [0, wait_for) have completed (wait_for = 0: no dependency; wait_for = i: depends on the op
 * before it).  x is read as a plain vector once every CTA has counted itself out of op
 * wait_for - 1 (arrival counters in global memory).  With "plan.dataflow" = 1, an x that is a range
 * of the output y of an earlier op that is waited for travels instead as {value, stamp} elements of a
 * vector the plan owns and the consumer waits per 32-element block, which is what plans over several
 * GPUs do (mgq_plan_create_linked).  y always receives the plain result.  An addend must be complete before the op that produces this op's activations starts.
 * All pointers are device pointers and must stay valid for the plan's lifetime.
 * Limits: at most MGQ_PLAN_MAX_OPS ops (MGQ_ERR_SIZE beyond: split the list), m = 1, 256 <= K <= 12288, K*N/32 a multiple of 4, 16-byte aligned w and x.  Launches of one plan must not overlap.  Every device-side wait
 * has a time limit ("plan.deadline_us", default 20 ms), after which the launch finishes with
 * undefined results, publishes nothing more to consumers, and mgq_plan_check reports
 * MGQ_ERR_TIMEOUT. */
#define MGQ_PLAN_MAX_OPS 152                 /* ops per plan (their descriptors are kept in shared memory) */
typedef struct mgq_plan mgq_plan;
typedef struct mgq_plan_op {
    int fmt;                 /* MGQ_FMT_Q4 / MGQ_FMT_Q8 */
    const float *x;          /* [1, k] */
    const void *w;           /* packed [k, n] */
    const float *addend;     /* [1, n] or NULL */
    float *y;                /* [1, n] */
    uint32_t m, k, n;
    uint32_t wait_for;       /* number of leading ops that must be complete before this one starts */
} mgq_plan_op;

int mgq_plan_create(const mgq_plan_op *ops, size_t count, mgq_plan **out);
/* Enqueues the whole list as one kernel on `stream` (capturable in a CUDA graph). */
int mgq_plan_launch(mgq_plan *plan, void *stream);
/* Synchronises `stream` and returns MGQ_ERR_TIMEOUT if a wait of an earlier launch gave up
 * (results of such a launch are undefined; the plan is rearmed). */
int mgq_plan_check(mgq_plan *plan, void *stream);
int mgq_plan_info(const mgq_plan *plan, uint32_t *grid, uint32_t *threads, uint32_t *ring_slots, size_t *smem_bytes);
void mgq_plan_destroy(mgq_plan *plan);

/* The same kernel with caller-owned gathered vectors: the column-sharded multi-GPU decode step as
 * one launch per rank (no reference counterpart, like mgq_gemv_exchange whose protocol it uses).
 * links[i].push_dev (device memory, may be NULL): op i also stores its leading gather_cols columns
 * as {value, stamp} elements into every listed rank's vector, with plain stores over NVLink.
 * links[i].wait_vec (may be NULL): op i takes its k activations from this LOCAL gathered vector,
 * waiting per block for this token's stamps; x and wait_for of the op are then ignored.
 * `epoch` is the token index (stamp = *epoch + 1) and `error` the timeout flag, both in local
 * device memory; the launch adds one to *epoch when it ends.  With final_vec set the launch also
 * waits until all final_len elements of that local vector (normally the last op's) carry this
 * token's stamp, so that the host may read it after the launch.  A gathered vector may be written
 * again only after every rank has consumed it: chains of three or more linked ops satisfy this by
 * construction, because a rank can start the next token only after every rank has contributed to
 * the last ops of this one. */
typedef struct mgq_plan_link {
    const mgq_exchange_push *push_dev;
    const mgq_exchange_elem *wait_vec;
} mgq_plan_link;
int mgq_plan_create_linked(const mgq_plan_op *ops, const mgq_plan_link *links, size_t count, unsigned long long *epoch,
                           unsigned int *error, const mgq_exchange_elem *final_vec, uint32_t final_len, mgq_plan **out);

/* Allocation-free variant of the plan kernel.  No counterpart in meganeura: the reference's
 * session allocates all its buffers when it is built and has no second, allocation-free way to run.
 *
 * Runs `count` single-row GEMVs (same op rules as mgq_plan_create) as one persistent kernel on
 * `stream` and returns when they have finished (it synchronises the stream; MGQ_ERR_TIMEOUT if a
 * wait gave up).  It never calls cudaMalloc/cudaFree or any allocating routine: the kernel's
 * scratch -- op descriptors, arrival counters, token index, error word -- is a fixed device array
 * of MGQ_STATIC_PLAN_MAX_OPS entries (about 18 KB) that every GPU using the library holds until
 * the process exits; dependent ops wait on the arrival counters (no gathered vectors).  It is meant for callers that must not allocate on their execution path, e.g. a
 * serving loop with a fixed device-memory budget or a host application that forbids cudaMalloc after
 * start-up (it can synchronise the device and can fail when memory is tight).
 *
 *   - count > MGQ_STATIC_PLAN_MAX_OPS is rejected with MGQ_ERR_SIZE.
 *   - The first call on each device looks up the array's device address and opts the kernels into
 *     their shared-memory size; make that first call before starting any stream capture.
 *   - The call copies the descriptors in, launches, reads the error word back and synchronises
 *     `stream`, so it cannot itself be part of a stream capture (MGQ_ERR_STATE on a capturing
 *     stream), and `stream` must belong to the device that is current on the calling thread.
 *   - All calls on a device share the one array, and it keeps the previous call's contents; the
 *     entry point rewrites the descriptors and zeroes the counters itself, but two calls that
 *     overlap on the same GPU (different streams or threads) race on it. */
#define MGQ_STATIC_PLAN_MAX_OPS 128
int mgq_plan_run_static(const mgq_plan_op *ops, size_t count, void *stream);

/* ---- Graph / Session surface (src/graph.rs:714-795, src/train.rs:380-389,
 *      src/runtime.rs:2327-2345, 2496-2550, 2612-2643, 2786-2791, 2835-2959).
 *
 * The nodes of the quantized-matmul path and of a decode step exist: inputs, parameters (matmul
 * weights must be Q4, Q8 or f16; f32 parameters are addends, norm weights, tables and caches),
 * matmul, add and the decode-step operators below.  MatMul+Add is fused to FusedMatMulAdd like
 * apply_matmul_add_fusions (src/optimize.rs:724-767) and the plan's dispatches carry the
 * reference's shader names, workgroups, params and labels. */
typedef struct mgq_graph mgq_graph;
typedef struct mgq_session mgq_session;

/* ShaderEntry values used by plan dispatches (names as in src/compile.rs). */
#define MGQ_SHADER_MATMUL            0
#define MGQ_SHADER_FUSED_MATMUL_ADD  1
#define MGQ_SHADER_MATMUL_GEMV       2
#define MGQ_SHADER_MATMUL_GEMV_ADD   3
#define MGQ_SHADER_ADD               4
#define MGQ_SHADER_EMBEDDING         5
#define MGQ_SHADER_RMS_NORM          6
#define MGQ_SHADER_ROPE_DYNAMIC      7
#define MGQ_SHADER_CACHE_WRITE       8
#define MGQ_SHADER_CACHED_ATTENTION  9
#define MGQ_SHADER_SWIGLU            10
#define MGQ_SHADER_SWIGLU_CONCAT     11
#define MGQ_SHADER_ROPE_CACHE_WRITE  12   /* RoPEDynamic x2 + CacheWrite x2 merged (no reference entry) */
#define MGQ_SHADER_ALL_GATHER        13   /* column-sharded sessions: slice -> whole vector over peer memory (no reference entry) */
#define MGQ_SHADER_MATMUL_GEMV_BT    14

mgq_graph *mgq_graph_new(void);
void mgq_graph_free(mgq_graph *g);
/* Each builder returns the new node id (>= 0) or -status. */
int mgq_graph_input(mgq_graph *g, const char *name, const size_t *shape, size_t rank);
int mgq_graph_parameter(mgq_graph *g, const char *name, const size_t *shape, size_t rank);
int mgq_graph_parameter_q4(mgq_graph *g, const char *name, const size_t *shape, size_t rank);
int mgq_graph_parameter_q8(mgq_graph *g, const char *name, const size_t *shape, size_t rank);
/* Graph::parameter_f16 (src/graph.rs:739-748): a [K, N] weight kept as row-major binary16; usable as the
 * right operand of a matmul with at most MGQ_GEMV_MAX_M rows and N % 8 == 0. */
int mgq_graph_parameter_f16(mgq_graph *g, const char *name, const size_t *shape, size_t rank);
int mgq_graph_matmul(mgq_graph *g, int a, int b);
/* Graph::matmul_bt (src/graph.rs:809-817): a [M, K] times the transpose of an f32 parameter b [N, K].
 * Only the single-row form (MatMulGemvBT) is lowered; m > 1 is refused when the session is built. */
int mgq_graph_matmul_bt(mgq_graph *g, int a, int b);
int mgq_graph_add(mgq_graph *g, int a, int b);
/* decode-step nodes: Graph::{input_u32, embedding, rms_norm, rope_dynamic_offset, cache_write,
 * cached_attention, swiglu, swiglu_concat} (src/graph.rs:1003-1009, 1029-1040, 1062-1087, 1148-1170,
 * 1659-1700), same argument checks; a cache is an f32 parameter [max_seq, kv_dim] written in place. */
int mgq_graph_input_u32(mgq_graph *g, const char *name, const size_t *shape, size_t rank);
int mgq_graph_embedding(mgq_graph *g, int indices, int table);
int mgq_graph_rms_norm(mgq_graph *g, int x, int weight, float eps);
int mgq_graph_rope_dynamic_offset(mgq_graph *g, int x, float theta, int offset_input, uint32_t head_dim);
int mgq_graph_cache_write(mgq_graph *g, int new_kv, int cache, int kv_pos);
int mgq_graph_cached_attention(mgq_graph *g, int q, int k_cache, int v_cache, int kv_pos, uint32_t num_heads,
                               uint32_t num_kv_heads, uint32_t head_dim);
int mgq_graph_swiglu(mgq_graph *g, int gate, int up);
int mgq_graph_swiglu_concat(mgq_graph *g, int input);
/* No reference counterpart (the reference is single-device): x is this rank's [1, n] slice of a
 * vector that every rank needs whole; the node is the [1, n * world] vector, rank-major.  A graph
 * that holds such nodes is one rank's part of a column-sharded model: its weights are this rank's
 * column slices, its attention works on this rank's heads, and every all_gather must be bound to
 * peer-visible memory (mgq_session_bind_exchange) before the first step. */
int mgq_graph_all_gather(mgq_graph *g, int x, uint32_t world);
/* Columns [first, first + count) of a [1, n] f32 node, without a copy (first % 4 == 0): the part of
 * a whole vector that belongs to this rank, e.g. the residual a sharded projection adds to. */
int mgq_graph_slice_columns(mgq_graph *g, int x, uint32_t first, uint32_t count);
int mgq_graph_set_outputs(mgq_graph *g, const int *ids, size_t count);

/* build_inference_session (src/train.rs:380-389): fuse, lower, allocate zero-filled buffers. */
int mgq_build_inference_session(const mgq_graph *g, mgq_session **out);
void mgq_session_free(mgq_session *s);
/* set_parameter quantizes f32 data on the host for Q4/Q8 parameters (src/runtime.rs:2327-2345). */
int mgq_session_set_parameter(mgq_session *s, const char *name, const float *data, size_t len);
/* upload_param: raw bytes into the parameter buffer, no conversion (src/runtime.rs:2786-2791). */
int mgq_session_upload_param(mgq_session *s, const char *name, const void *bytes, size_t nbytes);
int mgq_session_set_input(mgq_session *s, const char *name, const float *data, size_t len);
/* Session::save_checkpoint / load_checkpoint (src/runtime.rs:4205-4336), same file layout: a
 * safetensors file with every parameter buffer -- packed Q4/Q8 bytes as they are -- stored as a flat
 * F32 tensor of byte_len/4 elements under the parameter's name, metadata adam_step.  A file written
 * by either side loads on the other when parameter names and shapes agree; loading skips
 * re-quantization.  Parameters missing from the file keep their contents. */
int mgq_session_save_checkpoint(mgq_session *s, const char *path);
int mgq_session_load_checkpoint(mgq_session *s, const char *path);
int mgq_session_set_input_u32(mgq_session *s, const char *name, const uint32_t *data, size_t len);
int mgq_session_step(mgq_session *s);
/* No reference counterpart (the reference re-records its command buffer every step,
 * src/runtime.rs:2843-2881): captures the dispatch list once into a CUDA graph; later steps replay
 * it.  Needs one ordinary step first.  Inputs and parameters may still be rewritten between steps
 * (their buffers do not move). */
int mgq_session_capture(mgq_session *s);
/* No reference counterpart (the reference picks the next token on the host,
 * bench/bench_meganeura.rs:255-273): after the dispatches of every step, pick argmax of output
 * `output_index` on the device, store it at history[position], write it into the u32 input
 * `token_input` and add one to the u32 input `pos_input`.  Call before mgq_session_capture.
 * mgq_session_read_tokens copies history[first_pos, first_pos + count) to the host. */
int mgq_session_enable_greedy(mgq_session *s, size_t output_index, const char *token_input, const char *pos_input,
                              uint32_t history_cap);
int mgq_session_read_tokens(mgq_session *s, uint32_t first_pos, uint32_t *out, size_t count);
int mgq_session_wait(mgq_session *s);
int mgq_session_read_output(mgq_session *s, float *out, size_t len);
int mgq_session_read_output_by_index(mgq_session *s, size_t index, float *out, size_t len);
/* plan() inspection (tests/gemv_parity.rs:32-52 reads dispatches[i].shader). */
int mgq_session_num_dispatches(const mgq_session *s);
int mgq_session_dispatch_info(const mgq_session *s, size_t index, int *shader, uint32_t workgroups[3],
                              uint32_t params[4], int *weight_format, char *label, size_t label_cap);
/* Number of kernels launched by this session so far. */
uint64_t mgq_session_launch_count(const mgq_session *s);

/* Session::set_profiling / dump_gpu_timings / num_groups (src/runtime.rs:1965-1967, 2798-2832,
 * 4192-4199).  With profiling on, step() runs every dispatch on its own between CUDA events (and
 * inside an NVTX range named by the dispatch label; step and wait are NVTX ranges "step" / "wait"
 * like the reference's spans) instead of replaying the captured graph.  mgq_session_gpu_timings
 * copies the microseconds of each dispatch of the last profiled step (count must equal the number
 * of dispatches); mgq_session_dump_gpu_timings writes the reference's report -- totals per pass
 * name, largest first -- as text into `out`.  Both synchronise the session's stream.
 * mgq_session_num_groups is the number of barrier groups of the plan: the reference's
 * reorder_by_level + compute_groups (src/runtime.rs:1202-1256), available on plain buffer-id lists
 * as mgq_barrier_groups (four input and four output ids per dispatch, -1 for none; reorder != 0
 * sorts by dependency level first, as the reference does when it builds a session). */
/* Column-sharded sessions.  mgq_session_num_exchanges counts the all_gather nodes (in execution
 * order); mgq_session_exchange_info gives the floats this rank contributes and the number of ranks.
 * mgq_session_bind_exchange hands exchange `index` its push record (device memory, gather_cols ==
 * slice length) and this rank's gathered vector of slice_len * world elements, which every rank must
 * be able to store into (symmetric or IPC memory).  mgq_session_bind_exchange_state gives the token
 * index, the error word and a zeroed scratch word, all in local device memory; every rank must have
 * made the same number of steps.  A single-row GEMV that feeds an all_gather pushes its columns
 * itself ("session.fuse_exchange", default 1).  Every step ends by adding one to the token index.
 * mgq_session_check_exchange synchronises the stream and returns MGQ_ERR_TIMEOUT if a bounded wait
 * of an earlier step ran out (the word is cleared). */
int mgq_session_num_exchanges(const mgq_session *s);
int mgq_session_exchange_info(const mgq_session *s, size_t index, uint32_t *slice_len, uint32_t *world);
int mgq_session_bind_exchange(mgq_session *s, size_t index, const mgq_exchange_push *push_dev, mgq_exchange_elem *local_vec);
int mgq_session_bind_exchange_state(mgq_session *s, unsigned long long *epoch, unsigned int *error, unsigned int *blocks_done);
int mgq_session_check_exchange(mgq_session *s);

int mgq_session_set_profiling(mgq_session *s, int enabled);
int mgq_session_gpu_timings(mgq_session *s, float *microseconds, size_t count);
int mgq_session_dump_gpu_timings(mgq_session *s, char *out, size_t cap);
int mgq_session_num_groups(const mgq_session *s);
int mgq_barrier_groups(const int32_t *inputs, const int32_t *outputs, size_t n, int reorder);

#ifdef __cplusplus
}
#endif
#endif /* MGQ_H */
