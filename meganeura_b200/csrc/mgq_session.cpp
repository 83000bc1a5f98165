// Graph -> plan -> Session for the quantized-matmul path and the decode step around it, behind the
// C ABI.
//
// Mirrors, for this path only, meganeura's builder and runtime surface:
//   Graph::{input, input_u32, parameter, parameter_q4, parameter_q8, matmul, add, embedding,
//           rms_norm, rope_dynamic_offset, cache_write, cached_attention, swiglu, swiglu_concat,
//           set_outputs}                                src/graph.rs:714-795, 1003-1009, 1029-1040,
//                                                       1062-1087, 1148-1170, 1659-1700
//   MatMul+Add -> FusedMatMulAdd                          src/optimize.rs:724-767
//   gate|up -> one concatenated weight + SwiGLUConcat     src/optimize.rs:776-879
//   lowering of these ops, labels                         src/compile.rs:1275-1285, 1381-1421,
//                                                       1486-1524, 1814-1950
//   build_inference_session                               src/train.rs:380-389
//   Session::{set_parameter, upload_param, set_input, step, wait, read_output*}
//                                                        src/runtime.rs:2327-2345, 2786-2791, 2496-2550,
//                                                        2835-2959, 2612-2643
// One session = one device = one stream with the dispatches enqueued in plan order; kernels run
// asynchronously until wait().  Where the reference panics, these calls return a status.
//
// Beyond the reference: (1) every group of single-row GEMVs that read the same activation is
// lowered to ONE GEMV over the column-concatenated packed weight (the reference does this for
// gate|up only); the original results are views into its output.  (2) The dispatch list can be
// captured once into a CUDA graph and replayed per step.  (3) A greedy pick can run on the device
// after the dispatches and feed the next token and position back, so consecutive decode steps need
// no host round trip.
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "mgq_internal.h"

namespace {

constexpr int kU32 = 100;         // node dtype of input_u32 (not a weight format)

enum class Op {
    Input, Parameter, MatMul, Add, FusedMatMulAdd, Embedding, RmsNorm, RoPE, CacheWrite, CachedAttention,
    SwiGLU, SwiGLUConcat, AllGather, MatMulBT, View, Nop
};

struct Node {
    Op op;
    std::string name;
    std::vector<size_t> shape;
    int dtype;                    // MGQ_FMT_F32 / Q4 / Q8, or kU32
    std::vector<int> inputs;
    float f0 = 0.f;               // eps (RmsNorm), theta (RoPE)
    uint32_t u0 = 0, u1 = 0, u2 = 0;   // head_dim (RoPE); num_heads, num_kv_heads, head_dim (CachedAttention); column offset (View)
    size_t elements() const { size_t e = 1; for (size_t s : shape) e *= s; return e; }
};

struct Dispatch {
    int shader;
    uint32_t workgroups[3];
    uint32_t params[4];           // matmuls: [m, k, n, 0] like the reference
    int in[4];                    // node ids of the inputs (-1: none)
    int out;                      // node id of the output
    int extra[3];                 // further outputs of a merged dispatch (node ids, -1: none)
    int weight_format;
    float f0;
    void *workspace;
    int exchange = -1;            // all_gather: which exchange; GEMV: the exchange it pushes its columns to (-1: none)
    bool push_done = false;       // all_gather: the producing GEMV has pushed the slice already
    std::string label;
};

struct Buffer {
    size_t bytes = 0;
    void *dev = nullptr;
};

// A packed weight that holds several parameters side by side (columns concatenated).
struct ConcatWeight {
    int node;                          // the derived Parameter node
    std::vector<int> members;          // original Parameter nodes, in column order
    std::vector<size_t> col0;          // first column of each member
};

__global__ void add_kernel(const float *a, const float *b, float *c, size_t len)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < len) c[i] = a[i] + b[i];
}

const char *shader_name(int s)
{
    switch (s) {
        case MGQ_SHADER_MATMUL: return "MatMul";
        case MGQ_SHADER_FUSED_MATMUL_ADD: return "FusedMatMulAdd";
        case MGQ_SHADER_MATMUL_GEMV: return "MatMulGemv";
        case MGQ_SHADER_MATMUL_GEMV_ADD: return "MatMulGemvAdd";
        case MGQ_SHADER_ADD: return "Add";
        case MGQ_SHADER_EMBEDDING: return "Embedding";
        case MGQ_SHADER_RMS_NORM: return "RmsNorm";
        case MGQ_SHADER_ROPE_DYNAMIC: return "RoPEDynamic";
        case MGQ_SHADER_CACHE_WRITE: return "CacheWrite";
        case MGQ_SHADER_CACHED_ATTENTION: return "CachedAttention";
        case MGQ_SHADER_SWIGLU: return "SwiGLU";
        case MGQ_SHADER_SWIGLU_CONCAT: return "SwiGLUConcat";
        case MGQ_SHADER_ROPE_CACHE_WRITE: return "RoPEDynamic+CacheWrite";
        case MGQ_SHADER_ALL_GATHER: return "AllGather";
        case MGQ_SHADER_MATMUL_GEMV_BT: return "MatMulGemvBT";
    }
    return "?";
}

int g_fuse_rope_cache = 1;        // "session.fuse_rope_cache"
int g_horizontal_fusion = 2;      // "session.horizontal_fusion": 0 none, 1 gate|up only (the reference's), 2 every same-input GEMV group
int g_fuse_exchange = 1;          // "session.fuse_exchange": a GEMV that feeds an all_gather pushes its columns itself

// One all_gather of a column-sharded session: what the caller bound to it.
struct Exchange {
    uint32_t slice_len = 0, world = 0;
    const mgq_exchange_push *push_dev = nullptr;
    mgq_exchange_elem *local_vec = nullptr;
};

}  // namespace

namespace mgq {
int set_session_option(const char *name, long value)
{
    if (!std::strcmp(name, "session.horizontal_fusion")) {
        if (value < 0 || value > 2) return fail(MGQ_ERR_SHAPE, "%s must be 0, 1 or 2", name);
        g_horizontal_fusion = (int)value;
        return MGQ_OK;
    }
    if (!std::strcmp(name, "session.fuse_rope_cache")) {
        g_fuse_rope_cache = value ? 1 : 0;
        return MGQ_OK;
    }
    if (!std::strcmp(name, "session.fuse_exchange")) {
        g_fuse_exchange = value ? 1 : 0;
        return MGQ_OK;
    }
    return fail(MGQ_ERR_NAME, "unknown option: %s", name);
}
}  // namespace mgq

struct mgq_graph {
    std::vector<Node> nodes;
    std::vector<int> outputs;
};

struct mgq_session {
    std::vector<Node> nodes;                   // after fusion
    std::vector<int> order;                    // node ids in execution order
    std::vector<int> outputs;
    std::vector<int> node_buffer;              // node id -> buffer index (-1: none)
    std::vector<size_t> node_offset;           // byte offset inside the buffer (views)
    std::vector<Buffer> buffers;
    std::vector<ConcatWeight> concats;
    std::vector<Dispatch> dispatches;
    std::vector<void *> workspaces;
    std::vector<uint8_t> staging;              // host scratch for quantize-on-upload
    cudaStream_t stream = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    uint64_t launches = 0;
    int device = 0;
    // per-dispatch timing (set_profiling): one event before every dispatch and one after the last
    bool profiling = false, profiled = false;
    std::vector<cudaEvent_t> events;
    // greedy feedback
    bool greedy = false;
    int greedy_output = -1, greedy_token_input = -1, greedy_pos_input = -1;
    void *greedy_ws = nullptr;
    uint32_t *greedy_token = nullptr, *greedy_history = nullptr;
    uint32_t greedy_cap = 0;
    // column-sharded sessions: the all_gathers and the words of the exchange protocol
    std::vector<Exchange> exchanges;
    unsigned long long *xchg_epoch = nullptr;
    unsigned int *xchg_error = nullptr, *xchg_blocks = nullptr;

    void *ptr(int node) const
    {
        const int b = node_buffer[node];
        return b < 0 ? nullptr : static_cast<uint8_t *>(buffers[b].dev) + node_offset[node];
    }
};

using mgq::fail;

// Bytes of a node's buffer: packed blocks for Q4/Q8, 2 per element for f16 weights, else 4.
static size_t node_bytes(const Node &nd)
{
    if (mgq::is_quant(nd.dtype)) return mgq_packed_bytes(nd.dtype, nd.shape[0], nd.shape[1]);
    return nd.elements() * (nd.dtype == MGQ_FMT_F16 ? 2 : 4);
}

static int add_leaf(mgq_graph *g, Op op, const char *name, const size_t *shape, size_t rank, int dtype)
{
    if (!g || !name || !shape) return -fail(MGQ_ERR_NULL, "null argument");
    if (rank == 0 || rank > 4) return -fail(MGQ_ERR_SHAPE, "rank %zu not supported", rank);
    Node nd{op, name, std::vector<size_t>(shape, shape + rank), dtype, {}};
    if (nd.elements() == 0) return -fail(MGQ_ERR_SHAPE, "empty tensor '%s'", name);
    if (mgq::is_quant(dtype)) {
        if (rank != 2) return -fail(MGQ_ERR_SHAPE, "quantized parameter '%s' must be 2-D [K,N]", name);
        if (shape[0] % 32 != 0) return -fail(MGQ_ERR_SHAPE, "quantized parameter '%s': rows (K dim) must be a multiple of 32", name);
    }
    g->nodes.push_back(std::move(nd));
    return (int)g->nodes.size() - 1;
}

static bool valid(const mgq_graph *g, int id) { return id >= 0 && id < (int)g->nodes.size(); }

static int push_node(mgq_graph *g, Node nd)
{
    g->nodes.push_back(std::move(nd));
    return (int)g->nodes.size() - 1;
}

extern "C" {

mgq_graph *mgq_graph_new(void) { return new mgq_graph(); }
void mgq_graph_free(mgq_graph *g) { delete g; }

int mgq_graph_input(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Input, name, shape, rank, MGQ_FMT_F32); }
int mgq_graph_input_u32(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Input, name, shape, rank, kU32); }
int mgq_graph_parameter(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Parameter, name, shape, rank, MGQ_FMT_F32); }
int mgq_graph_parameter_q4(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Parameter, name, shape, rank, MGQ_FMT_Q4); }
int mgq_graph_parameter_q8(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Parameter, name, shape, rank, MGQ_FMT_Q8); }
int mgq_graph_parameter_f16(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Parameter, name, shape, rank, MGQ_FMT_F16); }

int mgq_graph_matmul(mgq_graph *g, int a, int b)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, a) || !valid(g, b)) return -fail(MGQ_ERR_NAME, "matmul: node id out of range");
    const Node &na = g->nodes[a], &nb = g->nodes[b];
    if (na.shape.size() != 2 || nb.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "matmul requires 2D tensors");
    if (na.shape[1] != nb.shape[0]) return -fail(MGQ_ERR_SHAPE, "matmul inner dimensions must match (%zu vs %zu)", na.shape[1], nb.shape[0]);
    if (na.dtype != MGQ_FMT_F32) return -fail(MGQ_ERR_FORMAT, "matmul: the left operand must be f32");
    return push_node(g, Node{Op::MatMul, "", {na.shape[0], nb.shape[1]}, MGQ_FMT_F32, {a, b}});
}

int mgq_graph_matmul_bt(mgq_graph *g, int a, int b)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, a) || !valid(g, b)) return -fail(MGQ_ERR_NAME, "matmul_bt: node id out of range");
    const Node &na = g->nodes[a], &nb = g->nodes[b];
    if (na.shape.size() != 2 || nb.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "matmul_bt requires 2D tensors");
    if (na.shape[1] != nb.shape[1]) return -fail(MGQ_ERR_SHAPE, "MatMulBT: K dimensions must match (%zu vs %zu)", na.shape[1], nb.shape[1]);
    if (na.dtype != MGQ_FMT_F32 || nb.dtype != MGQ_FMT_F32) return -fail(MGQ_ERR_FORMAT, "matmul_bt: both operands must be f32");
    return push_node(g, Node{Op::MatMulBT, "", {na.shape[0], nb.shape[0]}, MGQ_FMT_F32, {a, b}});
}

int mgq_graph_add(mgq_graph *g, int a, int b)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, a) || !valid(g, b)) return -fail(MGQ_ERR_NAME, "add: node id out of range");
    const Node &na = g->nodes[a], &nb = g->nodes[b];
    if (na.shape != nb.shape) return -fail(MGQ_ERR_SHAPE, "add: shapes differ");
    if (na.dtype != MGQ_FMT_F32 || nb.dtype != MGQ_FMT_F32) return -fail(MGQ_ERR_FORMAT, "add: operands must be f32");
    return push_node(g, Node{Op::Add, "", na.shape, MGQ_FMT_F32, {a, b}});
}

int mgq_graph_embedding(mgq_graph *g, int indices, int table)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, indices) || !valid(g, table)) return -fail(MGQ_ERR_NAME, "embedding: node id out of range");
    const Node &ni = g->nodes[indices], &nt = g->nodes[table];
    if (ni.dtype != kU32) return -fail(MGQ_ERR_FORMAT, "embedding indices must be U32");
    if (ni.shape.size() != 1) return -fail(MGQ_ERR_SHAPE, "embedding indices must be 1D");
    if (nt.shape.size() != 2 || nt.dtype != MGQ_FMT_F32) return -fail(MGQ_ERR_SHAPE, "embedding table must be 2D f32");
    return push_node(g, Node{Op::Embedding, "", {ni.shape[0], nt.shape[1]}, MGQ_FMT_F32, {indices, table}});
}

int mgq_graph_rms_norm(mgq_graph *g, int x, int weight, float eps)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, x) || !valid(g, weight)) return -fail(MGQ_ERR_NAME, "rms_norm: node id out of range");
    const Node &nx = g->nodes[x], &nw = g->nodes[weight];
    if (nx.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "rms_norm requires 2D input");
    if (nw.shape.size() != 1) return -fail(MGQ_ERR_SHAPE, "rms_norm weight must be 1D");
    if (nx.shape[1] != nw.shape[0]) return -fail(MGQ_ERR_SHAPE, "rms_norm weight size must match last dim");
    if (nx.dtype != MGQ_FMT_F32 || nw.dtype != MGQ_FMT_F32) return -fail(MGQ_ERR_FORMAT, "rms_norm operands must be f32");
    Node nd{Op::RmsNorm, "", nx.shape, MGQ_FMT_F32, {x, weight}};
    nd.f0 = eps;
    return push_node(g, nd);
}

int mgq_graph_rope_dynamic_offset(mgq_graph *g, int x, float theta, int offset_input, uint32_t head_dim)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, x) || !valid(g, offset_input)) return -fail(MGQ_ERR_NAME, "rope: node id out of range");
    const Node &nx = g->nodes[x];
    if (nx.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "rope requires 2D input");
    if (g->nodes[offset_input].dtype != kU32) return -fail(MGQ_ERR_FORMAT, "rope offset must be a U32 input");
    const size_t dim = nx.shape[1];
    if (dim % 2 != 0) return -fail(MGQ_ERR_SHAPE, "rope requires even last dim");
    if (head_dim == 0 || dim % head_dim != 0) return -fail(MGQ_ERR_SHAPE, "rope: dim must be divisible by head_dim");
    if (head_dim % 2 != 0) return -fail(MGQ_ERR_SHAPE, "rope: head_dim must be even");
    Node nd{Op::RoPE, "", nx.shape, MGQ_FMT_F32, {x, offset_input}};
    nd.f0 = theta;
    nd.u0 = head_dim;
    return push_node(g, nd);
}

int mgq_graph_cache_write(mgq_graph *g, int new_kv, int cache, int kv_pos)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, new_kv) || !valid(g, cache) || !valid(g, kv_pos)) return -fail(MGQ_ERR_NAME, "cache_write: node id out of range");
    const Node &nk = g->nodes[new_kv], &nc = g->nodes[cache];
    if (nk.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "new_kv must be 2D");
    if (nk.shape[0] != 1) return -fail(MGQ_ERR_SHAPE, "new_kv must have seq_len=1");
    if (nc.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "cache must be 2D");
    if (nk.shape[1] != nc.shape[1]) return -fail(MGQ_ERR_SHAPE, "dim must match");
    if (nc.op != Op::Parameter || nc.dtype != MGQ_FMT_F32) return -fail(MGQ_ERR_FORMAT, "cache must be an f32 parameter");
    if (g->nodes[kv_pos].dtype != kU32) return -fail(MGQ_ERR_FORMAT, "kv_pos must be a U32 input");
    return push_node(g, Node{Op::CacheWrite, "", nc.shape, MGQ_FMT_F32, {new_kv, cache, kv_pos}});
}

int mgq_graph_cached_attention(mgq_graph *g, int q, int k_cache, int v_cache, int kv_pos, uint32_t num_heads,
                               uint32_t num_kv_heads, uint32_t head_dim)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, q) || !valid(g, k_cache) || !valid(g, v_cache) || !valid(g, kv_pos)) return -fail(MGQ_ERR_NAME, "cached_attention: node id out of range");
    const Node &nq = g->nodes[q], &nk = g->nodes[k_cache], &nv = g->nodes[v_cache];
    if (nq.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "q must be 2D");
    if (nq.shape[0] != 1) return -fail(MGQ_ERR_SHAPE, "q must have seq_len=1 for cached attention");
    if (nq.shape[1] != (size_t)num_heads * head_dim) return -fail(MGQ_ERR_SHAPE, "q dim mismatch");
    if (nk.shape.size() != 2 || nv.shape != nk.shape || nk.shape[1] != (size_t)num_kv_heads * head_dim) return -fail(MGQ_ERR_SHAPE, "cache shape mismatch");
    if (g->nodes[kv_pos].dtype != kU32) return -fail(MGQ_ERR_FORMAT, "kv_pos must be a U32 input");
    Node nd{Op::CachedAttention, "", {1, (size_t)num_heads * head_dim}, MGQ_FMT_F32, {q, k_cache, v_cache, kv_pos}};
    nd.u0 = num_heads; nd.u1 = num_kv_heads; nd.u2 = head_dim;
    return push_node(g, nd);
}

int mgq_graph_swiglu(mgq_graph *g, int gate, int up)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, gate) || !valid(g, up)) return -fail(MGQ_ERR_NAME, "swiglu: node id out of range");
    const Node &ng = g->nodes[gate], &nu = g->nodes[up];
    if (ng.shape.size() != 2 || ng.shape != nu.shape) return -fail(MGQ_ERR_SHAPE, "swiglu: shapes differ");
    if (ng.dtype != MGQ_FMT_F32 || nu.dtype != MGQ_FMT_F32) return -fail(MGQ_ERR_FORMAT, "swiglu operands must be f32");
    return push_node(g, Node{Op::SwiGLU, "", ng.shape, MGQ_FMT_F32, {gate, up}});
}

int mgq_graph_swiglu_concat(mgq_graph *g, int input)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, input)) return -fail(MGQ_ERR_NAME, "swiglu_concat: node id out of range");
    const Node &ni = g->nodes[input];
    if (ni.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "swiglu_concat requires 2D input");
    if (ni.shape[1] % 2 != 0) return -fail(MGQ_ERR_SHAPE, "SwiGLUConcat requires even N");
    return push_node(g, Node{Op::SwiGLUConcat, "", {ni.shape[0], ni.shape[1] / 2}, MGQ_FMT_F32, {input}});
}

int mgq_graph_slice_columns(mgq_graph *g, int x, uint32_t first, uint32_t count)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, x)) return -fail(MGQ_ERR_NAME, "slice_columns: node id out of range");
    const Node &nx = g->nodes[x];
    if (nx.dtype != MGQ_FMT_F32 || nx.shape.size() != 2 || nx.shape[0] != 1)
        return -fail(MGQ_ERR_SHAPE, "slice_columns: the source must be a [1, n] f32 tensor");
    if (count == 0 || (size_t)first + count > nx.shape[1] || first % 4 != 0)
        return -fail(MGQ_ERR_SHAPE, "slice_columns: [%u, %u) is not a 16-byte aligned range of %zu columns", first, first + count, nx.shape[1]);
    Node nd{Op::View, "", {1, count}, MGQ_FMT_F32, {x}};
    nd.u0 = first;
    return push_node(g, std::move(nd));
}

int mgq_graph_all_gather(mgq_graph *g, int x, uint32_t world)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    if (!valid(g, x)) return -fail(MGQ_ERR_NAME, "all_gather: node id out of range");
    const Node &nx = g->nodes[x];
    if (nx.dtype != MGQ_FMT_F32 || nx.shape.size() != 2 || nx.shape[0] != 1)
        return -fail(MGQ_ERR_SHAPE, "all_gather: the slice must be a [1, n] f32 tensor");
    if (world < 1 || world > MGQ_MAX_PEERS) return -fail(MGQ_ERR_SHAPE, "all_gather: world must be 1..%d", MGQ_MAX_PEERS);
    Node nd{Op::AllGather, "", {1, nx.shape[1] * world}, MGQ_FMT_F32, {x}};
    nd.u0 = world;
    return push_node(g, std::move(nd));
}

int mgq_graph_set_outputs(mgq_graph *g, const int *ids, size_t count)
{
    if (!g || !ids) return fail(MGQ_ERR_NULL, "null argument");
    for (size_t i = 0; i < count; i++)
        if (!valid(g, ids[i])) return fail(MGQ_ERR_NAME, "set_outputs: node id out of range");
    g->outputs.assign(ids, ids + count);
    return MGQ_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------ build

namespace {

int count_uses(const std::vector<Node> &nodes, int id)
{
    int uses = 0;
    for (const Node &nd : nodes)
        if (nd.op != Op::Nop)
            for (int in : nd.inputs) if (in == id) { uses++; break; }
    return uses;
}

// MatMul + Add -> FusedMatMulAdd when the matmul has exactly one use and is not an output.
void fuse_matmul_add(mgq_session *s)
{
    auto is_output = [&](int id) { for (int o : s->outputs) if (o == id) return true; return false; };
    for (size_t id = 0; id < s->nodes.size(); id++) {
        if (s->nodes[id].op != Op::Add) continue;
        const int lhs = s->nodes[id].inputs[0], rhs = s->nodes[id].inputs[1];
        int mm, addend;
        if (s->nodes[lhs].op == Op::MatMul) { mm = lhs; addend = rhs; }
        else if (s->nodes[rhs].op == Op::MatMul) { mm = rhs; addend = lhs; }
        else continue;
        if (count_uses(s->nodes, mm) != 1 || is_output(mm)) continue;
        const int a = s->nodes[mm].inputs[0], b = s->nodes[mm].inputs[1];
        s->nodes[id].op = Op::FusedMatMulAdd;
        s->nodes[id].inputs = {a, b, addend};
        s->nodes[mm].op = Op::Nop;
        s->nodes[mm].inputs.clear();
    }
}

// Single-row matmuls that read the same activation and whose weights are quantized parameters of
// one format become one matmul over the column-concatenated weight; each original node turns into
// a view of its column range.  `order` receives the fused node right before the first member.
void fuse_horizontal(mgq_session *s, int mode)
{
    if (mode == 0) return;
    const size_t n0 = s->nodes.size();
    std::vector<bool> taken(n0, false);
    std::vector<std::pair<int, int>> insert_before;           // (first member, fused node)
    for (size_t id = 0; id < n0; id++) {
        if (taken[id] || s->nodes[id].op != Op::MatMul) continue;
        const int a = s->nodes[id].inputs[0];
        const Node &w0 = s->nodes[s->nodes[id].inputs[1]];
        if (s->nodes[id].shape[0] != 1 || w0.op != Op::Parameter || !mgq::is_quant(w0.dtype)) continue;
        std::vector<int> group{(int)id};
        for (size_t j = id + 1; j < n0; j++) {
            const Node &nj = s->nodes[j];
            if (taken[j] || nj.op != Op::MatMul || nj.inputs[0] != a) continue;
            const Node &wj = s->nodes[nj.inputs[1]];
            if (wj.op != Op::Parameter || wj.dtype != w0.dtype) continue;
            group.push_back((int)j);
        }
        // every weight must be used by its matmul alone
        bool ok = group.size() >= 2;
        for (int m : group) ok = ok && count_uses(s->nodes, s->nodes[m].inputs[1]) == 1;
        if (ok && mode == 1) {
            // the reference's rule: exactly gate and up, consumed together by one SwiGLU
            ok = false;
            if (group.size() == 2)
                for (const Node &nd : s->nodes)
                    if (nd.op == Op::SwiGLU && nd.inputs[0] == group[0] && nd.inputs[1] == group[1]) ok = true;
        }
        if (!ok) continue;
        ConcatWeight cw;
        size_t cols = 0;
        std::string name = "concat(";
        for (size_t i = 0; i < group.size(); i++) {
            const int w = s->nodes[group[i]].inputs[1];
            cw.members.push_back(w);
            cw.col0.push_back(cols);
            cols += s->nodes[w].shape[1];
            name += (i ? "|" : "") + s->nodes[w].name;
        }
        name += ")";
        const size_t k = w0.shape[0];
        const int fmt = w0.dtype;
        s->nodes.push_back(Node{Op::Parameter, name, {k, cols}, fmt, {}});
        cw.node = (int)s->nodes.size() - 1;
        s->nodes.push_back(Node{Op::MatMul, "", {1, cols}, MGQ_FMT_F32, {a, cw.node}});
        const int fused = (int)s->nodes.size() - 1;
        for (size_t i = 0; i < group.size(); i++) {
            Node &m = s->nodes[group[i]];
            taken[group[i]] = true;
            m.op = Op::View;
            m.inputs = {fused};
            m.u0 = (uint32_t)cw.col0[i];
        }
        s->concats.push_back(cw);
        insert_before.push_back({group[0], fused});
    }
    // execution order: original node order, fused matmuls slotted in before their first member
    s->order.clear();
    for (size_t id = 0; id < n0; id++) {
        for (const auto &pr : insert_before)
            if (pr.first == (int)id) { s->order.push_back(pr.second - 1); s->order.push_back(pr.second); }
        s->order.push_back((int)id);
    }
}

// RoPE(q), RoPE(k), CacheWrite(rope(k)), CacheWrite(v) in a row, all on the same position input and
// with v produced earlier, become one dispatch.
void merge_rope_cache(mgq_session *s)
{
    std::vector<Dispatch> &ds = s->dispatches;
    auto produced_before = [&](int node, size_t index) {
        int root = node;
        while (s->nodes[root].op == Op::View) root = s->nodes[root].inputs[0];
        if (s->nodes[root].op == Op::Input || s->nodes[root].op == Op::Parameter) return true;
        for (size_t j = 0; j < index; j++) if (ds[j].out == root) return true;
        return false;
    };
    for (size_t i = 0; i + 3 < ds.size(); i++) {
        const Dispatch &a = ds[i], &b = ds[i + 1], &c = ds[i + 2], &e = ds[i + 3];
        if (a.shader != MGQ_SHADER_ROPE_DYNAMIC || b.shader != MGQ_SHADER_ROPE_DYNAMIC) continue;
        if (c.shader != MGQ_SHADER_CACHE_WRITE || e.shader != MGQ_SHADER_CACHE_WRITE) continue;
        if (a.params[0] != 1 || b.params[0] != 1) continue;                              // one token
        if (a.in[1] != b.in[1] || c.in[2] != a.in[1] || e.in[2] != a.in[1]) continue;    // one position input
        if (a.params[2] != b.params[2] || a.params[3] != b.params[3]) continue;          // same theta and head_dim
        if (c.in[0] != b.out || c.params[0] != b.params[1] || e.params[0] != b.params[1]) continue;
        if (c.params[1] != e.params[1] || !produced_before(e.in[0], i)) continue;
        Dispatch m = a;
        m.shader = MGQ_SHADER_ROPE_CACHE_WRITE;
        m.in[0] = a.in[0]; m.in[1] = b.in[0]; m.in[2] = e.in[0]; m.in[3] = a.in[1];
        m.out = a.out; m.extra[0] = b.out; m.extra[1] = c.out; m.extra[2] = e.out;
        m.params[0] = a.params[1]; m.params[1] = b.params[1]; m.params[2] = a.params[3]; m.params[3] = c.params[1];   // q_dim, kv_dim, head_dim, max_seq
        m.workgroups[0] = (m.params[0] / 2 + m.params[1] / 2 + m.params[1] + 255) / 256;
        char lab[96];
        std::snprintf(lab, sizeof lab, "RoPEDynamic+CacheWrite[q%u kv%u]", m.params[0], m.params[1]);
        m.label = lab;
        ds[i] = m;
        ds.erase(ds.begin() + i + 1, ds.begin() + i + 4);
    }
}

void set_label(Dispatch &d, const char *fmt, ...)
{
    char lab[128];
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(lab, sizeof lab, fmt, ap);
    va_end(ap);
    d.label = lab;
}

}  // namespace

extern "C" {

int mgq_build_inference_session(const mgq_graph *g, mgq_session **out)
{
    if (!g || !out) return fail(MGQ_ERR_NULL, "null argument");
    *out = nullptr;
    if (g->outputs.empty()) return fail(MGQ_ERR_STATE, "graph has no outputs");
    mgq_session *s = new mgq_session();
    s->nodes = g->nodes;
    s->outputs = g->outputs;
    for (size_t id = 0; id < s->nodes.size(); id++) s->order.push_back((int)id);

    fuse_matmul_add(s);
    fuse_horizontal(s, g_horizontal_fusion);

    // Buffers: one per live node; views and cache writes alias their source; members of a
    // concatenated weight have no buffer of their own.
    s->node_buffer.assign(s->nodes.size(), -1);
    s->node_offset.assign(s->nodes.size(), 0);
    std::vector<bool> is_member(s->nodes.size(), false);
    for (const ConcatWeight &cw : s->concats) for (int m : cw.members) is_member[m] = true;
    for (int id : s->order) {
        const Node &nd = s->nodes[id];
        if (nd.op == Op::Nop || is_member[id]) continue;
        if (nd.op == Op::View) {
            s->node_buffer[id] = s->node_buffer[nd.inputs[0]];
            s->node_offset[id] = s->node_offset[nd.inputs[0]] + (size_t)nd.u0 * 4;
            continue;
        }
        if (nd.op == Op::CacheWrite) {
            s->node_buffer[id] = s->node_buffer[nd.inputs[1]];
            s->node_offset[id] = s->node_offset[nd.inputs[1]];
            continue;
        }
        Buffer buf;
        buf.bytes = node_bytes(nd);
        s->node_buffer[id] = (int)s->buffers.size();
        s->buffers.push_back(buf);
    }

    int rc = mgq::cuda_check((int)cudaGetDevice(&s->device), "cudaGetDevice", __FILE__, __LINE__);
    if (!rc) rc = mgq::cuda_check((int)cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking), "cudaStreamCreate", __FILE__, __LINE__);
    for (Buffer &b : s->buffers) {
        if (rc) break;
        rc = mgq_buffer_create(b.bytes, &b.dev);     // zero-filled, like the reference
    }
    if (rc) { mgq_session_free(s); return rc; }

    // Lowering, in execution order.
    for (int id : s->order) {
        const Node &nd = s->nodes[id];
        Dispatch d{};
        d.in[0] = d.in[1] = d.in[2] = d.in[3] = -1;
        d.extra[0] = d.extra[1] = d.extra[2] = -1;
        for (size_t i = 0; i < nd.inputs.size() && i < 4; i++) d.in[i] = nd.inputs[i];
        d.out = id;
        d.weight_format = MGQ_FMT_F32;
        d.workgroups[1] = d.workgroups[2] = 1;
        switch (nd.op) {
            case Op::MatMul:
            case Op::FusedMatMulAdd: {
                const Node &na = s->nodes[nd.inputs[0]], &nb = s->nodes[nd.inputs[1]];
                const bool f16w = nb.op == Op::Parameter && nb.dtype == MGQ_FMT_F16;
                if (nb.op != Op::Parameter || !(mgq::is_quant(nb.dtype) || f16w)) {
                    mgq_session_free(s);
                    return fail(MGQ_ERR_FORMAT, "matmul weight must be a parameter_q4 / parameter_q8 / parameter_f16 node (f32 weights are outside this library)");
                }
                const bool fused = nd.op == Op::FusedMatMulAdd;
                const uint32_t m = (uint32_t)na.shape[0], k = (uint32_t)na.shape[1], n = (uint32_t)nb.shape[1];
                if (f16w && (m > MGQ_GEMV_MAX_M || n % 8 != 0)) {
                    mgq_session_free(s);
                    return fail(MGQ_ERR_SHAPE, "f16 weights: at most %d rows and N %% 8 == 0 (got %ux%ux%u)", MGQ_GEMV_MAX_M, m, k, n);
                }
                if (m == 1 && n % 4 == 0) {
                    d.shader = fused ? MGQ_SHADER_MATMUL_GEMV_ADD : MGQ_SHADER_MATMUL_GEMV;
                    d.workgroups[0] = n / 4;
                } else {
                    d.shader = fused ? MGQ_SHADER_FUSED_MATMUL_ADD : MGQ_SHADER_MATMUL;
                    d.workgroups[0] = (n + 63) / 64; d.workgroups[1] = (m + 63) / 64;
                }
                d.params[0] = m; d.params[1] = k; d.params[2] = n; d.params[3] = 0;
                d.weight_format = nb.dtype;
                set_label(d, "%s[%ux%ux%u]", shader_name(d.shader), m, n, k);
                break;
            }
            case Op::MatMulBT: {
                const Node &na = s->nodes[nd.inputs[0]], &nb = s->nodes[nd.inputs[1]];
                const uint32_t m = (uint32_t)na.shape[0], k = (uint32_t)na.shape[1], n = (uint32_t)nb.shape[0];
                if (m != 1 || k % 4 != 0) {          // the reference's tiled MatMulBT (m > 1) is outside this library
                    mgq_session_free(s);
                    return fail(MGQ_ERR_SHAPE, "matmul_bt: only the single-row form with K %% 4 == 0 is lowered (got %ux%ux%u)", m, n, k);
                }
                d.shader = MGQ_SHADER_MATMUL_GEMV_BT;
                d.workgroups[0] = n;
                d.params[0] = m; d.params[1] = n; d.params[2] = k; d.params[3] = 0;      // [m, n, k, 0] like the reference
                set_label(d, "MatMulGemvBT[%ux%ux%u]", m, n, k);
                break;
            }
            case Op::Add: {
                d.shader = MGQ_SHADER_ADD;
                const uint32_t len = (uint32_t)nd.elements();
                d.workgroups[0] = (len + 255) / 256;
                d.params[0] = len;
                set_label(d, "Add[%u]", len);
                break;
            }
            case Op::Embedding: {
                d.shader = MGQ_SHADER_EMBEDDING;
                const uint32_t seq = (uint32_t)nd.shape[0], hidden = (uint32_t)nd.shape[1];
                d.workgroups[0] = (seq * hidden + 255) / 256;
                d.params[0] = seq; d.params[1] = hidden; d.params[2] = (uint32_t)s->nodes[nd.inputs[1]].shape[0];
                set_label(d, "Embedding[%ux%u]", seq, hidden);
                break;
            }
            case Op::RmsNorm: {
                d.shader = MGQ_SHADER_RMS_NORM;
                d.workgroups[0] = (uint32_t)nd.shape[0];
                d.params[0] = (uint32_t)nd.shape[0]; d.params[1] = (uint32_t)nd.shape[1];
                d.f0 = nd.f0;
                std::memcpy(&d.params[2], &nd.f0, 4);                  // eps_bits, like the reference's uniform
                set_label(d, "RmsNorm[%ux%u]", d.params[0], d.params[1]);
                break;
            }
            case Op::RoPE: {
                d.shader = MGQ_SHADER_ROPE_DYNAMIC;
                const uint32_t seq = (uint32_t)nd.shape[0], dim = (uint32_t)nd.shape[1];
                d.workgroups[0] = (seq * dim / 2 + 255) / 256;
                d.params[0] = seq; d.params[1] = dim; d.params[3] = nd.u0;
                std::memcpy(&d.params[2], &nd.f0, 4);                  // theta_bits
                d.f0 = nd.f0;
                set_label(d, "RoPEDynamic[%ux%u]", seq, dim);
                break;
            }
            case Op::CacheWrite: {
                d.shader = MGQ_SHADER_CACHE_WRITE;
                const uint32_t dim = (uint32_t)nd.shape[1];
                d.workgroups[0] = (dim + 255) / 256;
                d.params[0] = dim; d.params[1] = (uint32_t)nd.shape[0];
                set_label(d, "CacheWrite[%u]", dim);
                break;
            }
            case Op::CachedAttention: {
                d.shader = MGQ_SHADER_CACHED_ATTENTION;
                d.workgroups[0] = 1; d.workgroups[1] = nd.u0;
                d.params[0] = (uint32_t)s->nodes[nd.inputs[1]].shape[0];   // max_seq (the reference's slot is reserved)
                d.params[1] = nd.u0; d.params[2] = nd.u1; d.params[3] = nd.u2;
                if (d.params[0] > 4096) {           // the attention kernel's limit: refuse here, not at the first step
                    mgq_session_free(s);
                    return fail(MGQ_ERR_SHAPE, "cached_attention: a cache of %u rows exceeds the kernel's limit of 4096", d.params[0]);
                }
                const size_t ws = mgq_cached_attention_workspace(nd.u1, nd.u2, d.params[0]);
                rc = mgq_buffer_create(ws, &d.workspace);
                if (rc) { mgq_session_free(s); return rc; }
                s->workspaces.push_back(d.workspace);
                set_label(d, "CachedAttention[%ux%u]", nd.u0, nd.u2);
                break;
            }
            case Op::SwiGLU: {
                const Node &ga = s->nodes[nd.inputs[0]], &up = s->nodes[nd.inputs[1]];
                const uint32_t len = (uint32_t)nd.elements(), half_n = (uint32_t)nd.shape[1];
                // gate and up that are adjacent views of one fused matmul are the reference's SwiGLUConcat
                const bool concat = ga.op == Op::View && up.op == Op::View && ga.inputs[0] == up.inputs[0] &&
                                    up.u0 == ga.u0 + half_n;
                d.shader = concat ? MGQ_SHADER_SWIGLU_CONCAT : MGQ_SHADER_SWIGLU;
                d.workgroups[0] = (len + 255) / 256;
                d.params[0] = len; d.params[1] = half_n; d.params[2] = half_n;      // [len, half_n, pitch]
                set_label(d, "%s[%u]", shader_name(d.shader), len);
                break;
            }
            case Op::SwiGLUConcat: {
                d.shader = MGQ_SHADER_SWIGLU_CONCAT;
                const uint32_t len = (uint32_t)nd.elements(), half_n = (uint32_t)nd.shape[1];
                d.workgroups[0] = (len + 255) / 256;
                d.params[0] = len; d.params[1] = half_n; d.params[2] = 2 * half_n;
                set_label(d, "SwiGLUConcat[%u]", len);
                break;
            }
            case Op::AllGather: {
                d.shader = MGQ_SHADER_ALL_GATHER;
                Exchange ex;
                ex.slice_len = (uint32_t)s->nodes[nd.inputs[0]].elements();
                ex.world = nd.u0;
                d.exchange = (int)s->exchanges.size();
                s->exchanges.push_back(ex);
                d.params[0] = ex.slice_len; d.params[1] = ex.world; d.params[2] = ex.slice_len * ex.world;
                d.workgroups[0] = (d.params[2] + 255) / 256;
                set_label(d, "AllGather[%ux%u]", ex.world, ex.slice_len);
                // a single-row GEMV whose whole output is the slice stores its columns into the ranks'
                // gathered vectors itself; the all_gather then only waits and unpacks
                if (g_fuse_exchange && !s->dispatches.empty()) {
                    Dispatch &prev = s->dispatches.back();
                    const bool gemv = prev.shader == MGQ_SHADER_MATMUL_GEMV || prev.shader == MGQ_SHADER_MATMUL_GEMV_ADD;
                    if (gemv && prev.out == nd.inputs[0] && prev.params[0] == 1 && prev.params[2] == ex.slice_len &&
                        mgq::is_quant(prev.weight_format) && prev.exchange < 0) {
                        prev.exchange = d.exchange;
                        d.push_done = true;
                    }
                }
                break;
            }
            default: continue;           // Input, Parameter, View, Nop: nothing to run
        }
        s->dispatches.push_back(d);
    }
    if (g_fuse_rope_cache) merge_rope_cache(s);
    *out = s;
    return MGQ_OK;
}

void mgq_session_free(mgq_session *s)
{
    if (!s) return;
    if (s->stream) cudaStreamSynchronize(s->stream);
    if (s->graph_exec) cudaGraphExecDestroy(s->graph_exec);
    if (s->graph) cudaGraphDestroy(s->graph);
    for (Buffer &b : s->buffers) if (b.dev) cudaFree(b.dev);
    for (void *w : s->workspaces) if (w) cudaFree(w);
    if (s->greedy_ws) cudaFree(s->greedy_ws);
    if (s->greedy_token) cudaFree(s->greedy_token);
    if (s->greedy_history) cudaFree(s->greedy_history);
    for (cudaEvent_t e : s->events) cudaEventDestroy(e);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

static int find_named(const mgq_session *s, Op op, const char *name)
{
    for (size_t id = 0; id < s->nodes.size(); id++)
        if (s->nodes[id].op == op && s->nodes[id].name == name) return (int)id;
    return -1;
}

// Where the packed bytes of parameter `id` live: its own buffer, or a column range of a
// concatenated weight.  A Q4 weight is two regions (headers, then nibbles), a Q8 weight is one.
static int upload_packed(mgq_session *s, int id, const uint8_t *packed, size_t nbytes)
{
    const Node &nd = s->nodes[id];
    const size_t expect = mgq_packed_bytes(nd.dtype, nd.shape[0], nd.shape[1]);
    if (nbytes != expect) return fail(MGQ_ERR_SIZE, "parameter '%s' buffer is %zu bytes, got %zu", nd.name.c_str(), expect, nbytes);
    for (const ConcatWeight &cw : s->concats) {
        for (size_t i = 0; i < cw.members.size(); i++) {
            if (cw.members[i] != id) continue;
            uint8_t *base = static_cast<uint8_t *>(s->ptr(cw.node));
            const size_t bpc = nd.shape[0] / 32, n = nd.shape[1], n_total = s->nodes[cw.node].shape[1], c0 = cw.col0[i];
            if (nd.dtype == MGQ_FMT_Q8) return mgq_buffer_upload(base + c0 * bpc * 36, packed, nbytes, s->stream);
            int rc = mgq_buffer_upload(base + c0 * bpc * 4, packed, n * bpc * 4, s->stream);
            if (rc) return rc;
            return mgq_buffer_upload(base + n_total * bpc * 4 + c0 * bpc * 16, packed + n * bpc * 4, n * bpc * 16, s->stream);
        }
    }
    return mgq_buffer_upload(s->ptr(id), packed, nbytes, s->stream);
}

// The mirror of upload_packed: the raw bytes of parameter `id` as the reference would hold them.
static int download_param(mgq_session *s, int id, std::vector<uint8_t> &out)
{
    const Node &nd = s->nodes[id];
    if (!mgq::is_quant(nd.dtype)) {
        out.resize(node_bytes(nd));
        return mgq_buffer_download(s->ptr(id), out.data(), out.size(), s->stream);
    }
    out.resize(mgq_packed_bytes(nd.dtype, nd.shape[0], nd.shape[1]));
    for (const ConcatWeight &cw : s->concats) {
        for (size_t i = 0; i < cw.members.size(); i++) {
            if (cw.members[i] != id) continue;
            const uint8_t *base = static_cast<const uint8_t *>(s->ptr(cw.node));
            const size_t bpc = nd.shape[0] / 32, n = nd.shape[1], n_total = s->nodes[cw.node].shape[1], c0 = cw.col0[i];
            if (nd.dtype == MGQ_FMT_Q8) return mgq_buffer_download(base + c0 * bpc * 36, out.data(), out.size(), s->stream);
            int rc = mgq_buffer_download(base + c0 * bpc * 4, out.data(), n * bpc * 4, s->stream);
            if (rc) return rc;
            return mgq_buffer_download(base + n_total * bpc * 4 + c0 * bpc * 16, out.data() + n * bpc * 4, n * bpc * 16, s->stream);
        }
    }
    return mgq_buffer_download(s->ptr(id), out.data(), out.size(), s->stream);
}

// Checkpoints use the reference's file layout (Session::save_checkpoint / load_checkpoint,
// src/runtime.rs:4205-4336): a safetensors file in which every parameter buffer -- packed Q4/Q8
// bytes included -- is stored as a flat F32 tensor of byte_len / 4 elements under the parameter's
// name, with the Adam step counter as metadata (always "0" here: inference sessions).  The
// safetensors container itself is an 8-byte little-endian header length, a JSON header padded with
// spaces to a multiple of 8 bytes, and the tensor data in header order (sorted by name).
int mgq_session_save_checkpoint(mgq_session *s, const char *path)
{
    if (!s || !path) return fail(MGQ_ERR_NULL, "null argument");
    MGQ_CUDA(cudaStreamSynchronize(s->stream));
    std::map<std::string, int> params;                                   // sorted by name
    for (size_t id = 0; id < s->nodes.size(); id++) {
        const Node &nd = s->nodes[id];
        if (nd.op != Op::Parameter) continue;
        bool derived = false;
        for (const ConcatWeight &cw : s->concats) derived = derived || cw.node == (int)id;
        if (!derived) params[nd.name] = (int)id;
    }
    std::string header = "{\"__metadata__\":{\"adam_step\":\"0\"}";
    size_t offset = 0;
    for (const auto &kv : params) {
        const Node &nd = s->nodes[kv.second];
        const size_t bytes = node_bytes(nd);
        std::string key;
        for (char c : kv.first) { if (c == '"' || c == '\\') key += '\\'; key += c; }
        char item[160];
        std::snprintf(item, sizeof item, "\":{\"dtype\":\"F32\",\"shape\":[%zu],\"data_offsets\":[%zu,%zu]}", bytes / 4, offset, offset + bytes);
        header += ",\"" + key + item;
        offset += bytes;
    }
    header += "}";
    while (header.size() % 8 != 0) header += ' ';
    FILE *f = std::fopen(path, "wb");
    if (!f) return fail(MGQ_ERR_STATE, "cannot open %s for writing", path);
    const uint64_t hlen = header.size();
    bool ok = std::fwrite(&hlen, 8, 1, f) == 1 && std::fwrite(header.data(), 1, header.size(), f) == header.size();
    std::vector<uint8_t> bytes;
    for (const auto &kv : params) {
        if (!ok) break;
        if (int rc = download_param(s, kv.second, bytes)) { std::fclose(f); return rc; }
        ok = std::fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size();
    }
    ok = std::fclose(f) == 0 && ok;
    return ok ? MGQ_OK : fail(MGQ_ERR_STATE, "short write to %s", path);
}

// Restores every parameter the file holds under its name; parameters the file lacks keep their
// contents (the reference logs a warning), tensors the session lacks are ignored.
int mgq_session_load_checkpoint(mgq_session *s, const char *path)
{
    if (!s || !path) return fail(MGQ_ERR_NULL, "null argument");
    FILE *f = std::fopen(path, "rb");
    if (!f) return fail(MGQ_ERR_STATE, "cannot open %s", path);
    uint64_t hlen = 0;
    if (std::fread(&hlen, 8, 1, f) != 1 || hlen < 2 || hlen > (100u << 20)) { std::fclose(f); return fail(MGQ_ERR_FORMAT, "%s: not a safetensors file", path); }
    std::string header(hlen, '\0');
    if (std::fread(&header[0], 1, hlen, f) != hlen) { std::fclose(f); return fail(MGQ_ERR_FORMAT, "%s: truncated header", path); }
    // The header is flat JSON: "name":{"dtype":..,"shape":[..],"data_offsets":[b,e]}.  Find each
    // parameter's entry by its quoted name and read the two offsets.
    std::vector<uint8_t> bytes;
    int restored = 0;
    for (size_t id = 0; id < s->nodes.size(); id++) {
        const Node &nd = s->nodes[id];
        if (nd.op != Op::Parameter) continue;
        std::string key = "\"";
        for (char c : nd.name) { if (c == '"' || c == '\\') key += '\\'; key += c; }
        key += "\":{";
        const size_t at = header.find(key);
        if (at == std::string::npos) continue;
        const size_t end = header.find('}', at);
        const size_t off = header.find("\"data_offsets\":[", at);
        if (off == std::string::npos || off > end) { std::fclose(f); return fail(MGQ_ERR_FORMAT, "%s: entry of '%s' has no data_offsets", path, nd.name.c_str()); }
        unsigned long long b = 0, e = 0;
        if (std::sscanf(header.c_str() + off + 16, "%llu,%llu", &b, &e) != 2 || e < b) { std::fclose(f); return fail(MGQ_ERR_FORMAT, "%s: bad offsets for '%s'", path, nd.name.c_str()); }
        const size_t want = node_bytes(nd);
        if (e - b != want) { std::fclose(f); return fail(MGQ_ERR_SIZE, "%s: '%s' holds %llu bytes, the session needs %zu", path, nd.name.c_str(), e - b, want); }
        bytes.resize(want);
        if (std::fseek(f, (long)(8 + hlen + b), SEEK_SET) != 0 || std::fread(bytes.data(), 1, want, f) != want) { std::fclose(f); return fail(MGQ_ERR_FORMAT, "%s: truncated data for '%s'", path, nd.name.c_str()); }
        const int rc = mgq::is_quant(nd.dtype) ? upload_packed(s, (int)id, bytes.data(), want) : mgq_buffer_upload(s->ptr((int)id), bytes.data(), want, s->stream);
        if (rc) { std::fclose(f); return rc; }
        restored++;
    }
    std::fclose(f);
    if (restored == 0) return fail(MGQ_ERR_NAME, "%s holds none of this session's parameters", path);
    return MGQ_OK;
}

int mgq_session_set_parameter(mgq_session *s, const char *name, const float *data, size_t len)
{
    if (!s || !name || !data) return fail(MGQ_ERR_NULL, "null argument");
    const int id = find_named(s, Op::Parameter, name);
    if (id < 0) return fail(MGQ_ERR_NAME, "unknown parameter: %s", name);
    const Node &nd = s->nodes[id];
    if (len != nd.elements()) return fail(MGQ_ERR_SIZE, "parameter '%s' has %zu elements, got %zu", name, nd.elements(), len);
    if (nd.dtype == MGQ_FMT_F16) {                       // the reference converts with half::f16::from_f32 (src/runtime.rs:2335)
        s->staging.resize(len * 2);
        if (int rc = mgq_convert_f16(data, len, reinterpret_cast<uint16_t *>(s->staging.data()))) return rc;
        return mgq_buffer_upload(s->ptr(id), s->staging.data(), len * 2, s->stream);
    }
    if (!mgq::is_quant(nd.dtype)) return mgq_buffer_upload(s->ptr(id), data, len * 4, s->stream);
    s->staging.resize(mgq_packed_bytes(nd.dtype, nd.shape[0], nd.shape[1]));
    const int rc = nd.dtype == MGQ_FMT_Q4 ? mgq_quantize_q4(data, nd.shape[0], nd.shape[1], s->staging.data())
                                          : mgq_quantize_q8(data, nd.shape[0], nd.shape[1], s->staging.data());
    if (rc) return rc;
    return upload_packed(s, id, s->staging.data(), s->staging.size());
}

int mgq_session_upload_param(mgq_session *s, const char *name, const void *bytes, size_t nbytes)
{
    if (!s || !name || !bytes) return fail(MGQ_ERR_NULL, "null argument");
    const int id = find_named(s, Op::Parameter, name);
    if (id < 0) return fail(MGQ_ERR_NAME, "unknown parameter: %s", name);
    const Node &nd = s->nodes[id];
    if (mgq::is_quant(nd.dtype)) return upload_packed(s, id, static_cast<const uint8_t *>(bytes), nbytes);
    if (nbytes != node_bytes(nd)) return fail(MGQ_ERR_SIZE, "parameter '%s' buffer is %zu bytes, got %zu", name, node_bytes(nd), nbytes);
    return mgq_buffer_upload(s->ptr(id), bytes, nbytes, s->stream);
}

int mgq_session_set_input(mgq_session *s, const char *name, const float *data, size_t len)
{
    if (!s || !name || !data) return fail(MGQ_ERR_NULL, "null argument");
    const int id = find_named(s, Op::Input, name);
    if (id < 0 || s->nodes[id].dtype != MGQ_FMT_F32) return fail(MGQ_ERR_NAME, "unknown input: %s", name);
    const Node &nd = s->nodes[id];
    if (len != nd.elements()) return fail(MGQ_ERR_SIZE, "input '%s' has %zu elements, got %zu", name, nd.elements(), len);
    return mgq_buffer_upload(s->ptr(id), data, len * 4, s->stream);
}

int mgq_session_set_input_u32(mgq_session *s, const char *name, const uint32_t *data, size_t len)
{
    if (!s || !name || !data) return fail(MGQ_ERR_NULL, "null argument");
    const int id = find_named(s, Op::Input, name);
    if (id < 0 || s->nodes[id].dtype != kU32) return fail(MGQ_ERR_NAME, "unknown u32 input: %s", name);
    const Node &nd = s->nodes[id];
    if (len != nd.elements()) return fail(MGQ_ERR_SIZE, "input '%s' has %zu elements, got %zu", name, nd.elements(), len);
    return mgq_buffer_upload(s->ptr(id), data, len * 4, s->stream);
}

static int run_dispatch(mgq_session *s, const Dispatch &d)
{
    auto f = [&](int i) { return static_cast<const float *>(s->ptr(d.in[i])); };
    auto u = [&](int i) { return static_cast<const uint32_t *>(s->ptr(d.in[i])); };
    float *outp = static_cast<float *>(s->ptr(d.out));
    switch (d.shader) {
        case MGQ_SHADER_ADD:
            add_kernel<<<d.workgroups[0], 256, 0, s->stream>>>(f(0), f(1), outp, d.params[0]);
            MGQ_CUDA(cudaGetLastError());
            return MGQ_OK;
        case MGQ_SHADER_EMBEDDING: return mgq_embedding(u(0), f(1), outp, d.params[0], d.params[1], d.params[2], s->stream);
        case MGQ_SHADER_RMS_NORM: return mgq_rms_norm(f(0), f(1), outp, d.params[0], d.params[1], d.f0, s->stream);
        case MGQ_SHADER_ROPE_DYNAMIC: return mgq_rope_dynamic(f(0), outp, u(1), d.params[0], d.params[1], d.params[3], d.f0, s->stream);
        case MGQ_SHADER_CACHE_WRITE: return mgq_cache_write(f(0), outp, u(2), d.params[0], d.params[1], s->stream);
        case MGQ_SHADER_ROPE_CACHE_WRITE:
            return mgq_rope_cache_write(f(0), outp, f(1), static_cast<float *>(s->ptr(d.extra[0])), f(2), static_cast<float *>(s->ptr(d.extra[1])),
                                        static_cast<float *>(s->ptr(d.extra[2])), u(3), d.params[0], d.params[1], d.params[2], d.f0,
                                        d.params[3], s->stream);
        case MGQ_SHADER_CACHED_ATTENTION:
            return mgq_cached_attention(f(0), f(1), f(2), u(3), outp, d.params[1], d.params[2], d.params[3], d.params[0], d.workspace, s->stream);
        case MGQ_SHADER_SWIGLU: return mgq_swiglu(f(0), f(1), outp, d.params[0] / d.params[1], d.params[1], d.params[2], s->stream);
        case MGQ_SHADER_SWIGLU_CONCAT:
            if (d.in[1] >= 0) return mgq_swiglu(f(0), f(1), outp, d.params[0] / d.params[1], d.params[1], d.params[2], s->stream);
            return mgq_swiglu(f(0), f(0) + d.params[1], outp, d.params[0] / d.params[1], d.params[1], d.params[2], s->stream);
        case MGQ_SHADER_MATMUL_GEMV_BT: return mgq_gemv_bt(f(0), f(1), outp, d.params[2], d.params[1], s->stream);
        case MGQ_SHADER_ALL_GATHER: {
            const Exchange &ex = s->exchanges[d.exchange];
            return mgq_exchange_all_gather(d.push_done ? nullptr : f(0), ex.push_dev, ex.local_vec, outp, ex.slice_len,
                                           ex.slice_len * ex.world, s->xchg_epoch, s->xchg_error, s->stream);
        }
        default: {
            const float *addend = d.in[2] >= 0 ? f(2) : nullptr;
            if (d.exchange >= 0) {
                const Exchange &ex = s->exchanges[d.exchange];
                return mgq_gemv_exchange(d.weight_format, f(0), s->ptr(d.in[1]), addend, outp, d.params[1], d.params[2], ex.push_dev,
                                         nullptr, s->xchg_epoch, s->xchg_error, s->stream);
            }
            if (d.weight_format == MGQ_FMT_F16)
                return mgq_gemv_f16(f(0), s->ptr(d.in[1]), addend, outp, d.params[0], d.params[1], d.params[2], s->stream);
            return mgq_matmul(d.weight_format, s->ptr(d.in[0]), MGQ_A_F32, s->ptr(d.in[1]), addend, outp, d.params[0], d.params[1],
                              d.params[2], s->stream);
        }
    }
}

// A sharded step ends by adding one to the token index (every gathered vector of the step has been
// waited for by its all_gather, so nothing is left to poll).
static int end_token(mgq_session *s)
{
    if (s->exchanges.empty()) return MGQ_OK;
    return mgq_exchange_finish(nullptr, 0, s->xchg_epoch, s->xchg_error, s->xchg_blocks, s->stream);
}

static int exchanges_bound(const mgq_session *s)
{
    if (s->exchanges.empty()) return MGQ_OK;
    if (!s->xchg_epoch || !s->xchg_error || !s->xchg_blocks) return fail(MGQ_ERR_STATE, "sharded session: bind the exchange state before the first step");
    for (size_t i = 0; i < s->exchanges.size(); i++)
        if (!s->exchanges[i].push_dev || !s->exchanges[i].local_vec) return fail(MGQ_ERR_STATE, "sharded session: exchange %zu is not bound", i);
    return MGQ_OK;
}

static int enqueue_all(mgq_session *s)
{
    for (const Dispatch &d : s->dispatches)
        if (int rc = run_dispatch(s, d)) return rc;
    if (s->greedy) {
        const Node &lo = s->nodes[s->greedy_output];
        const int rc = mgq_argmax(static_cast<const float *>(s->ptr(s->greedy_output)), (uint32_t)lo.elements(), s->greedy_ws,
                                  s->greedy_token, static_cast<uint32_t *>(s->ptr(s->greedy_token_input)),
                                  static_cast<uint32_t *>(s->ptr(s->greedy_pos_input)), s->greedy_history, s->greedy_cap, s->stream);
        if (rc) return rc;
    }
    return end_token(s);
}

// Profiled step (Session::step with profiling on, src/runtime.rs:2851-2861): every dispatch on its own,
// bracketed by events and an NVTX range named by its label; the captured graph is not used.
static int enqueue_profiled(mgq_session *s)
{
    const size_t n = s->dispatches.size();
    while (s->events.size() < n + 1) {
        cudaEvent_t e = nullptr;
        MGQ_CUDA(cudaEventCreate(&e));
        s->events.push_back(e);
    }
    for (size_t i = 0; i < n; i++) {
        MGQ_CUDA(cudaEventRecord(s->events[i], s->stream));
        nvtxRangePushA(s->dispatches[i].label.c_str());
        const int rc = run_dispatch(s, s->dispatches[i]);
        nvtxRangePop();
        if (rc) return rc;
    }
    MGQ_CUDA(cudaEventRecord(s->events[n], s->stream));
    if (s->greedy) {
        const Node &lo = s->nodes[s->greedy_output];
        if (int rc = mgq_argmax(static_cast<const float *>(s->ptr(s->greedy_output)), (uint32_t)lo.elements(), s->greedy_ws,
                                s->greedy_token, static_cast<uint32_t *>(s->ptr(s->greedy_token_input)),
                                static_cast<uint32_t *>(s->ptr(s->greedy_pos_input)), s->greedy_history, s->greedy_cap, s->stream))
            return rc;
    }
    s->profiled = true;
    return end_token(s);
}

int mgq_session_step(mgq_session *s)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    MGQ_CUDA(cudaSetDevice(s->device));
    if (int rc = exchanges_bound(s)) return rc;
    nvtxRangePushA("step");                      // the reference's span name (src/runtime.rs:2843)
    int rc = MGQ_OK;
    if (s->profiling) {
        rc = enqueue_profiled(s);
    } else if (s->graph_exec) {
        rc = mgq::cuda_check((int)cudaGraphLaunch(s->graph_exec, s->stream), "cudaGraphLaunch", __FILE__, __LINE__);
    } else {
        rc = enqueue_all(s);
    }
    nvtxRangePop();
    if (rc) return rc;
    s->launches += s->dispatches.size() + (s->greedy ? 1 : 0) + (s->exchanges.empty() ? 0 : 1);
    return MGQ_OK;
}

int mgq_session_num_exchanges(const mgq_session *s) { return s ? (int)s->exchanges.size() : -fail(MGQ_ERR_NULL, "null session"); }

int mgq_session_exchange_info(const mgq_session *s, size_t index, uint32_t *slice_len, uint32_t *world)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    if (index >= s->exchanges.size()) return fail(MGQ_ERR_NAME, "exchange index %zu out of range", index);
    if (slice_len) *slice_len = s->exchanges[index].slice_len;
    if (world) *world = s->exchanges[index].world;
    return MGQ_OK;
}

int mgq_session_bind_exchange(mgq_session *s, size_t index, const mgq_exchange_push *push_dev, mgq_exchange_elem *local_vec)
{
    if (!s || !push_dev || !local_vec) return fail(MGQ_ERR_NULL, "null argument");
    if (index >= s->exchanges.size()) return fail(MGQ_ERR_NAME, "exchange index %zu out of range", index);
    if (s->graph_exec) return fail(MGQ_ERR_STATE, "bind exchanges before mgq_session_capture");
    if (reinterpret_cast<uintptr_t>(local_vec) % 16 != 0) return fail(MGQ_ERR_ALIGN, "the gathered vector must be 16-byte aligned");
    mgq_exchange_push rec;
    MGQ_CUDA(cudaMemcpy(&rec, push_dev, sizeof rec, cudaMemcpyDeviceToHost));
    const Exchange &ex = s->exchanges[index];
    if (rec.world != ex.world || rec.rank >= rec.world || rec.gather_cols != ex.slice_len)
        return fail(MGQ_ERR_SHAPE, "exchange %zu: the push record (world %u, rank %u, %u columns) does not fit the all_gather (world %u, %u columns)",
                    index, rec.world, rec.rank, rec.gather_cols, ex.world, ex.slice_len);
    s->exchanges[index].push_dev = push_dev;
    s->exchanges[index].local_vec = local_vec;
    return MGQ_OK;
}

int mgq_session_bind_exchange_state(mgq_session *s, unsigned long long *epoch, unsigned int *error, unsigned int *blocks_done)
{
    if (!s || !epoch || !error || !blocks_done) return fail(MGQ_ERR_NULL, "null argument");
    if (s->graph_exec) return fail(MGQ_ERR_STATE, "bind exchanges before mgq_session_capture");
    s->xchg_epoch = epoch; s->xchg_error = error; s->xchg_blocks = blocks_done;
    return MGQ_OK;
}

int mgq_session_check_exchange(mgq_session *s)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    if (s->exchanges.empty() || !s->xchg_error) return MGQ_OK;
    MGQ_CUDA(cudaStreamSynchronize(s->stream));
    unsigned int err = 0;
    MGQ_CUDA(cudaMemcpy(&err, s->xchg_error, sizeof err, cudaMemcpyDeviceToHost));
    if (!err) return MGQ_OK;
    MGQ_CUDA(cudaMemset(s->xchg_error, 0, sizeof err));
    return fail(MGQ_ERR_TIMEOUT, "a wait for another rank's part of a gathered vector ran out");
}

int mgq_session_set_profiling(mgq_session *s, int enabled)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    s->profiling = enabled != 0;
    return MGQ_OK;
}

int mgq_session_gpu_timings(mgq_session *s, float *microseconds, size_t count)
{
    if (!s || !microseconds) return fail(MGQ_ERR_NULL, "null argument");
    if (!s->profiled) return fail(MGQ_ERR_STATE, "no profiled step yet: call mgq_session_set_profiling(s, 1) and step");
    if (count != s->dispatches.size()) return fail(MGQ_ERR_SIZE, "the plan has %zu dispatches, asked for %zu timings", s->dispatches.size(), count);
    MGQ_CUDA(cudaStreamSynchronize(s->stream));
    for (size_t i = 0; i < count; i++) {
        float ms = 0.f;
        MGQ_CUDA(cudaEventElapsedTime(&ms, s->events[i], s->events[i + 1]));
        microseconds[i] = ms * 1000.f;
    }
    return MGQ_OK;
}

int mgq_session_dump_gpu_timings(mgq_session *s, char *out, size_t cap)
{
    if (!s || !out || cap == 0) return fail(MGQ_ERR_NULL, "null argument");
    out[0] = 0;
    std::vector<float> us(s->dispatches.size());
    if (int rc = mgq_session_gpu_timings(s, us.data(), us.size())) return rc;
    // aggregated by pass name like Session::dump_gpu_timings (src/runtime.rs:2798-2832); a pass is named by its label
    std::map<std::string, std::pair<unsigned, double>> by_label;
    double total = 0.0;
    for (size_t i = 0; i < us.size(); i++) {
        auto &e = by_label[s->dispatches[i].label];
        e.first++;
        e.second += us[i];
        total += us[i];
    }
    std::vector<std::pair<std::string, std::pair<unsigned, double>>> rows(by_label.begin(), by_label.end());
    std::sort(rows.begin(), rows.end(), [](const auto &a, const auto &b) { return a.second.second > b.second.second; });
    size_t at = 0;
    auto put = [&](const char *fmt, auto... args) {
        if (at + 1 >= cap) return;
        const int n = std::snprintf(out + at, cap - at, fmt, args...);
        if (n > 0) at += std::min((size_t)n, cap - at - 1);
    };
    put("--- GPU pass timings (%zu passes, %.2fms total) ---\n", us.size(), total / 1000.0);
    for (const auto &r : rows)
        put("  %32s: %3ux %8.3fms (%5.1f%%)\n", r.first.c_str(), r.second.first, r.second.second / 1000.0,
            total > 0 ? r.second.second / total * 100.0 : 0.0);
    put("---\n");
    return MGQ_OK;
}

int mgq_session_num_groups(const mgq_session *s)
{
    if (!s) return -fail(MGQ_ERR_NULL, "null session");
    const size_t n = s->dispatches.size();
    std::vector<int32_t> ins(n * 4), outs(n * 4);
    auto buf = [&](int node) { return node < 0 ? -1 : s->node_buffer[node]; };
    for (size_t i = 0; i < n; i++) {
        const Dispatch &d = s->dispatches[i];
        for (int j = 0; j < 4; j++) ins[i * 4 + j] = buf(d.in[j]);
        outs[i * 4] = buf(d.out);
        for (int j = 0; j < 3; j++) outs[i * 4 + 1 + j] = buf(d.extra[j]);
    }
    return mgq_barrier_groups(ins.data(), outs.data(), n, 1);
}

int mgq_session_capture(mgq_session *s)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    // the first launch of a kernel sets function attributes and asks for its occupancy: keep that out of the capture
    if (s->launches == 0) return fail(MGQ_ERR_STATE, "run one step before capturing the session");
    MGQ_CUDA(cudaSetDevice(s->device));
    if (s->graph_exec) { cudaGraphExecDestroy(s->graph_exec); s->graph_exec = nullptr; }
    if (s->graph) { cudaGraphDestroy(s->graph); s->graph = nullptr; }
    MGQ_CUDA(cudaStreamSynchronize(s->stream));
    MGQ_CUDA(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
    const int rc = enqueue_all(s);
    cudaGraph_t graph = nullptr;
    const cudaError_t end = cudaStreamEndCapture(s->stream, &graph);
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    MGQ_CUDA(end);
    s->graph = graph;
    MGQ_CUDA(cudaGraphInstantiate(&s->graph_exec, s->graph, 0));
    return MGQ_OK;
}

int mgq_session_enable_greedy(mgq_session *s, size_t output_index, const char *token_input, const char *pos_input, uint32_t history_cap)
{
    if (!s || !token_input || !pos_input) return fail(MGQ_ERR_NULL, "null argument");
    if (s->graph_exec) return fail(MGQ_ERR_STATE, "enable the greedy pick before capturing the session");
    if (output_index >= s->outputs.size()) return fail(MGQ_ERR_NAME, "output index %zu out of range", output_index);
    const int tok = find_named(s, Op::Input, token_input), pos = find_named(s, Op::Input, pos_input);
    if (tok < 0 || pos < 0 || s->nodes[tok].dtype != kU32 || s->nodes[pos].dtype != kU32) return fail(MGQ_ERR_NAME, "greedy feedback needs two u32 inputs");
    if (s->nodes[tok].elements() != 1 || s->nodes[pos].elements() != 1) return fail(MGQ_ERR_SHAPE, "greedy feedback takes one token and one position");
    if (history_cap == 0) return fail(MGQ_ERR_SHAPE, "history capacity must be positive");
    void *p = nullptr;
    if (!s->greedy_ws) {
        if (int rc = mgq_buffer_create(mgq_argmax_workspace(), &s->greedy_ws)) return rc;
        if (int rc = mgq_buffer_create(4, &p)) return rc;
        s->greedy_token = static_cast<uint32_t *>(p);
    }
    if (s->greedy_history) { cudaFree(s->greedy_history); s->greedy_history = nullptr; }
    if (int rc = mgq_buffer_create((size_t)history_cap * 4, &p)) return rc;
    s->greedy_history = static_cast<uint32_t *>(p);
    s->greedy_cap = history_cap;
    s->greedy_output = s->outputs[output_index];
    s->greedy_token_input = tok;
    s->greedy_pos_input = pos;
    s->greedy = true;
    return MGQ_OK;
}

int mgq_session_read_tokens(mgq_session *s, uint32_t first_pos, uint32_t *out, size_t count)
{
    if (!s || !out) return fail(MGQ_ERR_NULL, "null argument");
    if (!s->greedy) return fail(MGQ_ERR_STATE, "the greedy pick is not enabled");
    if ((size_t)first_pos + count > s->greedy_cap) return fail(MGQ_ERR_SIZE, "history holds %u positions", s->greedy_cap);
    return mgq_buffer_download(s->greedy_history + first_pos, out, count * 4, s->stream);
}

int mgq_session_wait(mgq_session *s)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    nvtxRangePushA("wait");                      // the reference's span name (src/runtime.rs:2835)
    const int rc = mgq::cuda_check((int)cudaStreamSynchronize(s->stream), "cudaStreamSynchronize", __FILE__, __LINE__);
    nvtxRangePop();
    return rc;
}

int mgq_session_read_output_by_index(mgq_session *s, size_t index, float *out, size_t len)
{
    if (!s || !out) return fail(MGQ_ERR_NULL, "null argument");
    if (index >= s->outputs.size()) return fail(MGQ_ERR_NAME, "output index %zu out of range", index);
    const int id = s->outputs[index];
    if (len > s->nodes[id].elements()) return fail(MGQ_ERR_SIZE, "output has %zu elements, asked for %zu", s->nodes[id].elements(), len);
    return mgq_buffer_download(s->ptr(id), out, len * 4, s->stream);
}

int mgq_session_read_output(mgq_session *s, float *out, size_t len) { return mgq_session_read_output_by_index(s, 0, out, len); }

int mgq_session_num_dispatches(const mgq_session *s) { return s ? (int)s->dispatches.size() : -fail(MGQ_ERR_NULL, "null session"); }

int mgq_session_dispatch_info(const mgq_session *s, size_t index, int *shader, uint32_t workgroups[3],
                              uint32_t params[4], int *weight_format, char *label, size_t label_cap)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    if (index >= s->dispatches.size()) return fail(MGQ_ERR_NAME, "dispatch index %zu out of range", index);
    const Dispatch &d = s->dispatches[index];
    if (shader) *shader = d.shader;
    if (workgroups) std::memcpy(workgroups, d.workgroups, sizeof d.workgroups);
    if (params) std::memcpy(params, d.params, sizeof d.params);
    if (weight_format) *weight_format = d.weight_format;
    if (label && label_cap) std::snprintf(label, label_cap, "%s", d.label.c_str());
    return MGQ_OK;
}

uint64_t mgq_session_launch_count(const mgq_session *s) { return s ? s->launches : 0; }

}  // extern "C"
