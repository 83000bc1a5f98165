// Graph -> plan -> Session for the quantized-matmul path, behind the C ABI.
//
// Mirrors, for this path only, meganeura's builder and runtime surface:
//   Graph::{input, parameter, parameter_q4, parameter_q8, matmul, add, set_outputs}
//                                                        src/graph.rs:714-795
//   MatMul+Add -> FusedMatMulAdd                          src/optimize.rs:724-767
//   Op::MatMul / Op::FusedMatMulAdd lowering, labels      src/compile.rs:1381-1421, 1486-1524, 1275-1285
//   build_inference_session                               src/train.rs:380-389
//   Session::{set_parameter, upload_param, set_input, step, wait, read_output*}
//                                                        src/runtime.rs:2327-2345, 2786-2791, 2496-2550,
//                                                        2835-2959, 2612-2643
// One session = one device = one stream with the dispatches enqueued in plan order; kernels run
// asynchronously until wait().  Where the reference panics, these calls return a status.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "mgq_internal.h"

namespace {

enum class Op { Input, Parameter, MatMul, Add, FusedMatMulAdd, Nop };

struct Node {
    Op op;
    std::string name;
    std::vector<size_t> shape;
    int dtype;                    // MGQ_FMT_F32 / Q4 / Q8
    std::vector<int> inputs;
    size_t elements() const { size_t e = 1; for (size_t s : shape) e *= s; return e; }
};

struct Dispatch {
    int shader;
    uint32_t workgroups[3];
    uint32_t params[4];           // [m, k, n, 0] like the reference
    int in_a, in_b, in_d;         // buffer indices (in_d = -1 when there is no addend)
    int out;
    int weight_format;
    std::string label;
};

struct Buffer {
    size_t bytes = 0;
    void *dev = nullptr;
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
    }
    return "?";
}

}  // namespace

struct mgq_graph {
    std::vector<Node> nodes;
    std::vector<int> outputs;
};

struct mgq_session {
    std::vector<Node> nodes;                   // after fusion
    std::vector<int> outputs;
    std::vector<int> node_buffer;              // node id -> buffer index (-1 for Nop)
    std::vector<Buffer> buffers;
    std::vector<Dispatch> dispatches;
    std::vector<uint8_t> staging;              // host scratch for quantize-on-upload
    cudaStream_t stream = nullptr;
    uint64_t launches = 0;
    int device = 0;
};

using mgq::fail;

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

extern "C" {

mgq_graph *mgq_graph_new(void) { return new mgq_graph(); }
void mgq_graph_free(mgq_graph *g) { delete g; }

int mgq_graph_input(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Input, name, shape, rank, MGQ_FMT_F32); }
int mgq_graph_parameter(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Parameter, name, shape, rank, MGQ_FMT_F32); }
int mgq_graph_parameter_q4(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Parameter, name, shape, rank, MGQ_FMT_Q4); }
int mgq_graph_parameter_q8(mgq_graph *g, const char *name, const size_t *shape, size_t rank)
{ return add_leaf(g, Op::Parameter, name, shape, rank, MGQ_FMT_Q8); }

int mgq_graph_matmul(mgq_graph *g, int a, int b)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    const int nn = (int)g->nodes.size();
    if (a < 0 || b < 0 || a >= nn || b >= nn) return -fail(MGQ_ERR_NAME, "matmul: node id out of range");
    const Node &na = g->nodes[a], &nb = g->nodes[b];
    if (na.shape.size() != 2 || nb.shape.size() != 2) return -fail(MGQ_ERR_SHAPE, "matmul requires 2D tensors");
    if (na.shape[1] != nb.shape[0]) return -fail(MGQ_ERR_SHAPE, "matmul inner dimensions must match (%zu vs %zu)", na.shape[1], nb.shape[0]);
    if (mgq::is_quant(na.dtype)) return -fail(MGQ_ERR_FORMAT, "matmul: the left operand cannot be quantized");
    g->nodes.push_back(Node{Op::MatMul, "", {na.shape[0], nb.shape[1]}, MGQ_FMT_F32, {a, b}});
    return (int)g->nodes.size() - 1;
}

int mgq_graph_add(mgq_graph *g, int a, int b)
{
    if (!g) return -fail(MGQ_ERR_NULL, "null graph");
    const int nn = (int)g->nodes.size();
    if (a < 0 || b < 0 || a >= nn || b >= nn) return -fail(MGQ_ERR_NAME, "add: node id out of range");
    const Node &na = g->nodes[a], &nb = g->nodes[b];
    if (na.shape != nb.shape) return -fail(MGQ_ERR_SHAPE, "add: shapes differ");
    if (mgq::is_quant(na.dtype) || mgq::is_quant(nb.dtype)) return -fail(MGQ_ERR_FORMAT, "add: quantized operand");
    g->nodes.push_back(Node{Op::Add, "", na.shape, MGQ_FMT_F32, {a, b}});
    return (int)g->nodes.size() - 1;
}

int mgq_graph_set_outputs(mgq_graph *g, const int *ids, size_t count)
{
    if (!g || !ids) return fail(MGQ_ERR_NULL, "null argument");
    for (size_t i = 0; i < count; i++)
        if (ids[i] < 0 || ids[i] >= (int)g->nodes.size()) return fail(MGQ_ERR_NAME, "set_outputs: node id out of range");
    g->outputs.assign(ids, ids + count);
    return MGQ_OK;
}

int mgq_build_inference_session(const mgq_graph *g, mgq_session **out)
{
    if (!g || !out) return fail(MGQ_ERR_NULL, "null argument");
    *out = nullptr;
    if (g->outputs.empty()) return fail(MGQ_ERR_STATE, "graph has no outputs");
    mgq_session *s = new mgq_session();
    s->nodes = g->nodes;
    s->outputs = g->outputs;
    auto is_output = [&](int id) { for (int o : s->outputs) if (o == id) return true; return false; };

    // MatMul + Add -> FusedMatMulAdd when the matmul has exactly one use and is not an output.
    for (size_t id = 0; id < s->nodes.size(); id++) {
        if (s->nodes[id].op != Op::Add) continue;
        const int lhs = s->nodes[id].inputs[0], rhs = s->nodes[id].inputs[1];
        int mm, addend;
        if (s->nodes[lhs].op == Op::MatMul) { mm = lhs; addend = rhs; }
        else if (s->nodes[rhs].op == Op::MatMul) { mm = rhs; addend = lhs; }
        else continue;
        int uses = 0;
        for (const Node &nd : s->nodes)
            if (nd.op != Op::Nop)
                for (int in : nd.inputs) if (in == mm) { uses++; break; }
        if (uses != 1 || is_output(mm)) continue;
        const int a = s->nodes[mm].inputs[0], b = s->nodes[mm].inputs[1];
        s->nodes[id].op = Op::FusedMatMulAdd;
        s->nodes[id].inputs = {a, b, addend};
        s->nodes[mm].op = Op::Nop;
        s->nodes[mm].inputs.clear();
    }

    // One buffer per live node; quantized parameters are sized by blocks.
    s->node_buffer.assign(s->nodes.size(), -1);
    for (size_t id = 0; id < s->nodes.size(); id++) {
        const Node &nd = s->nodes[id];
        if (nd.op == Op::Nop) continue;
        Buffer buf;
        buf.bytes = mgq::is_quant(nd.dtype) ? mgq_packed_bytes(nd.dtype, nd.shape[0], nd.shape[1]) : nd.elements() * 4;
        s->node_buffer[id] = (int)s->buffers.size();
        s->buffers.push_back(buf);
    }

    // Lowering, in node (= topological) order.
    for (size_t id = 0; id < s->nodes.size(); id++) {
        const Node &nd = s->nodes[id];
        if (nd.op == Op::MatMul || nd.op == Op::FusedMatMulAdd) {
            const Node &na = s->nodes[nd.inputs[0]], &nb = s->nodes[nd.inputs[1]];
            if (nb.op != Op::Parameter || !mgq::is_quant(nb.dtype)) {
                delete s;
                return fail(MGQ_ERR_FORMAT, "matmul weight must be a parameter_q4 / parameter_q8 node (f32/f16 weights are outside this library)");
            }
            const bool fused = nd.op == Op::FusedMatMulAdd;
            Dispatch d{};
            const uint32_t m = (uint32_t)na.shape[0], k = (uint32_t)na.shape[1], n = (uint32_t)nb.shape[1];
            if (m == 1 && n % 4 == 0) {
                d.shader = fused ? MGQ_SHADER_MATMUL_GEMV_ADD : MGQ_SHADER_MATMUL_GEMV;
                d.workgroups[0] = n / 4; d.workgroups[1] = 1; d.workgroups[2] = 1;
            } else {
                d.shader = fused ? MGQ_SHADER_FUSED_MATMUL_ADD : MGQ_SHADER_MATMUL;
                d.workgroups[0] = (n + 63) / 64; d.workgroups[1] = (m + 63) / 64; d.workgroups[2] = 1;
            }
            d.params[0] = m; d.params[1] = k; d.params[2] = n; d.params[3] = 0;
            d.in_a = s->node_buffer[nd.inputs[0]];
            d.in_b = s->node_buffer[nd.inputs[1]];
            d.in_d = fused ? s->node_buffer[nd.inputs[2]] : -1;
            d.out = s->node_buffer[id];
            d.weight_format = nb.dtype;
            char lab[96];
            std::snprintf(lab, sizeof lab, "%s[%ux%ux%u]", shader_name(d.shader), m, n, k);
            d.label = lab;
            s->dispatches.push_back(d);
        } else if (nd.op == Op::Add) {
            Dispatch d{};
            d.shader = MGQ_SHADER_ADD;
            const uint32_t len = (uint32_t)nd.elements();
            d.workgroups[0] = (len + 255) / 256; d.workgroups[1] = 1; d.workgroups[2] = 1;
            d.params[0] = len;
            d.in_a = s->node_buffer[nd.inputs[0]];
            d.in_b = s->node_buffer[nd.inputs[1]];
            d.in_d = -1;
            d.out = s->node_buffer[id];
            d.weight_format = MGQ_FMT_F32;
            char lab[64];
            std::snprintf(lab, sizeof lab, "Add[%u]", len);
            d.label = lab;
            s->dispatches.push_back(d);
        }
    }

    int rc = mgq::cuda_check((int)cudaGetDevice(&s->device), "cudaGetDevice", __FILE__, __LINE__);
    if (!rc) rc = mgq::cuda_check((int)cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking), "cudaStreamCreate", __FILE__, __LINE__);
    for (Buffer &b : s->buffers) {
        if (rc) break;
        rc = mgq_buffer_create(b.bytes, &b.dev);     // zero-filled, like the reference
    }
    if (rc) { mgq_session_free(s); return rc; }
    *out = s;
    return MGQ_OK;
}

void mgq_session_free(mgq_session *s)
{
    if (!s) return;
    if (s->stream) cudaStreamSynchronize(s->stream);
    for (Buffer &b : s->buffers) if (b.dev) cudaFree(b.dev);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

static int find_named(const mgq_session *s, Op op, const char *name)
{
    for (size_t id = 0; id < s->nodes.size(); id++)
        if (s->nodes[id].op == op && s->nodes[id].name == name) return (int)id;
    return -1;
}

int mgq_session_set_parameter(mgq_session *s, const char *name, const float *data, size_t len)
{
    if (!s || !name || !data) return fail(MGQ_ERR_NULL, "null argument");
    const int id = find_named(s, Op::Parameter, name);
    if (id < 0) return fail(MGQ_ERR_NAME, "unknown parameter: %s", name);
    const Node &nd = s->nodes[id];
    if (len != nd.elements()) return fail(MGQ_ERR_SIZE, "parameter '%s' has %zu elements, got %zu", name, nd.elements(), len);
    Buffer &buf = s->buffers[s->node_buffer[id]];
    if (!mgq::is_quant(nd.dtype)) return mgq_buffer_upload(buf.dev, data, len * 4, s->stream);
    s->staging.resize(buf.bytes);
    const int rc = nd.dtype == MGQ_FMT_Q4 ? mgq_quantize_q4(data, nd.shape[0], nd.shape[1], s->staging.data())
                                          : mgq_quantize_q8(data, nd.shape[0], nd.shape[1], s->staging.data());
    if (rc) return rc;
    return mgq_buffer_upload(buf.dev, s->staging.data(), buf.bytes, s->stream);
}

int mgq_session_upload_param(mgq_session *s, const char *name, const void *bytes, size_t nbytes)
{
    if (!s || !name || !bytes) return fail(MGQ_ERR_NULL, "null argument");
    const int id = find_named(s, Op::Parameter, name);
    if (id < 0) return fail(MGQ_ERR_NAME, "unknown parameter: %s", name);
    Buffer &buf = s->buffers[s->node_buffer[id]];
    if (nbytes != buf.bytes) return fail(MGQ_ERR_SIZE, "parameter '%s' buffer is %zu bytes, got %zu", name, buf.bytes, nbytes);
    return mgq_buffer_upload(buf.dev, bytes, nbytes, s->stream);
}

int mgq_session_set_input(mgq_session *s, const char *name, const float *data, size_t len)
{
    if (!s || !name || !data) return fail(MGQ_ERR_NULL, "null argument");
    const int id = find_named(s, Op::Input, name);
    if (id < 0) return fail(MGQ_ERR_NAME, "unknown input: %s", name);
    const Node &nd = s->nodes[id];
    if (len != nd.elements()) return fail(MGQ_ERR_SIZE, "input '%s' has %zu elements, got %zu", name, nd.elements(), len);
    return mgq_buffer_upload(s->buffers[s->node_buffer[id]].dev, data, len * 4, s->stream);
}

int mgq_session_step(mgq_session *s)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    MGQ_CUDA(cudaSetDevice(s->device));
    for (const Dispatch &d : s->dispatches) {
        float *outp = static_cast<float *>(s->buffers[d.out].dev);
        if (d.shader == MGQ_SHADER_ADD) {
            add_kernel<<<d.workgroups[0], 256, 0, s->stream>>>(static_cast<const float *>(s->buffers[d.in_a].dev),
                                                                static_cast<const float *>(s->buffers[d.in_b].dev), outp, d.params[0]);
            MGQ_CUDA(cudaGetLastError());
        } else {
            const float *addend = d.in_d >= 0 ? static_cast<const float *>(s->buffers[d.in_d].dev) : nullptr;
            const int rc = mgq_matmul(d.weight_format, s->buffers[d.in_a].dev, MGQ_A_F32, s->buffers[d.in_b].dev, addend, outp,
                                      d.params[0], d.params[1], d.params[2], s->stream);
            if (rc) return rc;
        }
        s->launches++;
    }
    return MGQ_OK;
}

int mgq_session_wait(mgq_session *s)
{
    if (!s) return fail(MGQ_ERR_NULL, "null session");
    MGQ_CUDA(cudaStreamSynchronize(s->stream));
    return MGQ_OK;
}

int mgq_session_read_output_by_index(mgq_session *s, size_t index, float *out, size_t len)
{
    if (!s || !out) return fail(MGQ_ERR_NULL, "null argument");
    if (index >= s->outputs.size()) return fail(MGQ_ERR_NAME, "output index %zu out of range", index);
    const int id = s->outputs[index];
    if (len > s->nodes[id].elements()) return fail(MGQ_ERR_SIZE, "output has %zu elements, asked for %zu", s->nodes[id].elements(), len);
    return mgq_buffer_download(s->buffers[s->node_buffer[id]].dev, out, len * 4, s->stream);
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
