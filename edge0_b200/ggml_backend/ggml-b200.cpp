// ggml backend over the B200 MoE-FFN C ABI (edge0_b200_moe.h).
//
// Compiled against the host application's ggml headers (ggml.h, ggml-backend.h and the interface structs in
// src/ggml-backend-impl.h); the ggml symbols it calls are resolved from the host application's ggml at load time.
// Device memory and copies use the CUDA runtime directly, compute goes through the b200moe_* entry points only.
//
// graph_compute recognises the sub-graphs that Builder::route / Builder::ffn emit
// (edge0-infer/src/models/edge0_35b/forward.cpp:262-271, 300-311) and runs each as one fused call, the way the reference's
// CUDA backend fuses its top-k MoE and MUL_MAT_ID + scale patterns (third_party/ggml/src/ggml-cuda/ggml-cuda.cu:3655-3673).
// Every other node it says it supports - the F32 operators around those sub-graphs, among them the shared expert and its
// sigmoid gate (forward.cpp:312-314) - runs as one operator call (b200moe_op_*), so supports_op promises nothing that
// graph_compute refuses (edge0-infer accepts a plan on supports_op and drops a backend for good on the first failed status,
// src/exec/execution.cpp:256-260, 404-407).
// A failure that only shows on the device (a rejected expert id, a wait that ran out) is latched when synchronize finds it and
// returned by the next graph_compute, empty graphs included: that is how the application confirms completion
// (src/platform/backend.cpp:151-159).
#include "ggml-b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "ggml-backend-impl.h"
#include "edge0_b200_moe.h"

namespace {

constexpr int    MAX_DEVICES = 16;
constexpr size_t ALIGNMENT   = 256;

struct DeviceCtx {
    int         index = 0;
    std::string name;
    std::string description;
};

struct BackendCtx {
    int           device = 0;
    b200moe_ctx * moe    = nullptr;
    cudaStream_t  stream = nullptr;
    char *        scratch = nullptr;       // results that cannot be written into graph memory at the time they are computed
    size_t        scratch_bytes = 0;
    ggml_b200_graph_stats stats = {};
    std::string   error;
    bool          failed = false;          // a device-side failure was found by synchronize and not yet reported
    struct GraphPlan * plan = nullptr;     // analysis of the last graph, reused while the graph stays the same
    uint64_t      plan_key = 0;
};

void free_plan(BackendCtx * b);

void set_error(BackendCtx * b, const char * fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    b->error = buf;
    fprintf(stderr, "ggml-b200: %s\n", buf);
}

// ------------------------------------------------------------------------------------------------ buffers

struct BufferCtx {
    int    device = 0;
    void * base   = nullptr;
};

void buffer_free(ggml_backend_buffer_t buffer) {
    auto * c = (BufferCtx *) buffer->context;
    cudaSetDevice(c->device);
    cudaFree(c->base);
    delete c;
}

void * buffer_get_base(ggml_backend_buffer_t buffer) { return ((BufferCtx *) buffer->context)->base; }

// Blocking transfers run on the calling thread's own stream, so they neither wait for nor stall a backend stream;
// ggml's contract is that the caller synchronises the backend before it reads results.
void buffer_memset_tensor(ggml_backend_buffer_t buffer, ggml_tensor * t, uint8_t value, size_t offset, size_t size) {
    cudaSetDevice(((BufferCtx *) buffer->context)->device);
    cudaMemsetAsync((char *) t->data + offset, value, size, cudaStreamPerThread);
    cudaStreamSynchronize(cudaStreamPerThread);
}

void buffer_set_tensor(ggml_backend_buffer_t buffer, ggml_tensor * t, const void * data, size_t offset, size_t size) {
    cudaSetDevice(((BufferCtx *) buffer->context)->device);
    cudaMemcpyAsync((char *) t->data + offset, data, size, cudaMemcpyHostToDevice, cudaStreamPerThread);
    cudaStreamSynchronize(cudaStreamPerThread);
}

void buffer_get_tensor(ggml_backend_buffer_t buffer, const ggml_tensor * t, void * data, size_t offset, size_t size) {
    cudaSetDevice(((BufferCtx *) buffer->context)->device);
    cudaMemcpyAsync(data, (const char *) t->data + offset, size, cudaMemcpyDeviceToHost, cudaStreamPerThread);
    cudaStreamSynchronize(cudaStreamPerThread);
}

void buffer_clear(ggml_backend_buffer_t buffer, uint8_t value) {
    auto * c = (BufferCtx *) buffer->context;
    cudaSetDevice(c->device);
    cudaMemsetAsync(c->base, value, buffer->size, cudaStreamPerThread);
    cudaStreamSynchronize(cudaStreamPerThread);
}

const ggml_backend_buffer_i buffer_iface = {
    /* free_buffer   */ buffer_free,
    /* get_base      */ buffer_get_base,
    /* init_tensor   */ nullptr,
    /* memset_tensor */ buffer_memset_tensor,
    /* set_tensor    */ buffer_set_tensor,
    /* get_tensor    */ buffer_get_tensor,
    /* set_tensor_2d */ nullptr,
    /* get_tensor_2d */ nullptr,
    /* cpy_tensor    */ nullptr,
    /* clear         */ buffer_clear,
    /* reset         */ nullptr,
};

const char * buft_get_name(ggml_backend_buffer_type_t buft) { return ((DeviceCtx *) buft->device->context)->name.c_str(); }

ggml_backend_buffer_t buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size) {
    const int device = ((DeviceCtx *) buft->device->context)->index;
    if (cudaSetDevice(device) != cudaSuccess) return nullptr;
    void * p = nullptr;
    if (cudaMalloc(&p, size ? size : 1) != cudaSuccess) {
        cudaGetLastError();
        fprintf(stderr, "ggml-b200: cudaMalloc of %zu bytes failed on device %d\n", size, device);
        return nullptr;
    }
    auto * c = new BufferCtx{device, p};
    return ggml_backend_buffer_init(buft, buffer_iface, c, size);
}

size_t buft_get_alignment(ggml_backend_buffer_type_t) { return ALIGNMENT; }

size_t buft_get_alloc_size(ggml_backend_buffer_type_t, const ggml_tensor * t) {
    // quantised rows are fetched with 16-byte bulk copies: keep a little slack after the last row
    return ggml_nbytes(t) + (ggml_is_quantized(t->type) ? 16 : 0);
}

bool buft_is_host(ggml_backend_buffer_type_t) { return false; }

const ggml_backend_buffer_type_i buft_iface = {
    /* get_name       */ buft_get_name,
    /* alloc_buffer   */ buft_alloc_buffer,
    /* get_alignment  */ buft_get_alignment,
    /* get_max_size   */ nullptr,
    /* get_alloc_size */ buft_get_alloc_size,
    /* is_host        */ buft_is_host,
};

}  // namespace

// ------------------------------------------------------------------------------------------------ graph analysis
namespace {

bool is_expert_type(ggml_type t) { return t == GGML_TYPE_Q3_K || t == GGML_TYPE_NVFP4; }
bool is_view_op(ggml_op op) {
    return op == GGML_OP_NONE || op == GGML_OP_VIEW || op == GGML_OP_RESHAPE || op == GGML_OP_PERMUTE || op == GGML_OP_TRANSPOSE;
}
bool has_flag(const ggml_tensor * t, int f) { return (t->flags & f) != 0; }
float op_param_f32(const ggml_tensor * t, int i) { float v; memcpy(&v, (const char *) t->op_params + 4 * i, 4); return v; }
int32_t op_param_i32(const ggml_tensor * t, int i) { int32_t v; memcpy(&v, (const char *) t->op_params + 4 * i, 4); return v; }
bool is_mat(const ggml_tensor * t, int64_t n0, int64_t n1) { return t->ne[0] == n0 && t->ne[1] == n1 && t->ne[2] == 1 && t->ne[3] == 1; }
bool is_3d(const ggml_tensor * t, int64_t n0, int64_t n1, int64_t n2) { return t->ne[0] == n0 && t->ne[1] == n1 && t->ne[2] == n2 && t->ne[3] == 1; }

enum GroupKind { GROUP_ROUTE, GROUP_FFN, GROUP_DENSE };

// A tensor the fused call has to leave in graph memory.  ggml's graph allocator gives a tensor its memory only from
// its own node position on, and that memory may belong to another live tensor earlier.  The fused call runs at the
// position of the group's FIRST node, so a result is written straight into graph memory only when nothing read
// between that position and the tensor's own overlaps it; otherwise it goes to backend scratch and is copied into
// place when execution reaches the tensor's own node.
struct Materialised {
    ggml_tensor * t = nullptr;
    int     node = -1;          // index of t in the graph
    size_t  bytes = 0;          // contiguous payload produced by the kernels
    size_t  width = 0, pitch = 0, rows = 0;   // width != 0: the graph tensor is row-strided (pitch) and gets `rows` rows of `width` bytes
    void *  where = nullptr;    // where the kernels write: graph memory or scratch
    bool    deferred = false;
    bool    always_scratch = false;
};

struct Group {
    GroupKind kind;
    int first = 1 << 30, last = -1;
    int exec_at = -1;   // node position at which the fused call is issued: the first member that reads a group input
    std::vector<int> members;
    // route
    ggml_tensor *x = nullptr, *rw = nullptr, *rb = nullptr, *logits = nullptr, *probs = nullptr, *argsort = nullptr,
                *ids_view = nullptr, *wts = nullptr;
    // ffn
    ggml_tensor *input = nullptr, *wg = nullptr, *wu = nullptr, *wd = nullptr, *sg = nullptr, *su = nullptr, *sd = nullptr,
                *ids = nullptr, *weights = nullptr, *hid = nullptr, *down = nullptr, *result = nullptr;
    // dense
    ggml_tensor *w = nullptr, *scale = nullptr, *dst = nullptr;
    int64_t E = 0, K = 0, T = 0, H = 0, I = 0, L = 0;
    // outputs, by role
    Materialised m_logits, m_probs, m_ids, m_argsort, m_wts, m_hid, m_down, m_result;
};

struct GraphPlan {
    int n = 0;
    std::vector<ggml_tensor *> nodes;
    std::unordered_map<const ggml_tensor *, int> index;
    std::vector<std::vector<int>> consumers;
    std::vector<int> group_of;
    std::vector<Group> groups;
    std::vector<std::vector<Materialised *>> deferred_at;   // per node: copies to do when execution reaches it
    std::unordered_map<const ggml_tensor *, const void *> resolved;   // tensors whose current values live outside graph memory
    size_t scratch_need = 0;
};

int node_index(const GraphPlan & p, const ggml_tensor * t) {
    auto it = p.index.find(t);
    return it == p.index.end() ? -1 : it->second;
}

void add_member(GraphPlan & p, Group & g, const ggml_tensor * t) {
    const int i = node_index(p, t);
    if (i < 0) return;
    for (int m : g.members) if (m == i) return;
    g.members.push_back(i);
    if (i < g.first) g.first = i;
    if (i > g.last) g.last = i;
}

bool in_group(const Group & g, int idx) {
    for (int m : g.members) if (m == idx) return true;
    return false;
}

// true when someone outside the group reads t, or the graph's owner asked for it as an output
bool wanted_outside(const GraphPlan & p, const Group & g, const ggml_tensor * t) {
    if (has_flag(t, GGML_TENSOR_FLAG_OUTPUT)) return true;
    const int i = node_index(p, t);
    if (i < 0) return false;
    for (int c : p.consumers[i]) {
        if (!in_group(g, c)) return true;
    }
    return false;
}

// same, looking through views of t that are members of the group (a reshape of a member is still that member's data)
bool wanted_outside_deep(const GraphPlan & p, const Group & g, const ggml_tensor * t) {
    if (wanted_outside(p, g, t)) return true;
    const int i = node_index(p, t);
    if (i < 0) return false;
    for (int c : p.consumers[i]) {
        const ggml_tensor * ct = p.nodes[c];
        if (in_group(g, c) && is_view_op(ct->op) && ct->src[0] == t && wanted_outside_deep(p, g, ct)) return true;
    }
    return false;
}

// MUL_MAT_ID, optionally followed by the per-expert scale pattern  mul(mm, get_rows(repeat(reshape(scale)), ids))
bool parse_scaled_mmid(GraphPlan & p, Group & g, ggml_tensor * t, ggml_tensor ** mm, ggml_tensor ** scale) {
    *scale = nullptr;
    if (t->op == GGML_OP_MUL_MAT_ID) { *mm = t; add_member(p, g, t); return true; }
    if (t->op != GGML_OP_MUL) return false;
    ggml_tensor * m = t->src[0], * gr = t->src[1];
    if (!m || !gr || m->op != GGML_OP_MUL_MAT_ID || gr->op != GGML_OP_GET_ROWS || gr->src[1] != m->src[2]) return false;
    ggml_tensor * rp = gr->src[0];
    if (!rp || rp->op != GGML_OP_REPEAT) return false;
    ggml_tensor * s = rp->src[0];
    ggml_tensor * rs = nullptr;
    if (s && s->op == GGML_OP_RESHAPE) { rs = s; s = s->src[0]; }
    const int64_t E = m->src[0]->ne[2];
    if (!s || s->type != GGML_TYPE_F32 || ggml_nelements(s) != E || !ggml_is_contiguous(s)) return false;
    if (!is_3d(gr, 1, m->ne[1], m->ne[2])) return false;
    *mm = m; *scale = s;
    add_member(p, g, t); add_member(p, g, m); add_member(p, g, gr); add_member(p, g, rp);
    if (rs) add_member(p, g, rs);
    return true;
}

// Builder::route, anchored at the normalising DIV (forward.cpp:262-271)
bool match_route(GraphPlan & p, int di, Group & g) {
    ggml_tensor * div = p.nodes[di];
    if (div->op != GGML_OP_DIV || div->type != GGML_TYPE_F32) return false;
    ggml_tensor * w2 = div->src[0], * cl = div->src[1];
    if (!w2 || !cl || w2->op != GGML_OP_RESHAPE || cl->op != GGML_OP_CLAMP) return false;
    ggml_tensor * sr = cl->src[0];
    if (!sr || sr->op != GGML_OP_SUM_ROWS || sr->src[0] != w2) return false;
    const float cmin = op_param_f32(cl, 0), cmax = op_param_f32(cl, 1);
    if (cmin != 6.103515625e-5f || !(std::isinf(cmax) && cmax > 0)) return false;
    ggml_tensor * gr = w2->src[0];
    if (!gr || gr->op != GGML_OP_GET_ROWS) return false;
    ggml_tensor * p3 = gr->src[0], * ids = gr->src[1];
    if (!p3 || !ids || p3->op != GGML_OP_RESHAPE || ids->op != GGML_OP_VIEW || ids->type != GGML_TYPE_I32) return false;
    ggml_tensor * probs = p3->src[0];
    if (!probs || probs->op != GGML_OP_SOFT_MAX || probs->src[1] || probs->src[2]) return false;
    if (op_param_f32(probs, 0) != 1.0f || op_param_f32(probs, 1) != 0.0f) return false;
    ggml_tensor * as = ids->src[0];
    if (!as || as->op != GGML_OP_ARGSORT || as->src[0] != probs || op_param_i32(as, 0) != (int32_t) GGML_SORT_ORDER_DESC) return false;
    if (ids->view_offs != 0 || ids->nb[1] != as->nb[1]) return false;
    ggml_tensor * lg = probs->src[0], * mm = lg, * rb = nullptr;
    if (lg && lg->op == GGML_OP_ADD) { mm = lg->src[0]; rb = lg->src[1]; }
    if (!mm || mm->op != GGML_OP_MUL_MAT) return false;
    ggml_tensor * rw = mm->src[0], * x = mm->src[1];
    if (!rw || !x || rw->type != GGML_TYPE_F32 || x->type != GGML_TYPE_F32 || !ggml_is_contiguous(rw) || !ggml_is_contiguous(x)) return false;
    const int64_t H = rw->ne[0], E = rw->ne[1], T = x->ne[1], K = ids->ne[0];
    if (!is_mat(rw, H, E) || !is_mat(x, H, T) || !is_mat(probs, E, T) || !is_mat(div, K, T) || !is_mat(ids, K, T)) return false;
    if (rb && (rb->type != GGML_TYPE_F32 || rb->ne[0] != E || ggml_nelements(rb) != E || !ggml_is_contiguous(rb))) return false;
    if (!is_3d(p3, 1, E, T) || !is_3d(gr, 1, K, T)) return false;

    g.kind = GROUP_ROUTE;
    g.x = x; g.rw = rw; g.rb = rb; g.logits = lg; g.probs = probs; g.argsort = as; g.ids_view = ids; g.wts = div;
    g.E = E; g.K = K; g.T = T; g.H = H;
    g.exec_at = node_index(p, mm);
    for (ggml_tensor * t : { mm, lg, probs, as, ids, p3, gr, w2, sr, cl, div }) add_member(p, g, t);
    // values the fused call never produces must not be wanted by anyone else
    if (rb && wanted_outside_deep(p, g, mm)) return false;
    for (ggml_tensor * t : { gr, sr, cl }) if (wanted_outside_deep(p, g, t)) return false;
    return true;
}

// Builder::ffn, anchored at the multiplication by the route weights (forward.cpp:300-311)
bool match_ffn(GraphPlan & p, int mi, Group & g) {
    ggml_tensor * dw = p.nodes[mi];
    if (dw->op != GGML_OP_MUL || dw->type != GGML_TYPE_F32) return false;
    ggml_tensor * down_s = dw->src[0], * wr = dw->src[1];
    if (!down_s || !wr || wr->op != GGML_OP_RESHAPE) return false;
    ggml_tensor * wts = wr->src[0];
    if (!wts || wts->type != GGML_TYPE_F32 || !ggml_is_contiguous(wts)) return false;
    g.kind = GROUP_FFN;
    ggml_tensor * mm_d = nullptr, * mm_g = nullptr, * mm_u = nullptr;
    if (!parse_scaled_mmid(p, g, down_s, &mm_d, &g.sd)) return false;
    ggml_tensor * hid = mm_d->src[1], * ids = mm_d->src[2];
    if (!hid || hid->op != GGML_OP_MUL) return false;
    ggml_tensor * act = hid->src[0], * up_s = hid->src[1];
    if (!act || !up_s || act->op != GGML_OP_UNARY || ggml_get_unary_op(act) != GGML_UNARY_OP_SILU) return false;
    ggml_tensor * gate_s = act->src[0];
    if (!gate_s || !parse_scaled_mmid(p, g, gate_s, &mm_g, &g.sg) || !parse_scaled_mmid(p, g, up_s, &mm_u, &g.su)) return false;
    if (mm_g->src[1] != mm_u->src[1] || mm_g->src[2] != ids || mm_u->src[2] != ids) return false;
    ggml_tensor * input = mm_g->src[1];
    ggml_tensor * wg = mm_g->src[0], * wu = mm_u->src[0], * wd = mm_d->src[0];
    if (!is_expert_type(wg->type) || wu->type != wg->type || wd->type != wg->type) return false;
    if (!ggml_is_contiguous(wg) || !ggml_is_contiguous(wu) || !ggml_is_contiguous(wd)) return false;
    const int64_t L = wg->ne[0], I = wg->ne[1], E = wg->ne[2], T = input->ne[2], K = ids->ne[0];
    if (!is_3d(wu, L, I, E) || !is_3d(wd, I, L, E) || !is_3d(input, L, 1, T) || input->type != GGML_TYPE_F32 || !ggml_is_contiguous(input)) return false;
    if (ids->type != GGML_TYPE_I32 || !is_mat(ids, K, T) || ids->nb[0] != 4) return false;
    if (!is_mat(wts, K, T) || !is_3d(wr, 1, K, T) || !is_3d(down_s, L, K, T) || !is_3d(hid, I, K, T)) return false;
    for (ggml_tensor * t : { dw, wr, hid, act }) add_member(p, g, t);

    // the sum over slots: K views of dw added left to right
    std::vector<ggml_tensor *> views(K, nullptr);
    const int dwi = node_index(p, dw);
    for (int c : p.consumers[dwi]) {
        ggml_tensor * v = p.nodes[c];
        if (v->op != GGML_OP_VIEW || v->src[0] != dw || !is_mat(v, L, T) || v->nb[1] != dw->nb[2] || v->view_offs % dw->nb[1]) return false;
        const int64_t slot = v->view_offs / dw->nb[1];
        if (slot >= K || views[slot]) return false;
        views[slot] = v;
        add_member(p, g, v);
    }
    for (ggml_tensor * v : views) if (!v) return false;
    ggml_tensor * cur = views[0];
    for (int64_t s = 1; s < K; ++s) {
        ggml_tensor * next = nullptr;
        for (int c : p.consumers[node_index(p, cur)]) {
            ggml_tensor * a = p.nodes[c];
            if (a->op == GGML_OP_ADD && a->src[0] == cur && a->src[1] == views[s]) { next = a; break; }
        }
        if (!next) return false;
        add_member(p, g, next);
        if (cur != views[0] && wanted_outside(p, g, cur)) return false;   // partial sums exist only inside the fused call
        cur = next;
    }
    g.input = input; g.wg = wg; g.wu = wu; g.wd = wd; g.ids = ids; g.weights = wts; g.hid = hid; g.down = down_s; g.result = cur;
    g.E = E; g.K = K; g.T = T; g.I = I; g.L = L;
    g.exec_at = std::min(node_index(p, mm_g), node_index(p, mm_u));
    // values the fused call never produces
    for (ggml_tensor * t : { mm_g, mm_u, gate_s, up_s, act }) if (wanted_outside_deep(p, g, t)) return false;
    if (g.sd && wanted_outside_deep(p, g, mm_d)) return false;
    if (K > 1 && has_flag(dw, GGML_TENSOR_FLAG_OUTPUT)) return false;
    for (int64_t s = 0; s < K; ++s) {
        if (K > 1 && has_flag(views[s], GGML_TENSOR_FLAG_OUTPUT)) return false;
    }
    return true;
}

// dense quantised MUL_MAT, optionally times a one-element scale
bool match_dense(GraphPlan & p, int mi, Group & g) {
    ggml_tensor * mm = p.nodes[mi];
    if (mm->op != GGML_OP_MUL_MAT) return false;
    ggml_tensor * w = mm->src[0], * x = mm->src[1];
    if (!w || !x || !is_expert_type(w->type) || x->type != GGML_TYPE_F32 || !ggml_is_contiguous(w) || !ggml_is_contiguous(x)) return false;
    if (w->ne[2] != 1 || w->ne[3] != 1 || x->ne[2] != 1 || x->ne[3] != 1 || x->ne[0] != w->ne[0]) return false;
    g.kind = GROUP_DENSE;
    g.w = w; g.x = x; g.dst = mm; g.scale = nullptr;
    g.T = x->ne[1];
    g.exec_at = mi;
    add_member(p, g, mm);
    const auto & cons = p.consumers[mi];
    if (cons.size() == 1 && !has_flag(mm, GGML_TENSOR_FLAG_OUTPUT)) {
        ggml_tensor * mul = p.nodes[cons[0]];
        if (mul->op == GGML_OP_MUL && mul->src[0] == mm && mul->src[1] && mul->src[1]->type == GGML_TYPE_F32 &&
            ggml_nelements(mul->src[1]) == 1 && node_index(p, mul->src[1]) < 0) {
            g.scale = mul->src[1];
            g.dst = mul;
            add_member(p, g, mul);
        }
    }
    return true;
}

}  // namespace

// ------------------------------------------------------------------------------------------------ planning
namespace {

size_t align_up(size_t v) { return (v + ALIGNMENT - 1) & ~(ALIGNMENT - 1); }

bool overlaps(const void * a, size_t an, const void * b, size_t bn) {
    const char * a0 = (const char *) a, * b0 = (const char *) b;
    return a0 < b0 + bn && b0 < a0 + an;
}

// Does anything that is read while the graph runs from position `from` up to t's own position live in t's memory?
// (Members of the same group are skipped: the fused call either never touches their memory or writes them itself in
// graph order.)
bool must_defer(const GraphPlan & p, const Group & g, const ggml_tensor * t, int from, int own) {
    const size_t tn = ggml_nbytes(t);
    for (int j = from; j < own; ++j) {
        const ggml_tensor * n = p.nodes[j];
        for (int s = 0; s < GGML_MAX_SRC; ++s) {
            const ggml_tensor * z = n->src[s];
            if (!z || z == t || !z->data) continue;
            const int zi = node_index(p, z);
            if (zi >= 0 && in_group(g, zi)) continue;
            if (overlaps(t->data, tn, z->data, ggml_nbytes(z))) return true;
        }
    }
    return false;
}

// decide where the fused call writes tensor t (own node index `own`) and book scratch if it has to be copied later
void place(GraphPlan & p, const Group & g, Materialised & m, ggml_tensor * t, size_t bytes) {
    m.t = t;
    m.node = node_index(p, t);
    m.bytes = bytes;
    m.deferred = m.always_scratch || must_defer(p, g, t, g.exec_at, m.node);
    if (m.deferred || m.always_scratch) p.scratch_need += align_up(bytes);
}

// inputs of a group must exist when the fused call is issued
bool input_ready(const GraphPlan & p, const ggml_tensor * z, int exec_at) {
    if (!z) return true;
    const int zi = node_index(p, z);
    return zi < exec_at;   // leaves have index -1
}

bool claim(GraphPlan & p, Group & g) {
    for (int m : g.members) if (p.group_of[m] >= 0) return false;
    const int id = (int) p.groups.size();
    for (int m : g.members) p.group_of[m] = id;
    p.groups.push_back(g);
    return true;
}

bool build_plan(BackendCtx * b, ggml_cgraph * cg, GraphPlan & p) {
    p.n = ggml_graph_n_nodes(cg);
    p.nodes.resize(p.n);
    p.consumers.assign(p.n, {});
    p.group_of.assign(p.n, -1);
    p.deferred_at.assign(p.n, {});
    p.index.reserve(p.n * 2);
    for (int i = 0; i < p.n; ++i) { p.nodes[i] = ggml_graph_node(cg, i); p.index[p.nodes[i]] = i; }
    for (int i = 0; i < p.n; ++i) {
        for (int s = 0; s < GGML_MAX_SRC; ++s) {
            const ggml_tensor * z = p.nodes[i]->src[s];
            if (!z) continue;
            const int zi = node_index(p, z);
            if (zi >= 0 && (p.consumers[zi].empty() || p.consumers[zi].back() != i)) p.consumers[zi].push_back(i);
        }
    }
    p.groups.reserve(64);
    for (int i = 0; i < p.n; ++i) {
        if (p.nodes[i]->op != GGML_OP_DIV) continue;
        Group g{};
        if (match_route(p, i, g) && input_ready(p, g.x, g.exec_at) && input_ready(p, g.rw, g.exec_at) && input_ready(p, g.rb, g.exec_at)) claim(p, g);
    }
    for (int i = 0; i < p.n; ++i) {
        if (p.nodes[i]->op != GGML_OP_MUL || p.group_of[i] >= 0) continue;
        Group g{};
        if (!match_ffn(p, i, g)) continue;
        bool ok = input_ready(p, g.input, g.exec_at);
        for (ggml_tensor * w : { g.wg, g.wu, g.wd, g.sg, g.su, g.sd }) ok = ok && input_ready(p, w, g.exec_at);
        // ids and weights either exist already or come from a route group that is issued earlier
        for (ggml_tensor * z : { g.ids, g.weights }) {
            const int zi = node_index(p, z);
            if (zi < g.exec_at) continue;
            const int rg = zi >= 0 ? p.group_of[zi] : -1;
            ok = ok && rg >= 0 && p.groups[rg].kind == GROUP_ROUTE && p.groups[rg].exec_at < g.exec_at;
        }
        if (ok) claim(p, g);
    }
    for (int i = 0; i < p.n; ++i) {
        if (p.nodes[i]->op != GGML_OP_MUL_MAT || p.group_of[i] >= 0) continue;
        Group g{};
        if (match_dense(p, i, g) && input_ready(p, g.x, g.exec_at)) {
            if (!claim(p, g) && g.scale) {
                // the scale multiplication belongs to someone else: run the bare matmul
                Group bare{};
                bare.kind = GROUP_DENSE; bare.w = g.w; bare.x = g.x; bare.dst = p.nodes[i]; bare.T = g.T; bare.exec_at = i;
                add_member(p, bare, p.nodes[i]);
                claim(p, bare);
            }
        }
    }

    // where each group's results go
    for (Group & g : p.groups) {
        const size_t f = sizeof(float);
        if (g.kind == GROUP_ROUTE) {
            g.m_ids.always_scratch = true;   // the kernels write ids densely; the graph's argsort tensor is row-strided
            place(p, g, g.m_ids, g.ids_view, (size_t) g.K * g.T * 4);
            place(p, g, g.m_wts, g.wts, (size_t) g.K * g.T * f);
            if (wanted_outside_deep(p, g, g.logits)) place(p, g, g.m_logits, g.logits, (size_t) g.E * g.T * f);
            if (wanted_outside_deep(p, g, g.probs)) {
                // the reshape that feeds get_rows is a member; readers outside the group are what counts
                place(p, g, g.m_probs, g.probs, (size_t) g.E * g.T * f);
            }
            // the strided top-k columns of the argsort tensor are filled only when someone other than a fused ffn reads them
            bool ext = has_flag(g.argsort, GGML_TENSOR_FLAG_OUTPUT) || has_flag(g.ids_view, GGML_TENSOR_FLAG_OUTPUT);
            for (const ggml_tensor * t : { g.argsort, g.ids_view }) {
                for (int c : p.consumers[node_index(p, t)]) {
                    if (in_group(g, c)) continue;
                    const int cg2 = p.group_of[c];
                    if (cg2 < 0 || p.groups[cg2].kind != GROUP_FFN || p.groups[cg2].ids != g.ids_view) ext = true;
                }
            }
            if (ext) {
                Materialised & m = g.m_argsort;
                m.t = g.argsort; m.node = node_index(p, g.argsort);
                m.width = (size_t) g.K * 4; m.pitch = g.argsort->nb[1]; m.rows = (size_t) g.T;
                m.deferred = must_defer(p, g, g.argsort, g.exec_at, m.node);
            }
        } else if (g.kind == GROUP_FFN) {
            place(p, g, g.m_result, g.result, (size_t) g.L * g.T * f);
            if (wanted_outside_deep(p, g, g.hid)) place(p, g, g.m_hid, g.hid, (size_t) g.I * g.K * g.T * f);
            if (wanted_outside_deep(p, g, g.down)) place(p, g, g.m_down, g.down, (size_t) g.L * g.K * g.T * f);
            if (g.ids->nb[1] != (size_t) g.K * 4) p.scratch_need += align_up((size_t) g.K * g.T * 4);   // dense copy of strided ids
        }
    }
    (void) b;
    return true;
}

}  // namespace

// ------------------------------------------------------------------------------------------------ execution
namespace {

struct Arena {
    char * base = nullptr;
    size_t size = 0, used = 0;
    void * take(size_t bytes) {
        void * p = base + used;
        used += align_up(bytes);
        return p;
    }
};

#define B200_CUDA(b, call)                                                                          \
    do {                                                                                            \
        cudaError_t e_ = (call);                                                                    \
        if (e_ != cudaSuccess) {                                                                    \
            set_error(b, "%s failed: %s", #call, cudaGetErrorString(e_));                           \
            return GGML_STATUS_FAILED;                                                              \
        }                                                                                           \
    } while (0)

const void * current(const GraphPlan & p, const ggml_tensor * t) {
    auto it = p.resolved.find(t);
    return it == p.resolved.end() ? t->data : it->second;
}

void assign(GraphPlan & p, Arena & a, Materialised & m) {
    if (!m.t || m.width) return;
    m.where = (m.deferred || m.always_scratch) ? a.take(m.bytes) : m.t->data;
    if (m.deferred && !m.always_scratch) p.deferred_at[m.node].push_back(&m);
}

ggml_status copy_deferred(BackendCtx * b, const Materialised & m, const void * src) {
    if (m.width) {
        B200_CUDA(b, cudaMemcpy2DAsync(m.t->data, m.pitch, src, m.width, m.width, m.rows, cudaMemcpyDeviceToDevice, b->stream));
    } else {
        B200_CUDA(b, cudaMemcpyAsync(m.t->data, src, m.bytes, cudaMemcpyDeviceToDevice, b->stream));
    }
    return GGML_STATUS_SUCCESS;
}

ggml_status moe_failed(BackendCtx * b, const char * what, int rc) {
    set_error(b, "%s: %s (%s)", what, b200moe_status_string(rc), b200moe_last_error(b->moe));
    return GGML_STATUS_FAILED;
}

ggml_status run_route(BackendCtx * b, GraphPlan & p, Group & g) {
    b200moe_layer l = {};
    l.n_embd = (int32_t) g.H; l.n_expert = (int32_t) g.E; l.n_expert_used = (int32_t) g.K;
    l.router_w = (const float *) g.rw->data;
    l.router_bias = g.rb ? (const float *) g.rb->data : nullptr;
    // scratch is sized per layer shape: describe the experts this routing feeds when the graph shows them
    l.n_ff = (int32_t) g.H; l.wtype = B200MOE_TYPE_NVFP4;
    for (const Group & f : p.groups) {
        if (f.kind == GROUP_FFN && f.ids == g.ids_view && f.L == g.H) { l.n_ff = (int32_t) f.I; l.wtype = (int32_t) f.wg->type; break; }
    }
    b200moe_observe ob = {};
    ob.ffn_moe_logits = (float *) g.m_logits.where;
    ob.ffn_moe_probs  = (float *) g.m_probs.where;
    const int rc = b200moe_route(b->moe, &l, current(p, g.x), B200MOE_TYPE_F32, (int32_t) g.T, (int32_t *) g.m_ids.where,
                                 (float *) g.m_wts.where, &ob, b->stream);
    if (rc) return moe_failed(b, "route", rc);
    p.resolved[g.ids_view] = g.m_ids.where;
    if (g.m_wts.deferred) p.resolved[g.wts] = g.m_wts.where;
    if (g.m_argsort.t) {
        if (g.m_argsort.deferred) p.deferred_at[g.m_argsort.node].push_back(&g.m_argsort);
        else return copy_deferred(b, g.m_argsort, g.m_ids.where);
    }
    return GGML_STATUS_SUCCESS;
}

ggml_status run_ffn(BackendCtx * b, GraphPlan & p, Arena & a, Group & g) {
    b200moe_layer l = {};
    l.n_embd = (int32_t) g.L; l.n_expert = (int32_t) g.E; l.n_expert_used = (int32_t) g.K; l.n_ff = (int32_t) g.I;
    l.wtype = (int32_t) g.wg->type;
    l.gate = g.wg->data; l.up = g.wu->data; l.down = g.wd->data;
    l.gate_scale = g.sg ? (const float *) g.sg->data : nullptr;
    l.up_scale   = g.su ? (const float *) g.su->data : nullptr;
    l.down_scale = g.sd ? (const float *) g.sd->data : nullptr;
    const int32_t * ids = nullptr;
    auto it = p.resolved.find(g.ids);
    if (it != p.resolved.end()) {
        ids = (const int32_t *) it->second;
    } else if (g.ids->nb[1] == (size_t) g.K * 4) {
        ids = (const int32_t *) g.ids->data;
    } else {
        int32_t * dense = (int32_t *) a.take((size_t) g.K * g.T * 4);
        B200_CUDA(b, cudaMemcpy2DAsync(dense, (size_t) g.K * 4, g.ids->data, g.ids->nb[1], (size_t) g.K * 4, (size_t) g.T,
                                       cudaMemcpyDeviceToDevice, b->stream));
        ids = dense;
    }
    b200moe_observe ob = {};
    ob.ffn_moe_hidden = (float *) g.m_hid.where;
    ob.ffn_moe_down   = (float *) g.m_down.where;
    const int rc = b200moe_ffn(b->moe, &l, current(p, g.input), B200MOE_TYPE_F32, (int32_t) g.T, ids, (const float *) current(p, g.weights),
                               (float *) g.m_result.where, &ob, b->stream);
    if (rc) return moe_failed(b, "ffn", rc);
    return GGML_STATUS_SUCCESS;
}

ggml_status run_dense(BackendCtx * b, GraphPlan & p, Group & g) {
    const int rc = b200moe_mul_mat(b->moe, (int) g.w->type, g.w->data, g.w->ne[0], g.w->ne[1], (const float *) current(p, g.x), g.T,
                                   g.scale ? (const float *) g.scale->data : nullptr, (float *) g.dst->data, b->stream);
    if (rc) return moe_failed(b, "mul_mat", rc);
    return GGML_STATUS_SUCCESS;
}

b200moe_tensor as_view(const ggml_tensor * t) {
    b200moe_tensor v;
    v.data = t->data;
    for (int i = 0; i < 4; ++i) { v.ne[i] = t->ne[i]; v.nb[i] = (int64_t) t->nb[i]; }
    return v;
}

bool f32(const ggml_tensor * t) { return t && t->type == GGML_TYPE_F32; }
bool same_shape(const ggml_tensor * a, const ggml_tensor * b) { return a->ne[0] == b->ne[0] && a->ne[1] == b->ne[1] && a->ne[2] == b->ne[2] && a->ne[3] == b->ne[3]; }
bool repeats_over(const ggml_tensor * small, const ggml_tensor * big) {
    for (int i = 0; i < 4; ++i) if (small->ne[i] <= 0 || big->ne[i] % small->ne[i]) return false;
    return true;
}

// Can this node run as one operator call?  The same answer serves supports_op and graph_compute.
bool operator_runs(const ggml_tensor * t) {
    const ggml_tensor * a = t->src[0], * c = t->src[1];
    switch (t->op) {
        case GGML_OP_ADD: case GGML_OP_MUL: case GGML_OP_DIV:
            return f32(t) && f32(a) && f32(c) && same_shape(a, t) && repeats_over(c, t);
        case GGML_OP_UNARY:
            return f32(t) && f32(a) && same_shape(a, t) && (ggml_get_unary_op(t) == GGML_UNARY_OP_SILU || ggml_get_unary_op(t) == GGML_UNARY_OP_SIGMOID);
        case GGML_OP_CLAMP:
            return f32(t) && f32(a) && same_shape(a, t);
        case GGML_OP_REPEAT:
            return f32(t) && f32(a) && repeats_over(a, t);
        case GGML_OP_GET_ROWS:
            return f32(t) && f32(a) && c && c->type == GGML_TYPE_I32 && c->ne[3] == 1 && t->ne[0] == a->ne[0] && t->ne[1] == c->ne[0] &&
                   t->ne[2] == c->ne[1] && t->ne[3] == c->ne[2] && (a->ne[2] == c->ne[1] || a->ne[2] == 1) && (a->ne[3] == c->ne[2] || a->ne[3] == 1);
        case GGML_OP_SUM_ROWS:
            return f32(t) && f32(a) && t->ne[0] == 1 && t->ne[1] == a->ne[1] && t->ne[2] == a->ne[2] && t->ne[3] == a->ne[3];
        case GGML_OP_SOFT_MAX:
            return f32(t) && f32(a) && !t->src[1] && !t->src[2] && same_shape(a, t) && a->ne[0] % 8 == 0 && a->ne[0] <= 1024 && op_param_f32(t, 1) == 0.0f;
        case GGML_OP_ARGSORT:
            return t->type == GGML_TYPE_I32 && f32(a) && same_shape(a, t) && a->ne[0] <= 1024 && op_param_i32(t, 0) == (int32_t) GGML_SORT_ORDER_DESC;
        case GGML_OP_MUL_MAT:
            return f32(t) && f32(a) && f32(c) && ggml_is_contiguous(a) && ggml_is_contiguous(c) && ggml_is_contiguous(t) && a->ne[2] == 1 && a->ne[3] == 1 &&
                   c->ne[2] == 1 && c->ne[3] == 1 && a->ne[0] == c->ne[0] && a->ne[0] % 32 == 0;
        default:
            return false;
    }
}

// returns B200MOE_OK, a positive library status, or -1 when the node is no operator of this backend
int run_operator(BackendCtx * b, ggml_tensor * t) {
    if (!operator_runs(t)) return -1;
    const b200moe_tensor d = as_view(t);
    const b200moe_tensor a = as_view(t->src[0]);
    switch (t->op) {
        case GGML_OP_ADD: case GGML_OP_MUL: case GGML_OP_DIV: {
            const b200moe_tensor c = as_view(t->src[1]);
            const int op = t->op == GGML_OP_ADD ? B200MOE_OP_ADD : t->op == GGML_OP_MUL ? B200MOE_OP_MUL : B200MOE_OP_DIV;
            return b200moe_op_binary(b->moe, op, &a, &c, &d, b->stream);
        }
        case GGML_OP_UNARY:
            return b200moe_op_unary(b->moe, ggml_get_unary_op(t) == GGML_UNARY_OP_SILU ? B200MOE_OP_SILU : B200MOE_OP_SIGMOID, &a, &d, 0.0f, 0.0f, b->stream);
        case GGML_OP_CLAMP:
            return b200moe_op_unary(b->moe, B200MOE_OP_CLAMP, &a, &d, op_param_f32(t, 0), op_param_f32(t, 1), b->stream);
        case GGML_OP_REPEAT:
            return b200moe_op_repeat(b->moe, &a, &d, b->stream);
        case GGML_OP_GET_ROWS: {
            const b200moe_tensor c = as_view(t->src[1]);
            return b200moe_op_get_rows(b->moe, &a, &c, &d, b->stream);
        }
        case GGML_OP_SUM_ROWS:
            return b200moe_op_sum_rows(b->moe, &a, &d, b->stream);
        case GGML_OP_SOFT_MAX:
            return b200moe_op_soft_max(b->moe, &a, &d, op_param_f32(t, 0), b->stream);
        case GGML_OP_ARGSORT:
            return b200moe_op_argsort_desc(b->moe, &a, &d, b->stream);
        case GGML_OP_MUL_MAT:
            return b200moe_op_mul_mat_f32(b->moe, (const float *) t->src[0]->data, t->src[0]->ne[0], t->src[0]->ne[1], (const float *) t->src[1]->data,
                                          t->src[1]->ne[1], (float *) t->data, b->stream);
        default:
            return -1;
    }
}

ggml_status run_single(BackendCtx * b, GraphPlan & p, ggml_tensor * t) {
    if (t->op == GGML_OP_CONT || t->op == GGML_OP_CPY || t->op == GGML_OP_DUP) {
        const ggml_tensor * s = t->src[0];
        const size_t es = ggml_type_size(s->type);
        if (ggml_is_quantized(s->type) || s->type != t->type || s->nb[0] != es || !ggml_is_contiguous(t) || s->ne[2] != 1 || s->ne[3] != 1 ||
            ggml_nelements(s) != ggml_nelements(t)) {
            set_error(b, "%s: only row-strided 2-D sources of the same type are copied", ggml_op_name(t->op));
            return GGML_STATUS_FAILED;
        }
        const size_t width = (size_t) s->ne[0] * es;
        B200_CUDA(b, cudaMemcpy2DAsync(t->data, width, s->data, s->nb[1], width, (size_t) s->ne[1], cudaMemcpyDeviceToDevice, b->stream));
        return GGML_STATUS_SUCCESS;
    }
    if (t->op == GGML_OP_MUL_MAT_ID) {
        const ggml_tensor * as = t->src[0], * x = t->src[1], * ids = t->src[2];
        if (!is_expert_type(as->type) || x->type != GGML_TYPE_F32 || !ggml_is_contiguous(as) || !ggml_is_contiguous(x) || ids->type != GGML_TYPE_I32 ||
            ids->nb[0] != 4 || as->ne[3] != 1 || x->ne[3] != 1) {
            set_error(b, "MUL_MAT_ID: unsupported operand layout");
            return GGML_STATUS_FAILED;
        }
        const int rc = b200moe_mul_mat_id(b->moe, (int) as->type, as->data, as->ne[0], as->ne[1], as->ne[2], (const float *) current(p, x), x->ne[1],
                                          (const int32_t *) current(p, ids), ids->ne[0], (int64_t) ids->nb[1], x->ne[2], (float *) t->data, b->stream);
        if (rc) return moe_failed(b, "mul_mat_id", rc);
        return GGML_STATUS_SUCCESS;
    }
    // the F32 operators around the fused sub-graphs, one call each
    const int rc = run_operator(b, t);
    if (rc == B200MOE_OK) return GGML_STATUS_SUCCESS;
    if (rc > 0) return moe_failed(b, ggml_op_name(t->op), rc);
    set_error(b, "node '%s' (%s) is not an operator this backend runs", t->name, ggml_op_desc(t));
    return GGML_STATUS_FAILED;
}

// Identity of a graph for the plan cache: the nodes, what they compute, where their operands and results live.
uint64_t graph_key(ggml_cgraph * cg) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) { h = (h ^ v) * 1099511628211ull; };
    const int n = ggml_graph_n_nodes(cg);
    mix((uint64_t) n);
    for (int i = 0; i < n; ++i) {
        const ggml_tensor * t = ggml_graph_node(cg, i);
        mix((uint64_t) (uintptr_t) t); mix((uint64_t) t->op); mix((uint64_t) (uintptr_t) t->data); mix((uint64_t) t->flags);
        mix((uint64_t) t->ne[0]); mix((uint64_t) t->ne[1]); mix((uint64_t) t->ne[2]); mix((uint64_t) t->ne[3]);
        mix((uint64_t) t->nb[1]); mix((uint64_t) t->view_offs);
        for (int s = 0; s < GGML_MAX_SRC; ++s) {
            const ggml_tensor * z = t->src[s];
            mix((uint64_t) (uintptr_t) z);
            if (z) { mix((uint64_t) (uintptr_t) z->data); mix((uint64_t) z->nb[1]); }
        }
        for (int k = 0; k < 4; ++k) mix((uint64_t) (uint32_t) op_param_i32(t, k));
    }
    return h ? h : 1;
}

ggml_status graph_compute_impl(BackendCtx * b, ggml_cgraph * cg) {
    B200_CUDA(b, cudaSetDevice(b->device));
    // The pattern match is kept for as long as the application submits the same graph (decode loops do): only the run-time
    // state of the plan is reset.
    const uint64_t key = graph_key(cg);
    if (b->plan && b->plan_key == key) {
        for (auto & v : b->plan->deferred_at) v.clear();
        b->plan->resolved.clear();
    } else {
        free_plan(b);
        b->plan = new GraphPlan();
        if (!build_plan(b, cg, *b->plan)) { free_plan(b); return GGML_STATUS_FAILED; }
        b->plan_key = key;
    }
    GraphPlan & p = *b->plan;
    // backend scratch for results that cannot be written into graph memory yet
    if (p.scratch_need > b->scratch_bytes) {
        B200_CUDA(b, cudaStreamSynchronize(b->stream));
        if (b->scratch) cudaFree(b->scratch);
        b->scratch = nullptr; b->scratch_bytes = 0;
        void * ptr = nullptr;
        B200_CUDA(b, cudaMalloc(&ptr, p.scratch_need));
        b->scratch = (char *) ptr; b->scratch_bytes = p.scratch_need;
    }
    Arena a{ b->scratch, b->scratch_bytes, 0 };
    for (Group & g : p.groups) {
        for (Materialised * m : { &g.m_ids, &g.m_wts, &g.m_logits, &g.m_probs, &g.m_hid, &g.m_down, &g.m_result }) assign(p, a, *m);
    }
    ggml_b200_graph_stats st = {};
    st.n_nodes = p.n;
    for (int i = 0; i < p.n; ++i) {
        for (size_t d = 0; d < p.deferred_at[i].size(); ++d) {
            const Materialised * m = p.deferred_at[i][d];
            // strided argsort columns come from the dense ids of the route group that owns the argsort node
            const void * src = m->width ? p.groups[p.group_of[i]].m_ids.where : m->where;
            ggml_status s = copy_deferred(b, *m, src);
            if (s != GGML_STATUS_SUCCESS) return s;
            st.n_deferred++;
        }
        ggml_tensor * t = p.nodes[i];
        const int gi = p.group_of[i];
        if (gi >= 0) {
            Group & g = p.groups[gi];
            if (g.exec_at != i) continue;
            ggml_status s = GGML_STATUS_SUCCESS;
            if (g.kind == GROUP_ROUTE)      { s = run_route(b, p, g); st.n_route++; }
            else if (g.kind == GROUP_FFN)   { s = run_ffn(b, p, a, g); st.n_ffn++; }
            else                            { s = run_dense(b, p, g); st.n_dense++; }
            if (s != GGML_STATUS_SUCCESS) return s;
            continue;
        }
        if (is_view_op(t->op)) continue;
        ggml_status s = run_single(b, p, t);
        if (s != GGML_STATUS_SUCCESS) return s;
        st.n_single++;
    }
    b->stats = st;
    return GGML_STATUS_SUCCESS;
}

void free_plan(BackendCtx * b) {
    delete b->plan;
    b->plan = nullptr;
    b->plan_key = 0;
}

}  // namespace

// ------------------------------------------------------------------------------------------------ backend, device, registry
namespace {

ggml_guid_t b200_guid() {
    static ggml_guid guid = { 0xb2, 0x00, 0x6d, 0x6f, 0x65, 0x2d, 0x66, 0x66, 0x6e, 0x2d, 0x73, 0x6d, 0x31, 0x30, 0x30, 0x61 };
    return &guid;
}

const char * backend_get_name(ggml_backend_t) { return GGML_B200_NAME; }

void backend_free(ggml_backend_t backend) {
    auto * b = (BackendCtx *) backend->context;
    cudaSetDevice(b->device);
    if (b->stream) cudaStreamSynchronize(b->stream);
    if (b->moe) b200moe_destroy(b->moe);
    free_plan(b);
    if (b->scratch) cudaFree(b->scratch);
    if (b->stream) cudaStreamDestroy(b->stream);
    delete b;
    delete backend;
}

void backend_synchronize(ggml_backend_t backend) {
    auto * b = (BackendCtx *) backend->context;
    cudaSetDevice(b->device);
    cudaError_t e = cudaStreamSynchronize(b->stream);
    if (e != cudaSuccess) { set_error(b, "synchronize: %s", cudaGetErrorString(e)); b->failed = true; }
    const int rc = b200moe_synchronize(b->moe, b->stream);   // also reads the kernels' own error flag
    if (rc) { set_error(b, "synchronize: %s (%s)", b200moe_status_string(rc), b200moe_last_error(b->moe)); b->failed = true; }
    // synchronize returns nothing: the failure is handed to the next graph_compute
}

void backend_set_tensor_async(ggml_backend_t backend, ggml_tensor * t, const void * data, size_t offset, size_t size) {
    auto * b = (BackendCtx *) backend->context;
    cudaSetDevice(b->device);
    cudaMemcpyAsync((char *) t->data + offset, data, size, cudaMemcpyHostToDevice, b->stream);
}

void backend_get_tensor_async(ggml_backend_t backend, const ggml_tensor * t, void * data, size_t offset, size_t size) {
    auto * b = (BackendCtx *) backend->context;
    cudaSetDevice(b->device);
    cudaMemcpyAsync(data, (const char *) t->data + offset, size, cudaMemcpyDeviceToHost, b->stream);
}

ggml_status backend_graph_compute(ggml_backend_t backend, ggml_cgraph * cg) {
    auto * b = (BackendCtx *) backend->context;
    if (b->failed) {   // found by the last synchronize; reported once, to whatever graph comes next (the empty one included)
        b->failed = false;
        return GGML_STATUS_FAILED;
    }
    const ggml_status s = graph_compute_impl(b, cg);
    return s;
}

const ggml_backend_i backend_iface = {
    /* get_name            */ backend_get_name,
    /* free                */ backend_free,
    /* set_tensor_async    */ backend_set_tensor_async,
    /* get_tensor_async    */ backend_get_tensor_async,
    /* set_tensor_2d_async */ nullptr,
    /* get_tensor_2d_async */ nullptr,
    /* cpy_tensor_async    */ nullptr,
    /* synchronize         */ backend_synchronize,
    /* graph_plan_create   */ nullptr,
    /* graph_plan_free     */ nullptr,
    /* graph_plan_update   */ nullptr,
    /* graph_plan_compute  */ nullptr,
    /* graph_compute       */ backend_graph_compute,
    /* event_record        */ nullptr,
    /* event_wait          */ nullptr,
    /* graph_optimize      */ nullptr,
};

// ---- device

struct Registry {
    std::vector<ggml_backend_device>      devices;
    std::vector<DeviceCtx>                ctxs;
    std::vector<ggml_backend_buffer_type> bufts;
    ggml_backend_reg                      reg;
};

Registry * registry();

const char * dev_get_name(ggml_backend_dev_t dev) { return ((DeviceCtx *) dev->context)->name.c_str(); }
const char * dev_get_description(ggml_backend_dev_t dev) { return ((DeviceCtx *) dev->context)->description.c_str(); }

void dev_get_memory(ggml_backend_dev_t dev, size_t * free, size_t * total) {
    *free = 0; *total = 0;
    b200moe_device_memory(((DeviceCtx *) dev->context)->index, free, total);
}

enum ggml_backend_dev_type dev_get_type(ggml_backend_dev_t) { return GGML_BACKEND_DEVICE_TYPE_GPU; }

void dev_get_props(ggml_backend_dev_t dev, ggml_backend_dev_props * props) {
    memset(props, 0, sizeof *props);
    props->name = dev_get_name(dev);
    props->description = dev_get_description(dev);
    props->type = GGML_BACKEND_DEVICE_TYPE_GPU;
    dev_get_memory(dev, &props->memory_free, &props->memory_total);
    props->device_id = nullptr;
    props->caps.async = true;
    props->caps.host_buffer = false;
    props->caps.buffer_from_host_ptr = false;
    props->caps.events = false;
}

ggml_backend_t dev_init_backend(ggml_backend_dev_t dev, const char *) {
    const int device = ((DeviceCtx *) dev->context)->index;
    auto * b = new BackendCtx();
    b->device = device;
    if (cudaSetDevice(device) != cudaSuccess || cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        delete b;
        return nullptr;
    }
    const int rc = b200moe_create(device, &b->moe);
    if (rc) {
        fprintf(stderr, "ggml-b200: b200moe_create(%d): %s\n", device, b200moe_status_string(rc));
        cudaStreamDestroy(b->stream);
        delete b;
        return nullptr;
    }
    return new ggml_backend{ b200_guid(), backend_iface, dev, b };
}

ggml_backend_buffer_type_t dev_get_buffer_type(ggml_backend_dev_t dev) {
    return &registry()->bufts[((DeviceCtx *) dev->context)->index];
}

bool dev_supports_buft(ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    return buft->iface.get_name == buft_get_name && buft->device == dev;
}

// A node is supported when graph_compute can run it on its own: as a view, as an indexed or dense quantised matmul, as a
// row-strided copy, or as one of the F32 operators (operator_runs).  Nodes inside a recognised route / ffn sub-graph are a
// subset of these, so fusing never adds a requirement.
bool dev_supports_op(ggml_backend_dev_t, const ggml_tensor * op) {
    switch (op->op) {
        case GGML_OP_NONE: case GGML_OP_VIEW: case GGML_OP_RESHAPE: case GGML_OP_PERMUTE: case GGML_OP_TRANSPOSE:
            return true;
        case GGML_OP_MUL_MAT_ID: {
            const ggml_tensor * as = op->src[0], * x = op->src[1], * ids = op->src[2];
            return is_expert_type(as->type) && x->type == GGML_TYPE_F32 && ids->type == GGML_TYPE_I32 && ids->nb[0] == 4 && ids->ne[0] <= 32 &&
                   ggml_is_contiguous(as) && ggml_is_contiguous(x) && as->ne[3] == 1 && x->ne[3] == 1 && as->ne[1] % 8 == 0 && as->ne[2] <= 1024 &&
                   b200moe_mul_mat_id_width_ok((int) as->type, as->ne[0]);
        }
        case GGML_OP_MUL_MAT:
            if (is_expert_type(op->src[0]->type))
                return op->src[1]->type == GGML_TYPE_F32 && ggml_is_contiguous(op->src[0]) && ggml_is_contiguous(op->src[1]) && op->src[0]->ne[2] == 1 &&
                       op->src[0]->ne[3] == 1 && op->src[1]->ne[2] == 1 && op->src[1]->ne[3] == 1 && op->src[0]->ne[1] % 8 == 0 &&
                       b200moe_mul_mat_id_width_ok((int) op->src[0]->type, op->src[0]->ne[0]);
            return operator_runs(op);
        case GGML_OP_CONT: case GGML_OP_CPY: case GGML_OP_DUP: {
            const ggml_tensor * z = op->src[0];
            return !ggml_is_quantized(z->type) && z->type == op->type && z->nb[0] == ggml_type_size(z->type) && ggml_is_contiguous(op) && z->ne[2] == 1 &&
                   z->ne[3] == 1 && ggml_nelements(z) == ggml_nelements(op);
        }
        default:
            return operator_runs(op);
    }
}

bool dev_offload_op(ggml_backend_dev_t, const ggml_tensor * op) { return op->op == GGML_OP_MUL_MAT_ID; }

const ggml_backend_device_i device_iface = {
    /* get_name             */ dev_get_name,
    /* get_description      */ dev_get_description,
    /* get_memory           */ dev_get_memory,
    /* get_type             */ dev_get_type,
    /* get_props            */ dev_get_props,
    /* init_backend         */ dev_init_backend,
    /* get_buffer_type      */ dev_get_buffer_type,
    /* get_host_buffer_type */ nullptr,
    /* buffer_from_host_ptr */ nullptr,
    /* supports_op          */ dev_supports_op,
    /* supports_buft        */ dev_supports_buft,
    /* offload_op           */ dev_offload_op,
    /* event_new            */ nullptr,
    /* event_free           */ nullptr,
    /* event_synchronize    */ nullptr,
};

// ---- registry

const char * reg_get_name(ggml_backend_reg_t) { return GGML_B200_NAME; }
size_t reg_get_device_count(ggml_backend_reg_t) { return registry()->devices.size(); }
ggml_backend_dev_t reg_get_device(ggml_backend_reg_t, size_t i) {
    Registry * r = registry();
    return i < r->devices.size() ? &r->devices[i] : nullptr;
}
void * reg_get_proc_address(ggml_backend_reg_t, const char * name) {
    if (!strcmp(name, "ggml_backend_b200_set_expert_path")) return (void *) ggml_backend_b200_set_expert_path;
    if (!strcmp(name, "ggml_backend_b200_graph_stats")) return (void *) ggml_backend_b200_graph_stats;
    return nullptr;
}

const ggml_backend_reg_i reg_iface = { reg_get_name, reg_get_device_count, reg_get_device, reg_get_proc_address };

Registry * registry() {
    static Registry * r = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        r = new Registry();
        r->reg = ggml_backend_reg{ GGML_BACKEND_API_VERSION, reg_iface, nullptr };
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); n = 0; }
        n = std::min(n, MAX_DEVICES);
        // the vectors must not move once pointers into them are handed out
        r->ctxs.reserve(n); r->devices.reserve(n); r->bufts.reserve(n);
        for (int i = 0; i < n; ++i) {
            cudaDeviceProp prop;
            if (cudaGetDeviceProperties(&prop, i) != cudaSuccess) { cudaGetLastError(); break; }
            if (prop.major != 10) break;   // device indices stay equal to CUDA ordinals: stop at the first foreign device
            DeviceCtx c;
            c.index = i;
            c.name = std::string(GGML_B200_NAME) + "_" + std::to_string(i);
            c.description = prop.name;
            r->ctxs.push_back(c);
            r->devices.push_back(ggml_backend_device{ device_iface, &r->reg, &r->ctxs.back() });
            r->bufts.push_back(ggml_backend_buffer_type{ buft_iface, &r->devices.back(), nullptr });
        }
    });
    return r;
}

}  // namespace

extern "C" {

ggml_backend_reg_t ggml_backend_b200_reg(void) { return &registry()->reg; }

ggml_backend_t ggml_backend_b200_init(int device) {
    Registry * r = registry();
    if (device < 0 || (size_t) device >= r->devices.size()) return nullptr;
    return dev_init_backend(&r->devices[device], nullptr);
}

bool ggml_backend_is_b200(ggml_backend_t backend) { return backend && ggml_guid_matches(backend->guid, b200_guid()); }

ggml_backend_buffer_type_t ggml_backend_b200_buffer_type(int device) {
    Registry * r = registry();
    if (device < 0 || (size_t) device >= r->bufts.size()) return nullptr;
    return &r->bufts[device];
}

int ggml_backend_b200_set_expert_path(ggml_backend_t backend, int path) {
    if (!ggml_backend_is_b200(backend)) return B200MOE_ERR_INVALID_ARG;
    return b200moe_set_expert_path(((BackendCtx *) backend->context)->moe, path);
}

int ggml_backend_b200_graph_stats(ggml_backend_t backend, struct ggml_b200_graph_stats * out) {
    if (!ggml_backend_is_b200(backend) || !out) return B200MOE_ERR_INVALID_ARG;
    *out = ((BackendCtx *) backend->context)->stats;
    return B200MOE_OK;
}

const char * ggml_backend_b200_last_error(ggml_backend_t backend) {
    if (!ggml_backend_is_b200(backend)) return "not a B200 backend";
    return ((BackendCtx *) backend->context)->error.c_str();
}

}  // extern "C"

// Entry points for ggml's dynamic backend loader (ggml-backend-impl.h:251-287): built with -DGGML_BACKEND_DL the library exports
// ggml_backend_init / ggml_backend_score and can be dropped next to the application's other backends instead of being registered
// explicitly.  The score is the number of sm_100 devices found.
static int b200_score() { return (int) registry()->devices.size(); }
GGML_BACKEND_DL_IMPL(ggml_backend_b200_reg)
GGML_BACKEND_DL_SCORE_IMPL(b200_score)
