// TEST INFRASTRUCTURE (parity checker + timed CPU baseline), not product code.
//
// Thin C entry points over the reference's own ggml CPU backend, compiled from the reference
// sources by oracle/Makefile into oracle/_ref/libedge0_ref.so.  The graph built here is the one
// edge0-infer builds for the quantised MoE FFN:
//   Builder::route  edge0-infer/src/models/edge0_35b/forward.cpp:262-271
//   Builder::ffn    edge0-infer/src/models/edge0_35b/forward.cpp:300-311 (routed experts only)
// plus three optional pieces the benchmark configurations ask for:
//   * a per-expert bias added to the router logits before the softmax (prefill config),
//   * the NVFP4 per-expert fp32 scale applied as reshape -> repeat -> get_rows -> mul, the pattern
//     recognised at third_party/ggml/src/ggml-cuda/ggml-cuda.cu:3655-3673,
//   * a latent wrapper  x -> D x -> experts in latent width -> U (.)  (edge0-strata
//     src/latent/latent_moe.cpp:38-92 with one label group).
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "ggml.h"
#include "ggml-alloc.h"
#include "ggml-backend.h"
#include "gguf.h"
#include "ggml-cpu.h"

extern "C" {

struct ref_moe_args {
    // shapes
    int32_t H;        // hidden width fed to the router (and to D when latent != 0)
    int32_t L;        // width the experts see (== H unless latent)
    int32_t E;        // experts
    int32_t K;        // experts per token
    int32_t I;        // expert intermediate width
    int32_t T;        // tokens
    int32_t wtype;    // ggml_type of the expert tensors (11 = Q3_K, 40 = NVFP4, 0 = F32)
    int32_t n_threads;
    int32_t repeats;  // timed graph computes after one warm-up (0: compute once, no timing)
    int32_t latent;   // 0/1
    // inputs
    const float * x;            // [T][H]
    const float * router_w;     // [E][H]
    const float * router_bias;  // [E] or null
    const void  * gate;         // [E][I][L] quantised rows
    const void  * up;           // [E][I][L]
    const void  * down;         // [E][L][I]
    const float * s_gate;       // [E] or null
    const float * s_up;
    const float * s_down;
    const void  * lat_d;        // [L][H] quantised (latent only)
    const void  * lat_u;        // [H][L] quantised (latent only)
    const float * s_lat_d;      // [1] or null
    const float * s_lat_u;      // [1] or null
    // outputs (any may be null)
    float   * logits;   // [T][E]
    float   * probs;    // [T][E]
    int32_t * ids;      // [T][K]
    float   * weights;  // [T][K]
    float   * hidden;   // [T][K][I]   silu(gate)*up
    float   * down_out; // [T][K][L]   before the route weight
    float   * moe_out;  // [T][L]      weighted sum in slot order
    float   * out;      // [T][H or L] final (== moe_out unless latent)
    double  * ms_best;
    double  * ms_median;
    // shared expert with its sigmoid gate (forward.cpp:312-314); null / 0 when the layer has none (non-latent layers only)
    const void  * sh_gate;      // [I_sh][H] quantised rows
    const void  * sh_up;        // [I_sh][H]
    const void  * sh_down;      // [H][I_sh]
    const float * sh_gate_inp;  // [H] F32
    float   * shexp_gated;      // [T][H] output or null
    int32_t   I_sh;
    int32_t   pad_;
};

int ref_type_row_size(int type, int64_t n, int64_t * out) {
    *out = (int64_t) ggml_row_size((ggml_type) type, n);
    return 0;
}

// ggml_quantize_chunk without an importance matrix = quantize_row_*_ref
// (third_party/ggml/src/ggml-quants.c:1229 Q3_K, :384 NVFP4).
int ref_quantize(int type, const float * src, void * dst, int64_t nrows, int64_t n_per_row) {
    ggml_quantize_chunk((ggml_type) type, src, dst, 0, nrows, n_per_row, nullptr);
    return 0;
}

int ref_dequantize(int type, const void * src, float * dst, int64_t n) {
    const auto * tr = ggml_get_type_traits((ggml_type) type);
    if (!tr || !tr->to_float) return 1;
    tr->to_float(src, dst, n);
    return 0;
}

// Activation quantiser of the CPU backend for a weight type (vec_dot_type's from_float):
// Q8_K for Q3_K, Q8_0 for NVFP4.  Returns the byte size written.
int64_t ref_quantize_activation(int wtype, const float * src, void * dst, int64_t n) {
    ggml_cpu_init();  // fills the fp16 / UE4M3 lookup tables the CPU kernels read (idempotent)
    const auto * tc = ggml_get_type_traits_cpu((ggml_type) wtype);
    const ggml_type vt = tc->vec_dot_type;
    ggml_get_type_traits_cpu(vt)->from_float(src, dst, n);
    return (int64_t) ggml_row_size(vt, n);
}

int ref_vec_dot(int wtype, int64_t n, const void * wrow, const void * act, float * out) {
    ggml_cpu_init();
    const auto * tc = ggml_get_type_traits_cpu((ggml_type) wtype);
    tc->vec_dot((int) n, out, 0, wrow, 0, act, 0, 1);
    return 0;
}

static ggml_tensor * scaled(ggml_context * c, ggml_tensor * mm, ggml_tensor * scale, ggml_tensor * ids, int E, int T) {
    if (!scale) return mm;
    ggml_tensor * s = ggml_reshape_2d(c, scale, 1, E);
    s = ggml_repeat_4d(c, s, 1, E, T, 1);
    s = ggml_get_rows(c, s, ids);  // [1, K, T]
    return ggml_mul(c, mm, s);
}

// backend == null: the reference's CPU backend (created and freed here).  Otherwise the same graph is computed on the
// given ggml backend (the caller keeps ownership) - this is how a ggml backend under test is driven by the reference's
// own graph.  use_gallocr != 0 allocates the graph's intermediate tensors with ggml's graph allocator (memory reused
// between tensors, as in edge0-infer's exec::build_plan) instead of giving every tensor its own memory.
static int run_layer(const ref_moe_args * a, ggml_backend_t backend, int use_gallocr) {
    const int H = a->H, L = a->latent ? a->L : a->H, E = a->E, K = a->K, I = a->I, T = a->T;
    const ggml_type wt = (ggml_type) a->wtype;

    ggml_init_params ipw = { ggml_tensor_overhead() * 40, nullptr, true };
    ggml_init_params ip  = { ggml_tensor_overhead() * 256 + ggml_graph_overhead_custom(512, false), nullptr, true };
    ggml_context * cw = ggml_init(ipw);
    ggml_context * c  = ggml_init(ip);
    if (!c || !cw) return 1;

    ggml_tensor * x   = ggml_new_tensor_2d(cw, GGML_TYPE_F32, H, T);
    ggml_tensor * rw  = ggml_new_tensor_2d(cw, GGML_TYPE_F32, H, E);
    ggml_tensor * rb  = a->router_bias ? ggml_new_tensor_1d(cw, GGML_TYPE_F32, E) : nullptr;
    ggml_tensor * wg  = ggml_new_tensor_3d(cw, wt, L, I, E);
    ggml_tensor * wu  = ggml_new_tensor_3d(cw, wt, L, I, E);
    ggml_tensor * wd  = ggml_new_tensor_3d(cw, wt, I, L, E);
    ggml_tensor * sg  = a->s_gate ? ggml_new_tensor_1d(cw, GGML_TYPE_F32, E) : nullptr;
    ggml_tensor * su  = a->s_up   ? ggml_new_tensor_1d(cw, GGML_TYPE_F32, E) : nullptr;
    ggml_tensor * sd  = a->s_down ? ggml_new_tensor_1d(cw, GGML_TYPE_F32, E) : nullptr;
    ggml_tensor * ld  = a->latent ? ggml_new_tensor_2d(cw, wt, H, L) : nullptr;
    ggml_tensor * lu  = a->latent ? ggml_new_tensor_2d(cw, wt, L, H) : nullptr;
    ggml_tensor * sld = (a->latent && a->s_lat_d) ? ggml_new_tensor_1d(cw, GGML_TYPE_F32, 1) : nullptr;
    ggml_tensor * slu = (a->latent && a->s_lat_u) ? ggml_new_tensor_1d(cw, GGML_TYPE_F32, 1) : nullptr;
    const bool shexp = a->sh_gate && !a->latent;
    ggml_tensor * shg = shexp ? ggml_new_tensor_2d(cw, wt, H, a->I_sh) : nullptr;
    ggml_tensor * shu = shexp ? ggml_new_tensor_2d(cw, wt, H, a->I_sh) : nullptr;
    ggml_tensor * shd = shexp ? ggml_new_tensor_2d(cw, wt, a->I_sh, H) : nullptr;
    ggml_tensor * shi = shexp ? ggml_new_tensor_2d(cw, GGML_TYPE_F32, H, 1) : nullptr;

    // ---- route (forward.cpp:262-271)
    ggml_tensor * logits = ggml_mul_mat(c, rw, x);                       // [E, T]
    if (rb) logits = ggml_add(c, logits, rb);
    ggml_tensor * probs  = ggml_soft_max(c, logits);
    ggml_tensor * ids    = ggml_argsort_top_k(c, probs, K);              // view [K, T] of [E, T]
    ggml_tensor * wts    = ggml_reshape_2d(c, ggml_get_rows(c, ggml_reshape_3d(c, probs, 1, E, T), ids), K, T);
    wts = ggml_div(c, wts, ggml_clamp(c, ggml_sum_rows(c, wts), 6.103515625e-5f, INFINITY));

    // ---- optional latent down-projection
    ggml_tensor * xe = x;
    if (a->latent) {
        xe = ggml_mul_mat(c, ld, x);                                     // [L, T]
        if (sld) xe = ggml_mul(c, xe, sld);
    }

    // ---- ffn (forward.cpp:300-311)
    ggml_tensor * input = ggml_reshape_3d(c, xe, L, 1, T);
    ggml_tensor * gate  = scaled(c, ggml_mul_mat_id(c, wg, input, ids), sg, ids, E, T);  // [I, K, T]
    ggml_tensor * up    = scaled(c, ggml_mul_mat_id(c, wu, input, ids), su, ids, E, T);
    ggml_tensor * hid   = ggml_mul(c, ggml_silu(c, gate), up);
    ggml_tensor * down  = scaled(c, ggml_mul_mat_id(c, wd, hid, ids), sd, ids, E, T);    // [L, K, T]
    ggml_tensor * dw    = ggml_mul(c, down, ggml_reshape_3d(c, wts, 1, K, T));
    ggml_tensor * sum   = ggml_view_2d(c, dw, L, T, dw->nb[2], 0);
    for (int i = 1; i < K; ++i) sum = ggml_add(c, sum, ggml_view_2d(c, dw, L, T, dw->nb[2], i * dw->nb[1]));
    ggml_tensor * moe = (K == 1) ? ggml_cont(c, sum) : sum;
    // ---- shared expert and its sigmoid gate (forward.cpp:312-314), added to the routed sum
    ggml_tensor * gated = nullptr;
    ggml_tensor * routed = moe;       // "ffn_moe_out" of the reference; `moe` becomes "ffn_out" below
    if (shexp) {
        ggml_tensor * sh = ggml_mul_mat(c, shd, ggml_mul(c, ggml_silu(c, ggml_mul_mat(c, shg, x)), ggml_mul_mat(c, shu, x)));
        gated = ggml_mul(c, sh, ggml_sigmoid(c, ggml_mul_mat(c, shi, x)));
        moe = ggml_add(c, moe, gated);
    }

    ggml_tensor * out = moe;
    if (a->latent) {
        out = ggml_mul_mat(c, lu, moe);                                  // [H, T]
        if (slu) out = ggml_mul(c, out, slu);
    }
    ggml_tensor * ids_c = ggml_cont(c, ids);

    ggml_cgraph * g = ggml_new_graph_custom(c, 512, false);
    ggml_build_forward_expand(g, out);
    ggml_build_forward_expand(g, ids_c);
    // observation points must not be overwritten by the allocator: mark them as outputs
    ggml_tensor * keep[] = { logits, probs, wts, hid, down, routed, moe, out, ids_c, gated };
    for (ggml_tensor * t : keep) if (t) ggml_set_output(t);

    ggml_backend_t be = backend ? backend : ggml_backend_cpu_init();
    if (!be) { ggml_free(c); ggml_free(cw); return 2; }
    if (!backend) ggml_backend_cpu_set_n_threads(be, a->n_threads > 0 ? a->n_threads : 1);

    // weights and the input in one backend buffer; graph results in a second one or under the graph allocator
    ggml_backend_buffer_t bufw = ggml_backend_alloc_ctx_tensors(cw, be);
    ggml_backend_buffer_t buf  = nullptr;
    ggml_gallocr_t galloc = nullptr;
    bool ok = bufw != nullptr;
    if (ok && use_gallocr) {
        galloc = ggml_gallocr_new(ggml_backend_get_default_buffer_type(be));
        ok = galloc && ggml_gallocr_alloc_graph(galloc, g);
    } else if (ok) {
        buf = ggml_backend_alloc_ctx_tensors(c, be);
        ok = buf != nullptr;
    }
    if (!ok) {
        if (galloc) ggml_gallocr_free(galloc);
        if (bufw) ggml_backend_buffer_free(bufw);
        if (!backend) ggml_backend_free(be);
        ggml_free(c); ggml_free(cw);
        return 3;
    }

    auto set = [](ggml_tensor * t, const void * p) { if (t && p) ggml_backend_tensor_set(t, p, 0, ggml_nbytes(t)); };
    set(x, a->x); set(rw, a->router_w); set(rb, a->router_bias);
    set(wg, a->gate); set(wu, a->up); set(wd, a->down);
    set(sg, a->s_gate); set(su, a->s_up); set(sd, a->s_down);
    set(ld, a->lat_d); set(lu, a->lat_u); set(sld, a->s_lat_d); set(slu, a->s_lat_u);
    set(shg, a->sh_gate); set(shu, a->sh_up); set(shd, a->sh_down); set(shi, a->sh_gate_inp);

    ggml_status st = ggml_backend_graph_compute(be, g);
    int rc = st == GGML_STATUS_SUCCESS ? 0 : 4;

    if (rc == 0) {
        auto get = [](ggml_tensor * t, void * p) { if (t && p) ggml_backend_tensor_get(t, p, 0, ggml_nbytes(t)); };
        get(logits, a->logits); get(probs, a->probs); get(ids_c, a->ids); get(wts, a->weights);
        get(hid, a->hidden); get(down, a->down_out); get(out, a->out); get(gated, a->shexp_gated);
        if (a->moe_out) {
            // moe may be a strided view when K > 1? no: ggml_add results are contiguous
            ggml_backend_tensor_get(routed, a->moe_out, 0, ggml_nbytes(routed));
        }
    }

    if (rc == 0 && a->repeats > 0) {
        std::vector<double> ms;
        for (int r = 0; r < a->repeats; ++r) {
            auto t0 = std::chrono::steady_clock::now();
            st = ggml_backend_graph_compute(be, g);
            auto t1 = std::chrono::steady_clock::now();
            if (st != GGML_STATUS_SUCCESS) { rc = 4; break; }
            ms.push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
        }
        if (rc == 0) {
            std::vector<double> s = ms;
            for (size_t i = 1; i < s.size(); ++i) for (size_t j = i; j > 0 && s[j] < s[j-1]; --j) std::swap(s[j], s[j-1]);
            if (a->ms_best)   *a->ms_best   = s.front();
            if (a->ms_median) *a->ms_median = s[s.size() / 2];
        }
    }

    if (galloc) ggml_gallocr_free(galloc);
    if (buf) ggml_backend_buffer_free(buf);
    ggml_backend_buffer_free(bufw);
    if (!backend) ggml_backend_free(be);
    ggml_free(c);
    ggml_free(cw);
    return rc;
}

int ref_moe_layer(const ref_moe_args * a) { return run_layer(a, nullptr, 0); }

int ref_moe_layer_backend(const ref_moe_args * a, void * backend, int use_gallocr) {
    return run_layer(a, (ggml_backend_t) backend, use_gallocr);
}

// One MUL_MAT_ID node, as [K, n_ids, T] = as[ne00, ne01, n_as] x b[ne00, n_ids, T] by ids[n_ids, T], on the given backend (null: the
// reference's CPU backend).  Returns the status of ggml_backend_graph_compute as 0 (success) or 4.
int ref_mul_mat_id_backend(void * backend, int wtype, const void * as, int64_t ne00, int64_t ne01, int64_t n_as, const float * b,
                           const int32_t * ids, int64_t n_ids, int64_t T, float * dst, int n_threads) {
    ggml_init_params ip = { ggml_tensor_overhead() * 16 + ggml_graph_overhead_custom(16, false), nullptr, true };
    ggml_context * c = ggml_init(ip);
    if (!c) return 1;
    ggml_tensor * w = ggml_new_tensor_3d(c, (ggml_type) wtype, ne00, ne01, n_as);
    ggml_tensor * x = ggml_new_tensor_3d(c, GGML_TYPE_F32, ne00, n_ids, T);
    ggml_tensor * id = ggml_new_tensor_2d(c, GGML_TYPE_I32, n_ids, T);
    ggml_tensor * y = ggml_mul_mat_id(c, w, x, id);
    ggml_set_output(y);
    ggml_cgraph * g = ggml_new_graph_custom(c, 16, false);
    ggml_build_forward_expand(g, y);
    ggml_backend_t be = backend ? (ggml_backend_t) backend : ggml_backend_cpu_init();
    if (!be) { ggml_free(c); return 2; }
    if (!backend) ggml_backend_cpu_set_n_threads(be, n_threads > 0 ? n_threads : 1);
    ggml_backend_buffer_t buf = ggml_backend_alloc_ctx_tensors(c, be);
    if (!buf) { if (!backend) ggml_backend_free(be); ggml_free(c); return 3; }
    ggml_backend_tensor_set(w, as, 0, ggml_nbytes(w));
    ggml_backend_tensor_set(x, b, 0, ggml_nbytes(x));
    ggml_backend_tensor_set(id, ids, 0, ggml_nbytes(id));
    const int rc = ggml_backend_graph_compute(be, g) == GGML_STATUS_SUCCESS ? 0 : 4;
    if (rc == 0 && dst) ggml_backend_tensor_get(y, dst, 0, ggml_nbytes(y));
    ggml_backend_buffer_free(buf);
    if (!backend) ggml_backend_free(be);
    ggml_free(c);
    return rc;
}

// Synchronize, then compute a graph without nodes: the way edge0-infer asks a backend whether earlier work completed
// (src/platform/backend.cpp:151-159).  Returns 0 (success) or 4.
int ref_backend_confirm(void * backend) {
    ggml_init_params ip = { ggml_graph_overhead_custom(4, false) + 1024, nullptr, true };
    ggml_context * c = ggml_init(ip);
    if (!c) return 1;
    ggml_cgraph * g = ggml_new_graph_custom(c, 4, false);
    ggml_backend_synchronize((ggml_backend_t) backend);
    const int rc = ggml_backend_graph_compute((ggml_backend_t) backend, g) == GGML_STATUS_SUCCESS ? 0 : 4;
    ggml_free(c);
    return rc;
}

// Writes a GGUF file with ONE MoE block through the reference's own gguf writer (third_party/ggml/src/gguf.cpp): metadata
// general.architecture = "qwen3next", qwen3next.block_count / expert_count / expert_used_count, and the tensors edge0-infer's graph
// names (forward.cpp:262-314): blk.<layer>.ffn_gate_inp.weight (F32), ffn_gate_exps / ffn_up_exps / ffn_down_exps .weight, and the
// four shared-expert tensors when the arguments hold them.  Test input for the product's GGUF reader.
int ref_write_moe_gguf(const char * path, const ref_moe_args * a, int layer) {
    if (!path || !a || a->latent) return 1;
    ggml_init_params ip = { ggml_tensor_overhead() * 16, nullptr, true };
    ggml_context * c = ggml_init(ip);
    gguf_context * g = gguf_init_empty();
    if (!c || !g) return 2;
    gguf_set_val_str(g, "general.architecture", "qwen3next");
    gguf_set_val_u32(g, "qwen3next.block_count", (uint32_t) layer + 1);
    gguf_set_val_u32(g, "qwen3next.expert_count", (uint32_t) a->E);
    gguf_set_val_u32(g, "qwen3next.expert_used_count", (uint32_t) a->K);
    const ggml_type wt = (ggml_type) a->wtype;
    const std::string prefix = "blk." + std::to_string(layer) + ".";
    auto add = [&](ggml_tensor * t, const char * name, const void * data) {
        ggml_set_name(t, (prefix + name).c_str());
        t->data = const_cast<void *>(data);
        gguf_add_tensor(g, t);
    };
    add(ggml_new_tensor_2d(c, GGML_TYPE_F32, a->H, a->E), "ffn_gate_inp.weight", a->router_w);
    add(ggml_new_tensor_3d(c, wt, a->H, a->I, a->E), "ffn_gate_exps.weight", a->gate);
    add(ggml_new_tensor_3d(c, wt, a->H, a->I, a->E), "ffn_up_exps.weight", a->up);
    add(ggml_new_tensor_3d(c, wt, a->I, a->H, a->E), "ffn_down_exps.weight", a->down);
    if (a->sh_gate) {
        add(ggml_new_tensor_2d(c, wt, a->H, a->I_sh), "ffn_gate_shexp.weight", a->sh_gate);
        add(ggml_new_tensor_2d(c, wt, a->H, a->I_sh), "ffn_up_shexp.weight", a->sh_up);
        add(ggml_new_tensor_2d(c, wt, a->I_sh, a->H), "ffn_down_shexp.weight", a->sh_down);
        add(ggml_new_tensor_1d(c, GGML_TYPE_F32, a->H), "ffn_gate_inp_shexp.weight", a->sh_gate_inp);
    }
    const bool ok = gguf_write_to_file(g, path, false);
    gguf_free(g);
    ggml_free(c);
    return ok ? 0 : 3;
}

void ref_backend_free(void * backend) { if (backend) ggml_backend_free((ggml_backend_t) backend); }

const char * ref_isa(void) {
    static char buf[256];
    snprintf(buf, sizeof buf, "avx=%d avx2=%d fma=%d f16c=%d avx512=%d avx_vnni=%d bmi2=%d",
             ggml_cpu_has_avx(), ggml_cpu_has_avx2(), ggml_cpu_has_fma(), ggml_cpu_has_f16c(),
             ggml_cpu_has_avx512(), ggml_cpu_has_avx_vnni(), ggml_cpu_has_bmi2());
    return buf;
}

}  // extern "C"
