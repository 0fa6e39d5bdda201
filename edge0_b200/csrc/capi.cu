// C ABI of the B200 MoE-FFN path (declared in include/edge0_b200_moe.h): context, device scratch,
// argument validation and kernel dispatch.  No torch types, no host fallback: without a CUDA device
// every compute entry point fails with B200MOE_ERR_NO_DEVICE / B200MOE_ERR_CUDA.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <type_traits>
#include <vector>

#include "../../include/edge0_b200_moe.h"
#include "expert_gemm.cuh"
#include "expert_gemm_fp4.cuh"
#include "expert_exchange.cuh"
#include "expert_gemm_tm.cuh"
#include "expert_gemv.cuh"
#include "expert_mma.cuh"
#include "fp4_probe.cuh"
#include "graph_ops.cuh"
#include "requant_fixup.cuh"
#include "router.cuh"

using namespace b200moe;

namespace {

struct Scratch {
    uint8_t * base = nullptr;
    size_t bytes = 0;
};

struct Plan {  // carved out of the scratch arena for one (layer shape, max_tokens)
    int max_tokens = 0, n_embd = 0, n_in = 0, n_expert = 0, k = 0, n_ff = 0, wtype = 0, n_ff_sh = 0;
    float * logits = nullptr;
    float * probs = nullptr;
    int32_t * ids = nullptr;
    float * wts = nullptr;
    Groups groups{};
    ActQuant xq{};    // [T][n_embd or n_in] (reused: latent-down input, then expert input)
    ActQuant xlq{};   // [T][n_in] expert input when latent
    ActQuant hq{};    // [T*k][n_ff]
    ActQuant moq{};   // [T][n_in] latent-up input
    float * xl = nullptr;   // [T][n_in] latent activations
    float * hid = nullptr;  // [T*k][n_ff]
    float * y = nullptr;    // [T*k][n_in]
    float * moe = nullptr;  // [T][n_in]
    float * xf = nullptr;   // [T][n_embd] fp32 copy of bf16 input (only for host entry / conversions)
    void * xin = nullptr;   // [T][n_embd] staging for the host entry point (input dtype bytes, <= 4 B/elt)
    float * outb = nullptr; // [T][n_embd] staging for the host entry point
    int * one_group_ids = nullptr;  // [T] group of every token when a dense matvec runs on the indexed-matmul kernel
    __half * afp16 = nullptr;       // [T*k][max(n_in, n_ff)] expert-sorted fp16 activations of the tensor-core path (or the FP4 digit planes)
    uint8_t * asf = nullptr;        // scale tiles of the FP4 digit planes: [token tiles][K / 256][2048]
    size_t asf_bytes = 0;
    float * arow_scale = nullptr;   // [T*k] power of two per expert-sorted routed row (FP4 digit planes)
    float * sh_a = nullptr;         // [T][n_ff_sh] shared expert: gate product, then silu(gate) * up
    float * sh_b = nullptr;         // [T][n_ff_sh] shared expert: up product
    float * sh_out = nullptr;       // [T][n_embd]  shared expert: down product
    float * sh_gate = nullptr;      // [T]          shared expert: logit of its sigmoid gate
    ActQuant shq{};                 // [T][n_ff_sh] quantised input of the shared expert's down product
    size_t total = 0;
};

}  // namespace

struct b200moe_ctx {
    int device = 0;
    int sm_count = 0;
    Scratch scratch;
    Plan plan;
    int * d_err = nullptr;  // 16 bytes: [error code][pad][fix-up overflow counter, 64 bit]
    int * h_err = nullptr;  // pinned copy of the same
    std::string last_error;
    b200moe_counters counters{};
    int64_t launches = 0;
    bool timing = false;
    int expert_path = 0;  // 0 auto, 1 integer GEMV always, 2 tensor-core GEMM whenever the shape allows
    bool overlap = false; // launch the layer's kernels as programmatic dependents of one another (opt-in)
    bool overlap_now = false;  // set per call: only the small-batch regime uses it (see layer_overlap)
    bool dense_now = false;    // the expert kernels are running a dense product (kernel-timing kind 2)
    struct Timed { cudaEvent_t beg, end; int kind; };
    std::vector<Timed> timed;
};

namespace {

int fail(b200moe_ctx * ctx, int code, const char * fmt, ...) {
    if (ctx) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        ctx->last_error = buf;
    }
    return code;
}

#define CUDA_TRY(ctx, expr)                                                                          \
    do {                                                                                             \
        cudaError_t _e = (expr);                                                                     \
        if (_e != cudaSuccess) return fail(ctx, B200MOE_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Carver {
    uint8_t * base;
    size_t off = 0;
    template <typename T>
    T * take(size_t n) {
        off = align_up(off, 256);
        T * p = base ? reinterpret_cast<T *>(base + off) : nullptr;
        off += n * sizeof(T);
        return p;
    }
    ActQuant act(size_t rows, size_t k) {
        ActQuant a;
        a.q = take<int8_t>(rows * k);
        a.d = take<float>(rows * (k / 32));
        a.bsum = take<int16_t>(rows * (k / 16));
        return a;
    }
};

void carve(Plan & p, uint8_t * base) {
    Carver c{base};
    const size_t T = p.max_tokens, E = p.n_expert, k = p.k, R = T * k;
    const size_t kin = p.n_in, H = p.n_embd, I = p.n_ff, Ish = p.n_ff_sh;
    p.logits = c.take<float>(T * E);
    p.probs = c.take<float>(T * E);
    p.ids = c.take<int32_t>(R);
    p.wts = c.take<float>(R);
    p.groups.counts = c.take<int>(std::max<size_t>(E, 1) + 8);
    p.groups.offsets = c.take<int>(E + 1);
    p.groups.pos = c.take<int>(std::max(R, T));
    p.groups.perm = c.take<int>(std::max(R, T));
    p.groups.active = c.take<int>(E);
    p.groups.meta = c.take<int>(4);
    p.groups.cost = c.take<int>(4 * (E + 1));
    p.xq = c.act(T, std::max(H, kin));
    p.xlq = c.act(T, kin);
    p.hq = c.act(R, I);
    p.moq = c.act(T, kin);
    p.xl = c.take<float>(T * kin);
    p.hid = c.take<float>(R * I);
    p.y = c.take<float>(R * kin);
    p.moe = c.take<float>(T * kin);
    p.xf = c.take<float>(T * H);
    p.xin = c.take<float>(T * H);
    p.outb = c.take<float>(T * H);
    p.one_group_ids = c.take<int>(T);
    p.afp16 = c.take<__half>(2 * std::max<size_t>(std::max(R, T), 64) * std::max({kin, I, H, Ish}));   // hi plane, then lo plane
    p.asf_bytes = (std::min(E, std::max(R, T)) + std::max(R, T) / FP4_RPT + 1) * ((std::max({kin, I, H, Ish}) + 255) / 256) * FP4_SF_TILE;
    p.asf = c.take<uint8_t>(p.asf_bytes);
    p.arow_scale = c.take<float>(std::max(R, T));
    if (Ish) {
        p.sh_a = c.take<float>(T * Ish);
        p.sh_b = c.take<float>(T * Ish);
        p.sh_out = c.take<float>(T * H);
        p.sh_gate = c.take<float>(T);
        p.shq = c.act(T, Ish);
    }
    p.total = align_up(c.off, 256);
}

bool gemv_supported(int wtype, int64_t k) {
    if (wtype == TYPE_NVFP4) return k == 256 || k == 512 || k == 768 || k == 1024 || k == 2048 || k == 4096;
    if (wtype == TYPE_Q3_K) return k == 256 || k == 512 || k == 768 || k == 2048;
    return false;
}

// Programmatic dependent launch (opt-in, b200moe_set_launch_overlap) is applied in the batched-decode regime only (few routed
// rows per expert), where launch latency and kernel prologues are a visible share of an eagerly launched step.  Measured:
// +7 % end to end through the host entry point, nothing under CUDA-graph replay (and slower at 8 tokens), which is why it is
// off by default.  With prefill-sized grids it gains nothing, and the gate/up grouped GEMM with 128-token tiles was measured
// to return wrong values when a large dependent grid was resident beside it (cause not found by reading; serial launches are
// correct), so large calls always launch serially, and the tensor-core kernels are never launched with the attribute nor
// release their dependents early: nothing becomes resident beside a kernel that holds tensor memory.
void layer_overlap(b200moe_ctx * ctx, int64_t rows, int n_expert) { ctx->overlap_now = rows < (int64_t) 24 * n_expert; }

// Launch with programmatic stream serialisation: the kernel may start while its predecessor in the stream is still running;
// every kernel of this library calls griddepcontrol.wait before it touches global memory, so only prologues (barrier and
// table set-up, tensor-memory allocation) and launch latency overlap.  Falls back to an ordinary launch when switched off.
template <typename... KArgs, typename... Args>
cudaError_t launch_k(const b200moe_ctx * ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (ctx->overlap && ctx->overlap_now) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Exact re-quantisation behind the tensor-core gate/up GEMM (requant_fixup.cuh): list the values of `hidden` whose int8
// rounding the GEMM's error could change, recompute them with the integer lane chains, patch `hidden`.
// The list lives in the `down` output buffer, which is not in use yet.
// after the kind::f16 GEMM (activations as fp16 hi + lo):
constexpr float FIX_STEP_MARGIN = 0.015f;  // quantisation steps; largest GEMM error measured: 3.8e-3 steps (p99.99: 1.8e-3)
constexpr float FIX_REL_MARGIN = 1.2e-4f;  // of the block maximum; largest error measured: 3.0e-5 of it
// after the block-scaled FP4 GEMM (exact digit planes; only fp32 accumulation differs):
constexpr float FIX_STEP_MARGIN_FP4 = 2.5e-3f;  // largest error measured: 2.3e-4 steps (p99.99: 1.0e-4)
constexpr float FIX_REL_MARGIN_FP4 = 2.0e-5f;   // largest error measured: 1.8e-6 of the block maximum

// need_router / need_experts: which weight pointers the entry point is going to read
int validate_layer(b200moe_ctx * ctx, const b200moe_layer * l, bool need_router = true, bool need_experts = true) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (!l) return fail(ctx, B200MOE_ERR_INVALID_ARG, "layer is null");
    if (l->n_embd <= 0 || l->n_expert <= 0 || l->n_expert_used <= 0 || l->n_ff <= 0 || l->n_latent < 0)
        return fail(ctx, B200MOE_ERR_INVALID_ARG, "non-positive layer dimension");
    if (l->n_expert_used > l->n_expert) return fail(ctx, B200MOE_ERR_INVALID_ARG, "n_expert_used > n_expert");
    if (l->n_expert_used > 32) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "n_expert_used > 32");
    if (l->n_expert > 1024) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "at most 1024 experts");
    if (need_router && l->n_expert % 8) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "routing needs n_expert to be a multiple of 8");
    if (l->n_embd % 32) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "n_embd must be a multiple of 32");
    if (l->wtype != TYPE_NVFP4 && l->wtype != TYPE_Q3_K) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "expert type %d has no kernel", l->wtype);
    const int n_in = l->n_latent ? l->n_latent : l->n_embd;
    if (!gemv_supported(l->wtype, n_in) || !gemv_supported(l->wtype, l->n_ff))
        return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no kernel for widths n_in=%d n_ff=%d of type %d", n_in, l->n_ff, l->wtype);
    if (l->n_latent && !gemv_supported(l->wtype, l->n_embd)) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no kernel for n_embd=%d", l->n_embd);
    if (l->n_ff % 8 || n_in % 8) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "row counts must be multiples of 8");
    if (need_router && !l->router_w) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null router weight pointer");
    if (need_experts && (!l->gate || !l->up || !l->down)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null weight pointer");
    if (need_router && need_experts && l->n_latent && (!l->lat_down || !l->lat_up))
        return fail(ctx, B200MOE_ERR_INVALID_ARG, "latent layer without projections");
    if (l->gate_shexp || l->up_shexp || l->down_shexp || l->gate_inp_shexp || l->n_ff_shexp) {
        if (!l->gate_shexp || !l->up_shexp || !l->down_shexp || !l->gate_inp_shexp || l->n_ff_shexp <= 0)
            return fail(ctx, B200MOE_ERR_INVALID_ARG, "shared expert needs its three matrices, its gate vector and n_ff_shexp");
        if (l->n_latent) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "shared expert on a latent layer");
        if (!gemv_supported(l->wtype, l->n_ff_shexp) || l->n_ff_shexp % 8)
            return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no kernel for shared-expert width %d of type %d", l->n_ff_shexp, l->wtype);
    }
    const uintptr_t al = (uintptr_t) l->gate | (uintptr_t) l->up | (uintptr_t) l->down | (uintptr_t) l->lat_down | (uintptr_t) l->lat_up |
                         (uintptr_t) l->gate_shexp | (uintptr_t) l->up_shexp | (uintptr_t) l->down_shexp;
    if (al & 15) return fail(ctx, B200MOE_ERR_INVALID_ARG, "quantised tensors must be 16-byte aligned");
    return B200MOE_OK;
}

int ensure_plan(b200moe_ctx * ctx, int n_embd, int n_in, int n_expert, int k, int n_ff, int wtype, int tokens, int n_ff_sh = 0) {
    Plan & p = ctx->plan;
    if (p.max_tokens >= tokens && p.n_embd == n_embd && p.n_in == n_in && p.n_expert == n_expert && p.k == k && p.n_ff == n_ff &&
        p.wtype == wtype && p.n_ff_sh >= n_ff_sh && ctx->scratch.base)
        return B200MOE_OK;
    Plan np;
    np.max_tokens = std::max(tokens, 1);
    np.n_embd = n_embd; np.n_in = n_in; np.n_expert = n_expert; np.k = k; np.n_ff = n_ff; np.wtype = wtype; np.n_ff_sh = n_ff_sh;
    carve(np, nullptr);
    if (np.total > ctx->scratch.bytes) {
        CUDA_TRY(ctx, cudaDeviceSynchronize());
        if (ctx->scratch.base) cudaFree(ctx->scratch.base);
        ctx->scratch.base = nullptr;
        ctx->scratch.bytes = 0;
        void * ptr = nullptr;
        if (cudaMalloc(&ptr, np.total) != cudaSuccess) {
            cudaGetLastError();
            ctx->plan = Plan{};
            return fail(ctx, B200MOE_ERR_ALLOC, "cannot allocate %zu bytes of device scratch", np.total);
        }
        ctx->scratch.base = static_cast<uint8_t *>(ptr);
        ctx->scratch.bytes = np.total;
    }
    carve(np, ctx->scratch.base);   // nothing needs clearing: every buffer is written by the call that reads it
    ctx->plan = np;
    return B200MOE_OK;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to the (function, device) pair, and one process may hold contexts on
// several devices: every kernel instantiation keeps one flag per device ordinal.
constexpr int MAX_DEVICE_ORDINALS = 64;

template <typename Kern>
int raise_smem_limit(b200moe_ctx * ctx, Kern kern, size_t smem, bool (&done)[MAX_DEVICE_ORDINALS]) {
    if (ctx->device < 0 || ctx->device >= MAX_DEVICE_ORDINALS) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "device ordinal %d out of range", ctx->device);
    if (!done[ctx->device]) {
        CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        done[ctx->device] = true;
    }
    return B200MOE_OK;
}

int check_launch(b200moe_ctx * ctx, const char * what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ctx, B200MOE_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return B200MOE_OK;
}

// ---- kernel dispatch -----------------------------------------------------------------------------------
template <int WT, int K, bool DUAL, int NT>
int launch_gemv_t(b200moe_ctx * ctx, const GemvParams & p, cudaStream_t st) {
    constexpr int GEMV_STAGES = gemv_stages<WT, K, DUAL>();
    constexpr size_t smem = gemv_smem_bytes<WT, K, DUAL, NT, GEMV_STAGES>();
    static_assert(smem <= 227 * 1024, "ring does not fit shared memory");
    auto kern = expert_gemv_kernel<WT, K, DUAL, NT, GEMV_STAGES>;
    static bool configured[MAX_DEVICE_ORDINALS] = {};  // per instantiation and device
    if (int rc = raise_smem_limit(ctx, kern, smem, configured)) return rc;
    b200moe_ctx::Timed tm{};
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventCreate(&tm.beg));
        CUDA_TRY(ctx, cudaEventCreate(&tm.end));
        tm.kind = DUAL ? 0 : ctx->dense_now ? 2 : 1;
        CUDA_TRY(ctx, cudaEventRecord(tm.beg, st));
    }
    launch_k(ctx, kern, dim3(ctx->sm_count), dim3(GemvCfg<WT, K>::NWARPS * 32), smem, st, p);
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventRecord(tm.end, st));
        ctx->timed.push_back(tm);
    }
    return check_launch(ctx, "expert_gemv");
}

// One or two tokens: the whole call is a few thousand weight rows.  Four-warp CTAs with a single 16-row stage, several per SM,
// give every CTA one pass over one chunk instead of two or three passes of a half-empty eight-warp CTA.
template <int WT, int K, bool DUAL>
int launch_gemv_tiny(b200moe_ctx * ctx, const GemvParams & p, int rows, cudaStream_t st) {
    constexpr int NW = 4;
    constexpr size_t smem = gemv_smem_bytes<WT, K, DUAL, 1, 1, NW>();
    auto kern = expert_gemv_kernel<WT, K, DUAL, 1, 1, NW>;
    static bool configured[MAX_DEVICE_ORDINALS] = {};  // per instantiation and device
    if (int rc = raise_smem_limit(ctx, kern, smem, configured)) return rc;
    b200moe_ctx::Timed tm{};
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventCreate(&tm.beg));
        CUDA_TRY(ctx, cudaEventCreate(&tm.end));
        tm.kind = DUAL ? 0 : ctx->dense_now ? 2 : 1;
        CUDA_TRY(ctx, cudaEventRecord(tm.beg, st));
    }
    // one CTA per stage-sized chunk; at most `rows` experts are active, CTAs past the end of the row list leave at once
    const int64_t chunks = ((int64_t) rows * p.n_out + GemvCfg<WT, K, NW>::ROWS_PER_STAGE - 1) / GemvCfg<WT, K, NW>::ROWS_PER_STAGE;
    const int grid = (int) std::max<int64_t>(1, chunks);
    launch_k(ctx, kern, dim3(grid), dim3(NW * 32), smem, st, p);
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventRecord(tm.end, st));
        ctx->timed.push_back(tm);
    }
    return check_launch(ctx, "expert_gemv");
}

template <int WT, int K, bool DUAL>
int launch_gemv_k(b200moe_ctx * ctx, const GemvParams & p, int nt, cudaStream_t st) {
    if constexpr (DUAL && K > 2048) {
        return fail(ctx, B200MOE_ERR_UNSUPPORTED, "fused gate/up kernel is not built for K=%d", K);
    } else {
        if (nt <= 0) return launch_gemv_tiny<WT, K, DUAL>(ctx, p, -nt, st);   // nt = -(routed rows): the one-or-two-token kernel
        if (nt <= 1) return launch_gemv_t<WT, K, DUAL, 1>(ctx, p, st);
        return launch_gemv_t<WT, K, DUAL, 4>(ctx, p, st);
    }
}

template <bool DUAL>
int launch_gemv(b200moe_ctx * ctx, int wtype, int k, const GemvParams & p, int nt, cudaStream_t st) {
#define CASE(WT, KK) \
    if (wtype == WT && k == KK) return launch_gemv_k<WT, KK, DUAL>(ctx, p, nt, st);
    CASE(TYPE_NVFP4, 256) CASE(TYPE_NVFP4, 512) CASE(TYPE_NVFP4, 768) CASE(TYPE_NVFP4, 1024) CASE(TYPE_NVFP4, 2048) CASE(TYPE_NVFP4, 4096)
    CASE(TYPE_Q3_K, 256) CASE(TYPE_Q3_K, 512) CASE(TYPE_Q3_K, 768) CASE(TYPE_Q3_K, 2048)
#undef CASE
    return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no expert kernel for type %d width %d", wtype, k);
}

// ---- tensor maps for the warp-specialised grouped GEMM (the encoder is a host-side driver entry point; looked up
// once through the runtime so the library does not link against the driver library)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void * ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        else
            cudaGetLastError();
    }
    return fn;
}

// 2-D map over a row-major [outer][inner] array whose rows are pitch_bytes apart
int make_map_2d(b200moe_ctx * ctx, CUtensorMap * m, CUtensorMapDataType dt, const void * base, uint64_t inner, uint64_t outer,
                uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(ctx, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = { inner, outer };
    const cuuint64_t strides[1] = { pitch_bytes };
    const cuuint32_t box[2] = { box_inner, box_outer };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = fn(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, B200MOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int) r);
    return B200MOE_OK;
}

template <int K, bool DUAL, int NT>
int launch_gemm_t(b200moe_ctx * ctx, const MmaParams & p, int rows, cudaStream_t st) {
    using C = GemmCfg<K, DUAL, NT>;
    auto kern = expert_gemm_nvfp4_kernel<K, DUAL, NT>;
    static bool configured[MAX_DEVICE_ORDINALS] = {};  // per instantiation and device
    if (int rc = raise_smem_limit(ctx, kern, C::SMEM, configured)) return rc;
    constexpr uint64_t ROW_BYTES = K / 64 * 36;
    CUtensorMap mw0, mw1, mhi, mlo;
    int rc;
    const uint64_t wrows = (uint64_t) p.n_as * p.n_out;
    if ((rc = make_map_2d(ctx, &mw0, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w0, ROW_BYTES, wrows, ROW_BYTES, GEMM_RAW_ROW, 128, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    if (DUAL) {
        if ((rc = make_map_2d(ctx, &mw1, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w1, ROW_BYTES, wrows, ROW_BYTES, GEMM_RAW_ROW, 128, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    } else {
        mw1 = mw0;
    }
    if ((rc = make_map_2d(ctx, &mhi, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.act, K, (uint64_t) rows, (uint64_t) K * 2, 64, NT, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_map_2d(ctx, &mlo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.act_lo, K, (uint64_t) rows, (uint64_t) K * 2, 64, NT, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    b200moe_ctx::Timed tm{};
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventCreate(&tm.beg));
        CUDA_TRY(ctx, cudaEventCreate(&tm.end));
        tm.kind = DUAL ? 0 : ctx->dense_now ? 2 : 1;
        CUDA_TRY(ctx, cudaEventRecord(tm.beg, st));
    }
    kern<<<dim3(ctx->sm_count), dim3(GEMM_THREADS), C::SMEM, st>>>(p, mw0, mw1, mhi, mlo);   // never as a programmatic dependent (layer_overlap)
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventRecord(tm.end, st));
        ctx->timed.push_back(tm);
    }
    return check_launch(ctx, "expert_gemm");
}

// tokens on the M side, 256 weight rows per instruction; activations as alternating hi / lo rows
template <int K, bool DUAL>
int launch_gemm_tm_t(b200moe_ctx * ctx, const MmaParams & p, int rows, cudaStream_t st) {
    using C = GemmTmCfg<K>;
    auto kern = expert_gemm_tm_kernel<K, DUAL>;
    static bool configured[MAX_DEVICE_ORDINALS] = {};  // per instantiation and device
    if (int rc = raise_smem_limit(ctx, kern, C::SMEM, configured)) return rc;
    constexpr uint64_t ROW_BYTES = K / 64 * 36;
    CUtensorMap mw0, mw1, mact;
    int rc;
    const uint64_t wrows = (uint64_t) p.n_as * p.n_out;
    if ((rc = make_map_2d(ctx, &mw0, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w0, ROW_BYTES, wrows, ROW_BYTES, GEMM_RAW_ROW, 128, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    if (DUAL) {
        if ((rc = make_map_2d(ctx, &mw1, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.w1, ROW_BYTES, wrows, ROW_BYTES, GEMM_RAW_ROW, 128, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    } else {
        mw1 = mw0;
    }
    if ((rc = make_map_2d(ctx, &mact, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.act, K, 2 * (uint64_t) rows, (uint64_t) K * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    b200moe_ctx::Timed tm{};
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventCreate(&tm.beg));
        CUDA_TRY(ctx, cudaEventCreate(&tm.end));
        tm.kind = DUAL ? 0 : ctx->dense_now ? 2 : 1;
        CUDA_TRY(ctx, cudaEventRecord(tm.beg, st));
    }
    kern<<<dim3(ctx->sm_count), dim3(GEMM_TM_THREADS), C::SMEM, st>>>(p, mw0, mw1, mact);   // never as a programmatic dependent (layer_overlap)
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventRecord(tm.end, st));
        ctx->timed.push_back(tm);
    }
    return check_launch(ctx, "expert_gemm_tm");
}

template <bool DUAL>
int launch_gemm_tm(b200moe_ctx * ctx, int k, const MmaParams & p, int rows, cudaStream_t st) {
#define GEMM_CASE(KK) case KK: return launch_gemm_tm_t<KK, DUAL>(ctx, p, rows, st);
    switch (k) { GEMM_CASE(256) GEMM_CASE(512) GEMM_CASE(768) GEMM_CASE(1024) GEMM_CASE(2048) }
#undef GEMM_CASE
    return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no tensor-core expert kernel for width %d", k);
}

// small_tiles: experts see few rows each (batched decode) -> 32-row token tiles, else 128
template <bool DUAL>
int launch_gemm(b200moe_ctx * ctx, int k, const MmaParams & p, int rows, bool small_tiles, cudaStream_t st) {
#define GEMM_CASE(KK) case KK: return small_tiles ? launch_gemm_t<KK, DUAL, 32>(ctx, p, rows, st) : launch_gemm_t<KK, DUAL, 128>(ctx, p, rows, st);
    switch (k) { GEMM_CASE(256) GEMM_CASE(512) GEMM_CASE(768) GEMM_CASE(1024) GEMM_CASE(2048) }
#undef GEMM_CASE
    return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no tensor-core expert kernel for width %d", k);
}

// block-scaled FP4 grouped GEMM (expert_gemm_fp4.cuh): digit planes of the routed rows, then the GEMM
template <int K, bool DUAL>
int launch_gemm_fp4_t(b200moe_ctx * ctx, const Fp4Params & fp, const void * w0, const void * w1, const uint8_t * planes, int rows, cudaStream_t st) {
    using C = Fp4Cfg<K>;
    auto kern = expert_gemm_fp4_kernel<K, DUAL>;
    static bool configured[MAX_DEVICE_ORDINALS] = {};  // per instantiation and device
    if (int rc = raise_smem_limit(ctx, kern, C::SMEM, configured)) return rc;
    constexpr uint64_t ROW_BYTES = K / 64 * 36;
    CUtensorMap mw0, mw1, mpl;
    int rc;
    const uint64_t wrows = (uint64_t) fp.n_as * fp.n_out;
    if ((rc = make_map_2d(ctx, &mw0, CU_TENSOR_MAP_DATA_TYPE_UINT8, w0, ROW_BYTES, wrows, ROW_BYTES, GEMM_RAW_ROW, 128, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    if (DUAL) {
        if ((rc = make_map_2d(ctx, &mw1, CU_TENSOR_MAP_DATA_TYPE_UINT8, w1, ROW_BYTES, wrows, ROW_BYTES, GEMM_RAW_ROW, 128, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    } else {
        mw1 = mw0;
    }
    const uint64_t prows = std::max<uint64_t>((uint64_t) rows * FP4_PLANES, FP4_NROW);
    if ((rc = make_map_2d(ctx, &mpl, CU_TENSOR_MAP_DATA_TYPE_UINT8, planes, K / 2, prows, K / 2, 128, FP4_NROW, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    b200moe_ctx::Timed tm{};
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventCreate(&tm.beg));
        CUDA_TRY(ctx, cudaEventCreate(&tm.end));
        tm.kind = DUAL ? 0 : ctx->dense_now ? 2 : 1;
        CUDA_TRY(ctx, cudaEventRecord(tm.beg, st));
    }
#ifdef B200MOE_FP4_PROF
    static long long * d_prof = nullptr;
    if (!d_prof) cudaMalloc(&d_prof, sizeof(long long) * 24 * 256);
    cudaMemsetAsync(d_prof, 0, sizeof(long long) * 24 * 256, st);
    Fp4Params fpp2 = fp;
    fpp2.prof = d_prof;
    kern<<<ctx->sm_count, FP4_THREADS, C::SMEM, st>>>(fpp2, mw0, mw1, mpl);
    if (getenv("B200MOE_FP4_PROF_PRINT")) {
        std::vector<long long> h(24 * 256);
        cudaStreamSynchronize(st);
        cudaMemcpy(h.data(), d_prof, sizeof(long long) * 24 * 256, cudaMemcpyDeviceToHost);
        const char * names[16] = {"raw: wait raw_empty", "raw: total", "act: wait act_empty", "act: total", "mma: wait acc_empty", "mma: wait act_full", "mma: wait tile+sf_full", "mma: total",
                                  "epi: wait acc_full", "epi: total", "repack: wait raw_full", "repack: wait tile_empty", "repack: total",
                                  "sfcopy: wait act_full", "sfcopy: wait tile_full", "sfcopy: total"};
        printf("fp4 kernel K=%d DUAL=%d role cycles (mean over CTAs / max):\n", K, (int) DUAL);
        for (int k = 0; k < 16; ++k) {
            double sum = 0; long long mx = 0;
            for (int b = 0; b < ctx->sm_count; ++b) { sum += h[b * 24 + k]; mx = std::max(mx, h[b * 24 + k]); }
            printf("  %-26s %10.0f %10lld\n", names[k], sum / ctx->sm_count, mx);
        }
    }
#else
    kern<<<ctx->sm_count, FP4_THREADS, C::SMEM, st>>>(fp, mw0, mw1, mpl);
#endif
    if (ctx->timing) {
        CUDA_TRY(ctx, cudaEventRecord(tm.end, st));
        ctx->timed.push_back(tm);
    }
    return check_launch(ctx, "expert_gemm_fp4");
}

template <bool DUAL>
int launch_gemm_fp4(b200moe_ctx * ctx, int k, const Fp4Params & fp, const void * w0, const void * w1, const uint8_t * planes, int rows, cudaStream_t st) {
#define GEMM_CASE(KK) case KK: return launch_gemm_fp4_t<KK, DUAL>(ctx, fp, w0, w1, planes, rows, st);
    switch (k) { GEMM_CASE(256) GEMM_CASE(512) GEMM_CASE(768) GEMM_CASE(1024) GEMM_CASE(2048) GEMM_CASE(4096) }
#undef GEMM_CASE
    return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no FP4 tensor-core expert kernel for width %d", k);
}

// gate/up: 128 features per item; down: 256 rows per item
bool fp4_width(int k) { return k == 256 || k == 512 || k == 768 || k == 1024 || k == 2048 || k == 4096; }
bool fp4_supported(int wtype, int n_in, int n_ff) { return wtype == TYPE_NVFP4 && fp4_width(n_in) && fp4_width(n_ff) && n_ff % 128 == 0 && n_in % 256 == 0; }

// digit planes + scale tiles of the expert-sorted routed rows (input of the FP4 kernels)
// act: rows already on the int8 grid; or src != null: fp32 rows (src_stride floats apart) that are quantised (Q8_0) on the way.
// ids: expert of every routed row; n_as experts; the token-tile prefix lies behind the three work prefixes of the group tables.
// emit (with src): also receives the quantised rows (for the exact re-quantisation fix-up, which recomputes with them)
int launch_act_planes(b200moe_ctx * ctx, ActQuant act, const float * src, const int32_t * ids, int rows, int k, int n_ids, int ne11, int n_as,
                      cudaStream_t st, ActQuant emit = ActQuant{}, int64_t src_stride = 0) {
    Plan & p = ctx->plan;
    PlaneOut po{ reinterpret_cast<uint8_t *>(p.afp16), p.asf, p.arow_scale, p.groups.pos /* free once the rows are grouped */ };
    const int * tiles = p.groups.cost + 3 * (n_as + 1);
    if (src_stride == 0) src_stride = k;
    if (src && (((uintptr_t) src & 15) || src_stride % 4)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "fp32 activation rows must be 16-byte aligned");
    const int rows_per_block = 256 / std::min(256, k / 8);
    const unsigned blocks = (unsigned) ((rows + rows_per_block - 1) / rows_per_block);
    if (src) act_planes_kernel<true><<<blocks, 256, 0, st>>>(act, src, src_stride, p.groups.perm, ids, p.groups.offsets, tiles, p.groups.meta, rows, k, n_ids, ne11, n_as, po, emit);
    else act_planes_kernel<false><<<blocks, 256, 0, st>>>(act, nullptr, 0, p.groups.perm, ids, p.groups.offsets, tiles, p.groups.meta, rows, k, n_ids, ne11, n_as, po, ActQuant{});
    return check_launch(ctx, "act_planes");
}

Fp4Params fp4_params(b200moe_ctx * ctx, const float * s0, const float * s1, float * out, int n_out, int n_as) {
    Plan & p = ctx->plan;
    Fp4Params f{};
    f.scale0 = s0; f.scale1 = s1; f.sf = p.asf; f.row_scale = p.arow_scale; f.offsets = p.groups.offsets; f.perm = p.groups.perm;
    f.active = p.groups.active; f.meta = p.groups.meta; f.tile_of_expert = p.groups.cost + 3 * (n_as + 1); f.tile_expert = p.groups.pos; f.out = out; f.n_out = n_out;
    f.n_as = n_as; f.err = ctx->d_err; f.prof = nullptr;
    return f;
}

bool mma_supported(int wtype, int k, int n_out) {
    return wtype == TYPE_NVFP4 && n_out % 128 == 0 && (k == 256 || k == 512 || k == 768 || k == 1024 || k == 2048);
}

// expert-sorted fp16 copy of quantised activations (input of the tensor-core kernels)
int launch_sorted_act(b200moe_ctx * ctx, ActQuant act, int rows, int k, int n_ids, int ne11, bool interleaved, cudaStream_t st) {
    Plan & p = ctx->plan;
    const int64_t warps = (int64_t) rows * (k / 32);
    __half * lo = interleaved ? p.afp16 + k : p.afp16 + (size_t) rows * k;
    launch_k(ctx, sorted_act_fp16_kernel, dim3((unsigned) ((warps * 32 + 255) / 256)), dim3(256), 0, st, act, p.groups.perm, p.groups.meta, rows, k, n_ids, ne11,
             p.afp16, lo, interleaved ? 2 * k : k);
    return check_launch(ctx, "sorted_act_fp16");
}

template <typename XT>
int launch_quantize(b200moe_ctx * ctx, const XT * src, int64_t stride, ActQuant dst, int rows, int k, int wtype, cudaStream_t st) {
    const int kind = wtype == TYPE_Q3_K ? 1 : 0;
    const int64_t warps = (int64_t) rows * (kind ? k / 256 : k / 32);
    if (warps == 0) return B200MOE_OK;
    const int blocks = (int) ((warps * 32 + 255) / 256);
    launch_k(ctx, quantize_act_kernel<XT>, dim3(blocks), dim3(256), 0, st, src, stride, dst, rows, k, kind);
    return check_launch(ctx, "quantize_act");
}

template <int WE, int WT, typename XT>
int launch_logits_smem(b200moe_ctx * ctx, const float * w, const float * bias, const XT * x, float * logits, int H, int E, int T, int * zero_buf,
                       int zero_n, cudaStream_t st) {
    auto kern = router_logits_smem_kernel<WE, WT, XT>;
    constexpr size_t smem = router_smem_bytes<WE, WT, XT>();
    static bool configured[MAX_DEVICE_ORDINALS] = {};
    if (int rc = raise_smem_limit(ctx, kern, smem, configured)) return rc;
    const int blocks = ((E + 8 * WE - 1) / (8 * WE)) * ((T + 8 * WT - 1) / (8 * WT));
    kern<<<blocks, WE * WT * 32, smem, st>>>(w, bias, x, logits, H, E, T, zero_buf, zero_n);
    return check_launch(ctx, "router_logits");
}

// F32 matrix times a batch in the reference's summation order: logits [T][E] = W [E][H] . x [T][H] (+ bias)
template <typename XT>
int launch_logits_any(b200moe_ctx * ctx, const float * w, const float * bias, const XT * x, float * logits, int H, int E, int T, int * zero_buf,
                      int zero_n, cudaStream_t st) {
    const bool staged = T >= 16 && H % ROUTER_KC == 0 && (((uintptr_t) w | (uintptr_t) x) & 15) == 0;
    if (staged) {   // shared-memory tiles: 32 experts x 16 tokens when that fills the GPU, else 16 x 8
        const int big = ((E + 31) / 32) * ((T + 15) / 16);
        if (big >= ctx->sm_count) return launch_logits_smem<4, 2, XT>(ctx, w, bias, x, logits, H, E, T, zero_buf, zero_n, st);
        return launch_logits_smem<2, 1, XT>(ctx, w, bias, x, logits, H, E, T, zero_buf, zero_n, st);
    }
    if (T >= 16) {   // batches: 4 experts x 8 tokens per warp
        constexpr int TE = 4, TT = 8;
        const int64_t warps = (int64_t) ((E + TE - 1) / TE) * ((T + TT - 1) / TT);
        router_logits_tiled_kernel<TE, TT, XT><<<(unsigned) ((warps * 32 + 255) / 256), 256, 0, st>>>(w, bias, x, logits, H, E, T, zero_buf, zero_n);
        return check_launch(ctx, "router_logits");
    }
    constexpr int TT = 4;
    const int64_t warps = (int64_t) E * ((T + TT - 1) / TT);
    router_logits_kernel<TT, XT><<<(unsigned) ((warps * 32 + 255) / 256), 256, 0, st>>>(w, bias, x, logits, H, E, T, zero_buf, zero_n);
    return check_launch(ctx, "router_logits");
}

template <typename XT>
int launch_logits(b200moe_ctx * ctx, const b200moe_layer * l, const XT * x, int T, cudaStream_t st) {
    Plan & p = ctx->plan;
    return launch_logits_any<XT>(ctx, l->router_w, l->router_bias, x, p.logits, l->n_embd, l->n_expert, T, p.groups.counts, l->n_expert, st);
}

template <int TT, typename XT>
int launch_front_t(b200moe_ctx * ctx, const b200moe_layer * l, const XT * x, int T, cudaStream_t st) {
    Plan & p = ctx->plan;
    const int64_t lwarps = (int64_t) l->n_expert * ((T + TT - 1) / TT);
    const int lblocks = (int) ((lwarps * 32 + 255) / 256);
    const int kind = l->wtype == TYPE_Q3_K ? 1 : 0;
    const int64_t qwarps = (int64_t) T * (kind ? l->n_embd / 256 : l->n_embd / 32);
    const int qblocks = (int) ((qwarps * 32 + 255) / 256);
    launch_k(ctx, route_front_kernel<TT, XT>, dim3(lblocks + qblocks), dim3(256), 0, st, l->router_w, l->router_bias, x, p.logits, l->n_embd,
             l->n_expert, T, p.groups.counts, l->n_expert, lblocks, p.xq, kind);
    return check_launch(ctx, "route_front");
}

template <typename XT>
int launch_front(b200moe_ctx * ctx, const b200moe_layer * l, const XT * x, int T, cudaStream_t st) {
    // few tokens: one warp per (expert, token) with deep load prefetch; otherwise 4 tokens share each weight load
    return T <= 8 ? launch_front_t<1, XT>(ctx, l, x, T, st) : launch_front_t<4, XT>(ctx, l, x, T, st);
}

int launch_select_group(b200moe_ctx * ctx, const b200moe_layer * l, int T, float * probs, cudaStream_t st) {
    Plan & p = ctx->plan;
    const int E = l->n_expert, K = l->n_expert_used;
    const size_t sh = (size_t) (3 * E + 1) * sizeof(int);
#define SELG(EPL) launch_k(ctx, route_select_group_kernel<EPL>, dim3(1), dim3(1024), sh, st, p.logits, E, K, T, p.ids, p.wts, probs, p.groups, ctx->d_err)
    if (E <= 32) SELG(1);
    else if (E <= 64) SELG(2);
    else if (E <= 128) SELG(4);
    else if (E <= 256) SELG(8);
    else if (E <= 512) SELG(16);
    else SELG(32);
#undef SELG
    return check_launch(ctx, "route_select_group");
}

int launch_select(b200moe_ctx * ctx, const b200moe_layer * l, int T, int32_t * ids, float * wts, float * probs, bool count, cudaStream_t st) {
    Plan & p = ctx->plan;
    const int blocks = (T * 32 + 255) / 256;
    const int E = l->n_expert, K = l->n_expert_used;
    int * counts = count ? p.groups.counts : nullptr;
#define SEL(EPL) launch_k(ctx, route_select_kernel<EPL>, dim3(blocks), dim3(256), 0, st, p.logits, E, K, T, ids, wts, probs, counts, p.groups.pos)
    if (E <= 32) SEL(1);
    else if (E <= 64) SEL(2);
    else if (E <= 128) SEL(4);
    else if (E <= 256) SEL(8);
    else if (E <= 512) SEL(16);
    else SEL(32);
#undef SEL
    return check_launch(ctx, "route_select");
}

int launch_group(b200moe_ctx * ctx, const int32_t * ids, int E, int rows, cudaStream_t st, bool allow_empty = false) {
    Plan & p = ctx->plan;
    const size_t sh = (size_t) (3 * E + 1) * sizeof(int);
    launch_k(ctx, group_scan_kernel, dim3(1), dim3(1024), sh, st, p.groups, ids, E, rows, ctx->d_err, allow_empty ? 1 : 0);
    return check_launch(ctx, "group_scan");
}

GemvParams gemv_params(b200moe_ctx * ctx, const void * w0, const void * w1, const float * s0, const float * s1, ActQuant act, float * out,
                       int n_out, int n_ids, int ne11, int n_as) {
    Plan & p = ctx->plan;
    GemvParams g{};
    g.w0 = static_cast<const uint8_t *>(w0);
    g.w1 = static_cast<const uint8_t *>(w1);
    g.scale0 = s0;
    g.scale1 = s1;
    g.act = act;
    g.offsets = p.groups.offsets;
    g.perm = p.groups.perm;
    g.active = p.groups.active;
    g.meta = p.groups.meta;
    g.cost = p.groups.cost;
    g.out = out;
    g.w_stride = n_out;
    g.n_out = n_out;
    g.n_ids = n_ids;
    g.ne11 = ne11;
    g.n_as = n_as;
    g.err = ctx->d_err;
    return g;
}

// activation rows per pass of the integer kernel: 4, 1 when experts see about one row each, -(rows) selects the
// one-or-two-token kernel
int tokens_per_pass(int rows, int n_as) { return rows <= 16 ? -rows : rows <= n_as ? (rows <= 32 ? 1 : 4) : 4; }

__global__ void scale_rows_kernel(float * v, const float * s, size_t n) {
    pdl_wait();
    pdl_launch_dependents();

    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] = __fmul_rn(v[i], s[0]);
}

__global__ void bf16_to_f32_kernel(const __nv_bfloat16 * src, float * dst, size_t n) {
    pdl_wait();
    pdl_launch_dependents();

    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __bfloat162float(src[i]);
}

// token t belongs to group t / group_size
__global__ void fill_group_ids_kernel(int * ids, int T, int group_size) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T) ids[t] = t / group_size;
}

// Dense quantised matvec y[T][n_out] = W[n_out][k] . x[T][k] on the indexed-matmul kernel: the tokens are cut into up to 32
// groups that all point at the same matrix (expert stride 0), so a matrix with few rows and many tokens still fills the grid
// (one group would leave a 1024-row matrix on a fifth of the SMs, walking all tokens in turn).  The matrix is re-read from L2.
int dense_matmul_fp4(b200moe_ctx * ctx, const void * w, const float * scale, const float * x, int k, int n_out, int T, float * y, cudaStream_t st,
                     bool exact_requant, ActQuant xq, void * list_room, size_t list_room_bytes, const void * w1 = nullptr);

// a[i] = silu(a[i]) * b[i]: ggml_silu then ggml_mul, the same bits as the fused swiglu of the expert kernels
__global__ void silu_mul_kernel(float * __restrict__ a, const float * __restrict__ b, size_t n) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = __fmul_rn(ggml_silu(a[i]), b[i]);
}

// Shared expert onto the routed sum (forward.cpp:313-314): gated = sh * sigmoid(logit), out += gated.  The reference's
// sigmoid is 1 / (1 + expf(-x)) through the C library (ggml-cpu/vec.h:936); expf is evaluated here as the double-precision
// exponential rounded to float, which is the correctly rounded value but for double-rounding cases rarer than 1 in 2^28.
__global__ void shexp_add_kernel(float * __restrict__ out, const float * __restrict__ sh, const float * __restrict__ logit, int H, int T,
                                 float * __restrict__ gated_out) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T || i >= H) return;
    const float e = (float) exp((double) -logit[t]);
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
    const size_t at = (size_t) t * H + i;
    const float g = __fmul_rn(sh[at], sig);
    if (gated_out) gated_out[at] = g;
    out[at] = __fadd_rn(out[at], g);
}

// The FP4 tensor-core kernel takes a dense product when the type and shape fit, several tokens share the matrix, and the caller
// has not asked for bit-identical results (expert paths 1, 5 and 7 are the ones documented as bit-identical).
bool dense_on_fp4(const b200moe_ctx * ctx, int wtype, int k, int n_out, int T) {
    const int path = ctx->expert_path;
    return wtype == TYPE_NVFP4 && fp4_width(k) && n_out % 256 == 0 && T >= 4 && path != 1 && path != 5 && path != 7;
}

// exact_requant: see dense_matmul_fp4; `hidden` scratch holds the list (free before the experts run)
// w1 != null: y = silu(w . x) * (w1 . x), the gate/up pair of a dense expert in one pass over x (no tensor scales, no exact_requant);
// y1_tmp [T][n_out] is used when the pair cannot be fused (integer kernel beyond 2048 columns)
int dense_matvec(b200moe_ctx * ctx, int wtype, const void * w, const float * scale, const float * x, ActQuant xq, int k, int n_out, int T,
                 float * y, cudaStream_t st, bool exact_requant = false, const void * w1 = nullptr, float * y1_tmp = nullptr) {
    Plan & p = ctx->plan;
    struct DenseMark { b200moe_ctx * c; DenseMark(b200moe_ctx * c_) : c(c_) { c->dense_now = true; } ~DenseMark() { c->dense_now = false; } } mark(ctx);
    if (dense_on_fp4(ctx, wtype, k, n_out, T) && (!exact_requant || n_out % 128 == 0))
        return dense_matmul_fp4(ctx, w, scale, x, k, n_out, T, y, st, exact_requant, xq, p.hid, (size_t) p.max_tokens * p.k * p.n_ff * sizeof(float), w1);
    int rc;
    if (w1 && k > 2048) {   // the fused pair is not built for this width: two products, then silu(a) * b
        if ((rc = dense_matvec(ctx, wtype, w, nullptr, x, xq, k, n_out, T, y, st))) return rc;
        if ((rc = dense_matvec(ctx, wtype, w1, nullptr, x, xq, k, n_out, T, y1_tmp, st))) return rc;
        const size_t n = (size_t) T * n_out;
        silu_mul_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, st>>>(y, y1_tmp, n);
        return check_launch(ctx, "silu_mul");
    }
    if ((rc = launch_quantize<float>(ctx, x, k, xq, T, k, wtype, st))) return rc;
    const int G = std::max(1, std::min({32, T / 8, p.n_expert}));
    const int gsize = (T + G - 1) / G;
    const int groups = (T + gsize - 1) / gsize;
    fill_group_ids_kernel<<<(T + 255) / 256, 256, 0, st>>>(p.one_group_ids, T, gsize);
    if ((rc = check_launch(ctx, "fill_group_ids"))) return rc;
    CUDA_TRY(ctx, cudaMemsetAsync(p.groups.counts, 0, sizeof(int) * std::max(groups, 8), st));
    count_ids_kernel<<<(T + 255) / 256, 256, 0, st>>>(p.one_group_ids, 1, 1, T, groups, p.groups.perm /*scratch: compact ids*/, p.groups.counts,
                                                      p.groups.pos, ctx->d_err);
    if ((rc = check_launch(ctx, "count_ids"))) return rc;
    // perm is about to be overwritten by the scan: read the ids from one_group_ids
    if ((rc = launch_group(ctx, p.one_group_ids, groups, T, st))) return rc;
    GemvParams g = gemv_params(ctx, w, w1, nullptr, nullptr, xq, y, n_out, 1, 1, groups);
    g.w_stride = 0;
    if (w1) return launch_gemv<true>(ctx, wtype, k, g, 4, st);
    if ((rc = launch_gemv<false>(ctx, wtype, k, g, 4, st))) return rc;
    if (scale) {
        const size_t n = (size_t) T * n_out;
        scale_rows_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, st>>>(y, scale, n);
        if ((rc = check_launch(ctx, "scale_rows"))) return rc;
    }
    return B200MOE_OK;
}

// The same product on the FP4 tensor-core kernel: the matrix is the single "expert" of a one-group routing, the tokens its routed
// rows (digit planes made straight from the fp32 activations).  Not bit-identical to the integer kernel: fp32 accumulation order.
template <int K>
int launch_fix_single_t(b200moe_ctx * ctx, const FixSingleParams & fp, cudaStream_t st) {
    requant_fix_single_kernel<K><<<ctx->sm_count * 8, 256, 0, st>>>(fp);
    return check_launch(ctx, "requant_fix_single");
}

// exact_requant: the caller re-quantises y (the latent down-projection): the values of y whose Q8_0 rounding the GEMM's error
// could change are recomputed with the integer kernel's arithmetic (requant_fixup.cuh), so the quantised y is the reference's.
// The list lives in `list_room`, memory the caller does not need yet.
int dense_matmul_fp4(b200moe_ctx * ctx, const void * w, const float * scale, const float * x, int k, int n_out, int T, float * y, cudaStream_t st,
                     bool exact_requant, ActQuant xq, void * list_room, size_t list_room_bytes, const void * w1) {
    Plan & p = ctx->plan;
    int rc;
    one_group_kernel<<<(T + 255) / 256, 256, 0, st>>>(p.groups, p.one_group_ids, T);
    if ((rc = check_launch(ctx, "one_group"))) return rc;
    // the fix-up recomputes with the quantised activations: have the plane kernel leave them in xq
    if ((rc = launch_act_planes(ctx, ActQuant{}, x, p.one_group_ids, T, k, 1, 1, 1, st, exact_requant ? xq : ActQuant{}))) return rc;
    if (w1) return launch_gemm_fp4<true>(ctx, k, fp4_params(ctx, nullptr, nullptr, y, n_out, 1), w, w1, reinterpret_cast<const uint8_t *>(p.afp16), T, st);
    if ((rc = launch_gemm_fp4<false>(ctx, k, fp4_params(ctx, scale, nullptr, y, n_out, 1), w, nullptr, reinterpret_cast<const uint8_t *>(p.afp16), T, st))) return rc;
    if (!exact_requant) return B200MOE_OK;
    FixList list;
    list.items = static_cast<int2 *>(list_room);
    list.count = p.groups.meta + 2;
    list.capacity = (int) std::min<size_t>(list_room_bytes / sizeof(int2), (size_t) T * n_out / 4);
    list.overflow = reinterpret_cast<unsigned long long *>(ctx->d_err + 2);
    CUDA_TRY(ctx, cudaMemsetAsync(list.count, 0, sizeof(int), st));
    const int64_t warps = (int64_t) T * (n_out / 128);
    requant_mark_kernel<<<(unsigned) ((warps * 32 + 255) / 256), 256, 0, st>>>(y, p.groups.perm, p.groups.meta, T, n_out, FIX_STEP_MARGIN_FP4, FIX_REL_MARGIN_FP4, list);
    if ((rc = check_launch(ctx, "requant_mark"))) return rc;
    FixSingleParams fs{ static_cast<const uint8_t *>(w), scale, xq, n_out, y, list, FIX_REL_MARGIN_FP4 };
    switch (k) {
        case 256: return launch_fix_single_t<256>(ctx, fs, st);
        case 512: return launch_fix_single_t<512>(ctx, fs, st);
        case 768: return launch_fix_single_t<768>(ctx, fs, st);
        case 1024: return launch_fix_single_t<1024>(ctx, fs, st);
        case 2048: return launch_fix_single_t<2048>(ctx, fs, st);
        case 4096: return launch_fix_single_t<4096>(ctx, fs, st);
    }
    return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no re-quantisation fix-up for width %d", k);
}

__global__ void gather_rows_kernel(const float4 * __restrict__ src, const int * __restrict__ idx, float4 * __restrict__ dst, int n_rows,
                                   int w4, int src_rows) {
    pdl_wait();
    pdl_launch_dependents();

    const int r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows || c >= w4) return;
    const int s = idx[r];
    if (s < 0 || s >= src_rows) return;  // out-of-range index: leave the row untouched rather than read outside src
    dst[(size_t) r * w4 + c] = src[(size_t) s * w4 + c];
}

int read_device_error(b200moe_ctx * ctx, cudaStream_t st) {
    CUDA_TRY(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, 16, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(ctx, cudaStreamSynchronize(st));
    ctx->counters.fixup_overflow = (int64_t) *reinterpret_cast<const unsigned long long *>(ctx->h_err + 2);
    if (*ctx->h_err != 0) {
        const int code = *ctx->h_err;
        cudaMemsetAsync(ctx->d_err, 0, sizeof(int), st);
        return fail(ctx, B200MOE_ERR_DEVICE_CHECK, "device check failed with code %d (1 barrier wait ran out, 2 expert id out of range, 3 shape)", code);
    }
    return B200MOE_OK;
}

template <typename XT>
int route_impl(b200moe_ctx * ctx, const b200moe_layer * l, const XT * x, int T, int32_t * ids, float * wts, const b200moe_observe * ob,
               bool count, cudaStream_t st) {
    Plan & p = ctx->plan;
    int rc = launch_logits<XT>(ctx, l, x, T, st);
    if (rc) return rc;
    float * probs = (ob && ob->ffn_moe_probs) ? ob->ffn_moe_probs : nullptr;
    if ((rc = launch_select(ctx, l, T, ids, wts, probs, count, st))) return rc;
    if (ob && ob->ffn_moe_logits)
        CUDA_TRY(ctx, cudaMemcpyAsync(ob->ffn_moe_logits, p.logits, sizeof(float) * (size_t) T * l->n_expert, cudaMemcpyDeviceToDevice, st));
    return B200MOE_OK;
}

template <int K>
int launch_fix_t(b200moe_ctx * ctx, const FixParams & fp, cudaStream_t st) {
    constexpr size_t smem = requant_fix_smem_bytes<K>();
    static bool configured[MAX_DEVICE_ORDINALS] = {};
    if (int rc = raise_smem_limit(ctx, requant_fix_kernel<K>, smem, configured)) return rc;
    launch_k(ctx, requant_fix_kernel<K>, dim3(ctx->sm_count * 8), dim3(256), smem, st, fp);
    return check_launch(ctx, "requant_fix");
}

int launch_requant_fixup(b200moe_ctx * ctx, const b200moe_layer * l, ActQuant xq, int rows, int n_in, int n_ids, bool after_fp4, cudaStream_t st) {
    Plan & p = ctx->plan;
    // two lists in the `down` output buffer (not in use yet): marked values, then the block-maximum candidates the first pass finds
    const size_t room = (size_t) rows * n_in * sizeof(float) / sizeof(int2);
    FixList list, more;
    list.items = reinterpret_cast<int2 *>(p.y);
    list.count = p.groups.meta + 2;
    list.capacity = (int) std::min<size_t>(room * 3 / 4, (size_t) rows * l->n_ff / 4);
    list.overflow = reinterpret_cast<unsigned long long *>(ctx->d_err + 2);
    more.items = list.items + room * 3 / 4;
    more.count = p.groups.meta + 3;
    more.capacity = (int) (room - room * 3 / 4);
    more.overflow = list.overflow;
    CUDA_TRY(ctx, cudaMemsetAsync(list.count, 0, 2 * sizeof(int), st));
    const int64_t warps = (int64_t) rows * (l->n_ff / 128);
    launch_k(ctx, requant_mark_kernel, dim3((unsigned) ((warps * 32 + 255) / 256)), dim3(256), 0, st, (const float *) p.hid,
             (const int *) p.groups.perm, (const int *) p.groups.meta, rows, l->n_ff, after_fp4 ? FIX_STEP_MARGIN_FP4 : FIX_STEP_MARGIN, after_fp4 ? FIX_REL_MARGIN_FP4 : FIX_REL_MARGIN, list);
    int rc = check_launch(ctx, "requant_mark");
    if (rc) return rc;
    FixParams fp{};
    fp.w0 = static_cast<const uint8_t *>(l->gate); fp.w1 = static_cast<const uint8_t *>(l->up);
    fp.scale0 = l->gate_scale; fp.scale1 = l->up_scale; fp.act = xq; fp.ids = p.ids; fp.n_ids = n_ids; fp.n_ff = l->n_ff;
    fp.n_as = l->n_expert; fp.hid = p.hid; fp.list = list; fp.more = more; fp.err = ctx->d_err; fp.rel_margin = after_fp4 ? FIX_REL_MARGIN_FP4 : FIX_REL_MARGIN;
    FixParams second = fp;      // the second pass recomputes what the first one found and looks no further
    second.list = more;
    second.more = FixList{};
    for (const FixParams * pass : { &fp, &second }) {
        switch (n_in) {
            case 256: rc = launch_fix_t<256>(ctx, *pass, st); break;
            case 512: rc = launch_fix_t<512>(ctx, *pass, st); break;
            case 768: rc = launch_fix_t<768>(ctx, *pass, st); break;
            case 1024: rc = launch_fix_t<1024>(ctx, *pass, st); break;
            case 2048: rc = launch_fix_t<2048>(ctx, *pass, st); break;
            default: return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no re-quantisation fix-up for width %d", n_in);
        }
        if (rc) return rc;
    }
    return B200MOE_OK;
}

// experts on activations xe [T][n_in] (fp32), routing already grouped in the plan
// y_direct != null: the per-row results of `down` go there ([rows][n_in]) and the weighted combine is left to the caller
// x_src != null: the activations are still fp32 (rows x_src_stride floats apart, indexed like xq's rows) and xq is only room for
// their quantised form: the engine that runs gate/up quantises them on its way in
int experts_impl(b200moe_ctx * ctx, const b200moe_layer * l, ActQuant xq, const int32_t * ids, const float * wts, int T, float * out,
                 const b200moe_observe * ob, cudaStream_t st, float * y_direct = nullptr, const float * x_src = nullptr, int64_t x_src_stride = 0) {
    Plan & p = ctx->plan;
    float * const y = y_direct ? y_direct : p.y;
    const int n_in = l->n_latent ? l->n_latent : l->n_embd;
    const int k = l->n_expert_used, rows = T * k;
    const int nt = tokens_per_pass(rows, l->n_expert);
    int rc;
    // Which engine runs which matmul (b200moe_set_expert_path documents the paths).
    //   integer kernels   reproduce the reference's fp32 summation order: bit-identical to the CPU path; cost grows with the rows an
    //                     expert receives
    //   FP4 tensor cores  (tcgen05 kind::mxf4nvf4, expert_gemm_fp4.cuh): NVFP4 rows as they lie in HBM, activations as exact digit
    //                     planes, 14 routed rows per pass over an expert; error = fp32 accumulation only (~5e-6 of RMS on `hidden`)
    //   f16 tensor cores  (tcgen05 kind::f16, expert_gemm.cuh): weights dequantised to fp16, activations as fp16 hi + lo, up to 128
    //                     routed rows per pass (~1.4e-4 of RMS on `hidden`): the prefill engine
    // After `down` nothing is re-quantised, so a tensor-core `down` only adds its own ~1e-5 to the output.  A tensor-core gate/up
    // moves a few values of `hidden` across int8 rounding boundaries of the reference's re-quantisation; the exact fix-up
    // (requant_fixup.cuh) removes those flips where the bar needs it: beyond 4096 routed rows on the f16 engine, and on latent
    // layers, which re-quantise once more after `down`.
    const bool can_mma = mma_supported(l->wtype, n_in, l->n_ff) && mma_supported(l->wtype, l->n_ff, n_in);
    const bool can_fp4 = fp4_supported(l->wtype, n_in, l->n_ff);
    const int path = ctx->expert_path;
    const bool latent = l->n_latent > 0;
    const bool few_rows = rows < 24 * l->n_expert;          // batched decode: on average fewer than 24 rows per expert
    bool fp4_gu = false, fp4_down = false, mma_gu = false, mma_down = false, fixup = false;
    switch (path) {
        case 0:
            if (rows <= 16) break;                           // one or two tokens: the small integer kernel, bit-identical
            if (can_fp4 && few_rows) { fp4_gu = fp4_down = true; fixup = latent; }
            else if (can_mma && rows >= 2 * l->n_expert) { mma_gu = true; mma_down = !latent; fixup = rows > 4096 || latent; }
            break;
        case 1: break;
        case 2: mma_gu = mma_down = can_mma; break;
        case 3: mma_down = can_mma; break;
        case 4: mma_gu = mma_down = fixup = can_mma; break;
        case 5: mma_gu = fixup = can_mma; break;
        case 6: fp4_gu = fp4_down = true; break;
        case 7: fp4_gu = fixup = true; break;
        case 8: fp4_gu = fp4_down = fixup = true; break;
    }
    if ((fp4_gu || fp4_down) && !can_fp4)
        return fail(ctx, B200MOE_ERR_UNSUPPORTED, "the FP4 tensor-core path needs NVFP4 experts, n_ff a multiple of 128 and n_in a multiple of 256");
    const bool small_tiles = few_rows;
    auto mp = [&](const void * w0, const void * w1, const float * s0, const float * s1, float * out, int n_out, int m_k) {
        MmaParams m{};
        m.w0 = static_cast<const uint8_t *>(w0); m.w1 = static_cast<const uint8_t *>(w1); m.scale0 = s0; m.scale1 = s1;
        m.act = p.afp16; m.act_lo = p.afp16 + (size_t) rows * m_k; m.offsets = p.groups.offsets; m.perm = p.groups.perm;
        m.active = p.groups.active; m.meta = p.groups.meta; m.out = out; m.n_out = n_out; m.n_as = l->n_expert; m.err = ctx->d_err;
        return m;
    };
    // Few rows per expert: `down` runs with tokens on the M side (256 weight rows per instruction, a quarter of the MMAs);
    // gate+up stays with weights on the M side, where the per-stage dequantisation work is the same and the kernel was
    // measured faster (167 us against 182 us at 64 tokens of configuration 2: there the tokens-on-M form is bound by
    // shared-memory traffic, twice the operand tile per stage).
    const bool tm_gu = false, tm_down = small_tiles && n_in % 256 == 0;
    if (x_src && !fp4_gu && (rc = launch_quantize<float>(ctx, x_src, x_src_stride, xq, T, n_in, l->wtype, st))) return rc;
    if (fp4_gu) {
        if (x_src) rc = launch_act_planes(ctx, ActQuant{}, x_src, p.ids, rows, n_in, k, 1, l->n_expert, st, fixup ? xq : ActQuant{}, x_src_stride);
        else rc = launch_act_planes(ctx, xq, nullptr, p.ids, rows, n_in, k, 1, l->n_expert, st);
        if (rc) return rc;
        if ((rc = launch_gemm_fp4<true>(ctx, n_in, fp4_params(ctx, l->gate_scale, l->up_scale, p.hid, l->n_ff, l->n_expert), l->gate, l->up, reinterpret_cast<const uint8_t *>(p.afp16), rows, st))) return rc;
    } else if (mma_gu) {
        if ((rc = launch_sorted_act(ctx, xq, rows, n_in, k, 1, tm_gu, st))) return rc;
        const MmaParams m = mp(l->gate, l->up, l->gate_scale, l->up_scale, p.hid, l->n_ff, n_in);
        if ((rc = tm_gu ? launch_gemm_tm<true>(ctx, n_in, m, rows, st) : launch_gemm<true>(ctx, n_in, m, rows, small_tiles, st))) return rc;
    } else {
        GemvParams gu = gemv_params(ctx, l->gate, l->up, l->gate_scale, l->up_scale, xq, p.hid, l->n_ff, k, 1, l->n_expert);
        if ((rc = launch_gemv<true>(ctx, l->wtype, n_in, gu, nt, st))) return rc;
    }
    if (fixup && (rc = launch_requant_fixup(ctx, l, xq, rows, n_in, k, fp4_gu, st))) return rc;
    // the integer down kernel quantises `hidden` itself while staging it (NVFP4 / Q8_0); otherwise a separate pass
    const bool fused_quant = !mma_down && !fp4_down && l->wtype == TYPE_NVFP4;
    if (!fused_quant && !fp4_down && (rc = launch_quantize<float>(ctx, p.hid, l->n_ff, p.hq, rows, l->n_ff, l->wtype, st))) return rc;
    if (fp4_down) {
        if ((rc = launch_act_planes(ctx, p.hq, p.hid, p.ids, rows, l->n_ff, k, k, l->n_expert, st))) return rc;   // quantises `hidden` itself
        if ((rc = launch_gemm_fp4<false>(ctx, l->n_ff, fp4_params(ctx, l->down_scale, nullptr, y, n_in, l->n_expert), l->down, nullptr, reinterpret_cast<const uint8_t *>(p.afp16), rows, st))) return rc;
    } else if (mma_down) {
        if ((rc = launch_sorted_act(ctx, p.hq, rows, l->n_ff, k, k, tm_down, st))) return rc;
        const MmaParams m = mp(l->down, nullptr, l->down_scale, nullptr, y, n_in, l->n_ff);
        if ((rc = tm_down ? launch_gemm_tm<false>(ctx, l->n_ff, m, rows, st) : launch_gemm<false>(ctx, l->n_ff, m, rows, small_tiles, st))) return rc;
    } else {
        GemvParams dn = gemv_params(ctx, l->down, nullptr, l->down_scale, nullptr, p.hq, y, n_in, k, k, l->n_expert);
        if (fused_quant) dn.act_f32 = p.hid;
        if ((rc = launch_gemv<false>(ctx, l->wtype, l->n_ff, dn, nt, st))) return rc;
    }
    if (!y_direct) {
        dim3 grid((n_in / 4 + 255) / 256, T);
        launch_k(ctx, combine_kernel, grid, dim3(256), 0, st, y, wts, out, n_in, k, T);
        if ((rc = check_launch(ctx, "combine"))) return rc;
    }
    if (ob && ob->ffn_moe_hidden)
        CUDA_TRY(ctx, cudaMemcpyAsync(ob->ffn_moe_hidden, p.hid, sizeof(float) * (size_t) rows * l->n_ff, cudaMemcpyDeviceToDevice, st));
    if (ob && ob->ffn_moe_down)
        CUDA_TRY(ctx, cudaMemcpyAsync(ob->ffn_moe_down, y, sizeof(float) * (size_t) rows * n_in, cudaMemcpyDeviceToDevice, st));
    (void) ids;
    return B200MOE_OK;
}

void account(b200moe_ctx * ctx, const b200moe_layer * l, int T) {
    ctx->counters.tokens += T;
    ctx->counters.kernel_launches = ctx->launches;
}

// The layer's shared expert and its sigmoid gate, added to the routed sum in `out` (forward.cpp:312-314).  Runs after the
// routed experts: the dense products borrow the plan's grouping buffers.
template <typename XT>
int shared_expert_impl(b200moe_ctx * ctx, const b200moe_layer * l, const XT * x, int T, float * out, const b200moe_observe * ob, cudaStream_t st) {
    Plan & p = ctx->plan;
    const int H = l->n_embd, Is = l->n_ff_shexp;
    int rc;
    const float * xf32;
    if (std::is_same<XT, float>::value) {
        xf32 = reinterpret_cast<const float *>(x);
    } else {
        const size_t n = (size_t) T * H;
        bf16_to_f32_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16 *>(x), p.xf, n);
        if ((rc = check_launch(ctx, "bf16_to_f32"))) return rc;
        xf32 = p.xf;
    }
    // logit of the gate: the reference's F32 dot product, lane chains as in the router
    constexpr int TT = 4;
    const int64_t warps = (T + TT - 1) / TT;
    router_logits_kernel<TT, float><<<(unsigned) ((warps * 32 + 255) / 256), 256, 0, st>>>(l->gate_inp_shexp, nullptr, xf32, p.sh_gate, H, 1, T, nullptr, 0);
    if ((rc = check_launch(ctx, "shexp_gate_logit"))) return rc;
    if ((rc = dense_matvec(ctx, l->wtype, l->gate_shexp, nullptr, xf32, p.xq, H, Is, T, p.sh_a, st, false, l->up_shexp, p.sh_b))) return rc;
    if ((rc = dense_matvec(ctx, l->wtype, l->down_shexp, nullptr, p.sh_a, p.shq, Is, H, T, p.sh_out, st))) return rc;
    dim3 grid((H + 255) / 256, T);
    shexp_add_kernel<<<grid, 256, 0, st>>>(out, p.sh_out, p.sh_gate, H, T, ob ? ob->ffn_shexp_gated : nullptr);
    return check_launch(ctx, "shexp_add");
}

template <typename XT>
int layer_impl(b200moe_ctx * ctx, const b200moe_layer * l, const XT * x, int T, float * out, const b200moe_observe * ob, cudaStream_t st) {
    Plan & p = ctx->plan;
    const int k = l->n_expert_used;
    int rc;
    const bool fused_front = !l->n_latent && T <= 128;  // decode-sized batches: 2 launches instead of 4
    if (fused_front) {
        if ((rc = launch_front<XT>(ctx, l, x, T, st))) return rc;
        float * probs = (ob && ob->ffn_moe_probs) ? ob->ffn_moe_probs : nullptr;
        if (T <= 32) {   // one warp per token fits one block: selection and grouping in a single launch
            if ((rc = launch_select_group(ctx, l, T, probs, st))) return rc;
        } else {
            if ((rc = launch_select(ctx, l, T, p.ids, p.wts, probs, true, st))) return rc;
            if ((rc = launch_group(ctx, p.ids, l->n_expert, T * k, st))) return rc;
        }
        if (ob && ob->ffn_moe_logits)
            CUDA_TRY(ctx, cudaMemcpyAsync(ob->ffn_moe_logits, p.logits, sizeof(float) * (size_t) T * l->n_expert, cudaMemcpyDeviceToDevice, st));
    } else {
        if ((rc = route_impl<XT>(ctx, l, x, T, p.ids, p.wts, ob, true, st))) return rc;
        if (!l->n_latent && (rc = launch_group(ctx, p.ids, l->n_expert, T * k, st))) return rc;
    }
    if (ob && ob->ffn_moe_topk) CUDA_TRY(ctx, cudaMemcpyAsync(ob->ffn_moe_topk, p.ids, sizeof(int32_t) * (size_t) T * k, cudaMemcpyDeviceToDevice, st));
    if (ob && ob->ffn_moe_weights_norm)
        CUDA_TRY(ctx, cudaMemcpyAsync(ob->ffn_moe_weights_norm, p.wts, sizeof(float) * (size_t) T * k, cudaMemcpyDeviceToDevice, st));

    if (!l->n_latent) {
        if (!fused_front && (rc = launch_quantize<XT>(ctx, x, l->n_embd, p.xq, T, l->n_embd, l->wtype, st))) return rc;
        rc = experts_impl(ctx, l, p.xq, p.ids, p.wts, T, out, ob, st);
        if (!rc && l->gate_shexp) rc = shared_expert_impl<XT>(ctx, l, x, T, out, ob, st);
        account(ctx, l, T);
        return rc;
    }
    // latent: routing was grouped into the plan's Groups, but the dense projections reuse the same Groups
    // buffers, so run the down-projection first and regroup afterwards.
    const float * xf32;
    if (std::is_same<XT, float>::value) {
        xf32 = reinterpret_cast<const float *>(x);
    } else {
        const size_t n = (size_t) T * l->n_embd;
        bf16_to_f32_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16 *>(x), p.xf, n);
        if ((rc = check_launch(ctx, "bf16_to_f32"))) return rc;
        xf32 = p.xf;
    }
    // the latent row is re-quantised for the experts: keep its quantised form the reference's (exact fix-up behind the FP4 engine)
    if ((rc = dense_matvec(ctx, l->wtype, l->lat_down, l->lat_down_scale, xf32, p.xq, l->n_embd, l->n_latent, T, p.xl, st, true))) return rc;
    // regroup the expert routing
    CUDA_TRY(ctx, cudaMemsetAsync(p.groups.counts, 0, sizeof(int) * l->n_expert, st));
    count_ids_kernel<<<(T * k + 255) / 256, 256, 0, st>>>(p.ids, k, k, T, l->n_expert, p.groups.perm, p.groups.counts, p.groups.pos, ctx->d_err);
    if ((rc = check_launch(ctx, "count_ids"))) return rc;
    if ((rc = launch_group(ctx, p.ids, l->n_expert, T * k, st))) return rc;
    if ((rc = experts_impl(ctx, l, p.xlq, p.ids, p.wts, T, p.moe, ob, st, nullptr, p.xl, l->n_latent))) return rc;
    rc = dense_matvec(ctx, l->wtype, l->lat_up, l->lat_up_scale, p.moe, p.moq, l->n_latent, l->n_embd, T, out, st);
    account(ctx, l, T);
    return rc;
}

}  // namespace

// ============================================================================================ C ABI

extern "C" {

const char * b200moe_status_string(int s) {
    switch (s) {
        case B200MOE_OK: return "ok";
        case B200MOE_ERR_INVALID_ARG: return "invalid argument";
        case B200MOE_ERR_UNSUPPORTED: return "unsupported type or shape";
        case B200MOE_ERR_ALLOC: return "device allocation failed";
        case B200MOE_ERR_CUDA: return "CUDA error";
        case B200MOE_ERR_DEVICE_CHECK: return "device-side check failed";
        case B200MOE_ERR_NO_DEVICE: return "no CUDA device";
        default: return "unknown status";
    }
}

int b200moe_create(int device, b200moe_ctx ** out) {
    if (!out) return B200MOE_ERR_INVALID_ARG;
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return B200MOE_ERR_NO_DEVICE; }
    if (device < 0 || device >= n) return B200MOE_ERR_INVALID_ARG;
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return B200MOE_ERR_CUDA; }
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); return B200MOE_ERR_CUDA; }
    if (prop.major != 10) return B200MOE_ERR_UNSUPPORTED;  // kernels are built for sm_100a only
    auto * ctx = new b200moe_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(&ctx->d_err, 16) != cudaSuccess || cudaMemset(ctx->d_err, 0, 16) != cudaSuccess ||
        cudaMallocHost(&ctx->h_err, 16) != cudaSuccess) {
        cudaGetLastError();
        delete ctx;
        return B200MOE_ERR_ALLOC;
    }
    memset(ctx->h_err, 0, 16);
    *out = ctx;
    return B200MOE_OK;
}

void b200moe_destroy(b200moe_ctx * ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->scratch.base) cudaFree(ctx->scratch.base);
    if (ctx->d_err) cudaFree(ctx->d_err);
    if (ctx->h_err) cudaFreeHost(ctx->h_err);
    delete ctx;
}

const char * b200moe_last_error(const b200moe_ctx * ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }

int b200moe_device_memory(int device, size_t * free_bytes, size_t * total_bytes) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return B200MOE_ERR_NO_DEVICE; }
    if (device < 0 || device >= n || !free_bytes || !total_bytes) return B200MOE_ERR_INVALID_ARG;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device);
    cudaError_t e = cudaMemGetInfo(free_bytes, total_bytes);
    cudaSetDevice(prev);
    return e == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int b200moe_get_counters(const b200moe_ctx * ctx, b200moe_counters * out) {
    if (!ctx || !out) return B200MOE_ERR_INVALID_ARG;
    *out = ctx->counters;
    out->kernel_launches = ctx->launches;
    return B200MOE_OK;
}

int b200moe_set_expert_path(b200moe_ctx * ctx, int path) {
    if (!ctx || path < 0 || path > 8) return B200MOE_ERR_INVALID_ARG;
    ctx->expert_path = path;
    return B200MOE_OK;
}

int b200moe_set_launch_overlap(b200moe_ctx * ctx, int enable) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    ctx->overlap = enable != 0;
    return B200MOE_OK;
}

int b200moe_enable_kernel_timing(b200moe_ctx * ctx, int enable) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    ctx->timing = enable != 0;
    return B200MOE_OK;
}

int b200moe_kernel_times(b200moe_ctx * ctx, int64_t launches[3], double total_ms[3]) {
    if (!ctx || !launches || !total_ms) return B200MOE_ERR_INVALID_ARG;
    launches[0] = launches[1] = launches[2] = 0;
    total_ms[0] = total_ms[1] = total_ms[2] = 0.0;
    for (auto & t : ctx->timed) {
        float ms = 0.0f;
        CUDA_TRY(ctx, cudaEventSynchronize(t.end));
        CUDA_TRY(ctx, cudaEventElapsedTime(&ms, t.beg, t.end));
        launches[t.kind] += 1;
        total_ms[t.kind] += ms;
        cudaEventDestroy(t.beg);
        cudaEventDestroy(t.end);
    }
    ctx->timed.clear();
    return B200MOE_OK;
}

int b200moe_synchronize(b200moe_ctx * ctx, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    return read_device_error(ctx, static_cast<cudaStream_t>(stream));
}

int b200moe_reserve(b200moe_ctx * ctx, const b200moe_layer * l, int32_t max_tokens) {
    int rc = validate_layer(ctx, l);
    if (rc) return rc;
    if (max_tokens <= 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "max_tokens must be positive");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return ensure_plan(ctx, l->n_embd, l->n_latent ? l->n_latent : l->n_embd, l->n_expert, l->n_expert_used, l->n_ff, l->wtype, max_tokens, l->n_ff_shexp);
}

int b200moe_mul_mat_id_width_ok(int type, int64_t ne00) { return gemv_supported(type, ne00) ? 1 : 0; }

int64_t b200moe_row_size(int type, int64_t n) {
    if (n < 0) return -1;
    if (type == TYPE_NVFP4 && n % 64) return -1;
    if (type == TYPE_Q3_K && n % 256) return -1;
    return weight_row_bytes(type, n);
}

// ---- host-side format helpers (ggml-quants.c:337-348, 384-417 for the quantiser; :589-612, :1305-1353 dequantisers)
static const int8_t k_fp4_values[16] = { 0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12 };

static uint8_t fp32_to_ue4m3(float x) {
    if (!(x > 0.0f)) return 0;
    if (x > 448.0f) x = 448.0f;
    uint32_t bits;
    memcpy(&bits, &x, 4);
    const int fexp = (int) ((bits >> 23) & 0xff) - 127, fman = (bits >> 20) & 7;
    int ue = fexp + 7;
    if (ue <= 0) {
        int man = (int) (x * 512.0f + 0.5f);
        if (man > 7) man = 7;
        return man < 1 ? 0 : (uint8_t) man;
    }
    if (ue >= 15) return 0x7e;
    int um = fman + ((bits >> 19) & 1);
    if (um > 7) { um = 0; if (++ue >= 15) return 0x7e; }
    return (uint8_t) ((ue << 3) | um);
}

static void quantize_row_nvfp4(const float * x, uint8_t * y, int64_t k) {
    for (int64_t b = 0; b < k / 64; ++b) {
        uint8_t * blk = y + b * 36;
        for (int s = 0; s < 4; ++s) {
            const float * xb = x + b * 64 + s * 16;
            float amax = 0.0f;
            for (int j = 0; j < 16; ++j) amax = std::max(amax, std::fabs(xb[j]));
            const uint8_t ue = fp32_to_ue4m3(amax / 6.0f);
            blk[s] = ue;
            const float d = ue4m3_half_to_f32(ue);
            auto best = [&](float v) {
                int bi = 0;
                float be = std::fabs(k_fp4_values[0] * d - v);
                for (int i = 1; i < 16; ++i) {
                    const float err = std::fabs(k_fp4_values[i] * d - v);
                    if (err < be) { bi = i; be = err; }
                }
                return (uint8_t) bi;
            };
            for (int j = 0; j < 8; ++j) blk[4 + s * 8 + j] = (uint8_t) (best(xb[j]) | (best(xb[8 + j]) << 4));
        }
    }
}

int b200moe_quantize_nvfp4_host(const float * src, void * dst, int64_t nrows, int64_t n_per_row) {
    if (!src || !dst || nrows < 0 || n_per_row <= 0 || n_per_row % 64) return B200MOE_ERR_INVALID_ARG;
    const int64_t rs = n_per_row / 64 * 36;
    const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    const int nthreads = (int) std::min<int64_t>(hw, std::max<int64_t>(1, nrows / 64));
    std::vector<std::thread> th;
    for (int t = 0; t < nthreads; ++t)
        th.emplace_back([=] {
            for (int64_t r = nrows * t / nthreads; r < nrows * (t + 1) / nthreads; ++r)
                quantize_row_nvfp4(src + r * n_per_row, static_cast<uint8_t *>(dst) + r * rs, n_per_row);
        });
    for (auto & t : th) t.join();
    return B200MOE_OK;
}

int64_t b200moe_expert_blob_bytes_nvfp4(int32_t n_embd, int32_t n_ff) {
    if (n_embd <= 0 || n_ff <= 0 || n_embd % 64 || n_ff % 64) return -1;
    const int64_t gu_row = (int64_t) n_embd / 64 * NVFP4_BLOCK_BYTES, d_row = (int64_t) n_ff / 64 * NVFP4_BLOCK_BYTES;
    return 2 * n_ff * gu_row + n_embd * d_row + 16;
}

int b200moe_unpack_expert_blobs_nvfp4(const void * blobs, int64_t blob_stride, int32_t n_expert, int32_t n_embd, int32_t n_ff, void * gate, void * up,
                                      void * down, float * gate_scale, float * up_scale, float * down_scale, int to_device, void * stream) {
    const int64_t bytes = b200moe_expert_blob_bytes_nvfp4(n_embd, n_ff);
    if (bytes < 0 || n_expert <= 0 || !blobs || !gate || !up || !down || !gate_scale || !up_scale || !down_scale || blob_stride < bytes)
        return B200MOE_ERR_INVALID_ARG;
    const size_t gu = (size_t) n_ff * ((size_t) n_embd / 64 * NVFP4_BLOCK_BYTES), dn = (size_t) n_embd * ((size_t) n_ff / 64 * NVFP4_BLOCK_BYTES);
    std::vector<float> sg(n_expert), su(n_expert), sd(n_expert);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int e = 0; e < n_expert; ++e) {
        const uint8_t * b = static_cast<const uint8_t *>(blobs) + (size_t) e * blob_stride;
        float tail[4];
        memcpy(tail, b + 2 * gu + dn, sizeof tail);
        sg[e] = tail[0]; su[e] = tail[1]; sd[e] = tail[2];
        uint8_t * dg = static_cast<uint8_t *>(gate) + (size_t) e * gu, * du = static_cast<uint8_t *>(up) + (size_t) e * gu,
                * dd = static_cast<uint8_t *>(down) + (size_t) e * dn;
        if (!to_device) {
            memcpy(dg, b, gu); memcpy(du, b + gu, gu); memcpy(dd, b + 2 * gu, dn);
        } else if (cudaMemcpyAsync(dg, b, gu, cudaMemcpyHostToDevice, st) != cudaSuccess ||
                   cudaMemcpyAsync(du, b + gu, gu, cudaMemcpyHostToDevice, st) != cudaSuccess ||
                   cudaMemcpyAsync(dd, b + 2 * gu, dn, cudaMemcpyHostToDevice, st) != cudaSuccess) {
            cudaGetLastError();
            return B200MOE_ERR_CUDA;
        }
    }
    const size_t sb = sizeof(float) * (size_t) n_expert;
    if (!to_device) {
        memcpy(gate_scale, sg.data(), sb); memcpy(up_scale, su.data(), sb); memcpy(down_scale, sd.data(), sb);
        return B200MOE_OK;
    }
    if (cudaMemcpyAsync(gate_scale, sg.data(), sb, cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaMemcpyAsync(up_scale, su.data(), sb, cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaMemcpyAsync(down_scale, sd.data(), sb, cudaMemcpyHostToDevice, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return B200MOE_ERR_CUDA;
    }
    return B200MOE_OK;
}

int b200moe_dequantize_host(int type, const void * src, float * dst, int64_t nrows, int64_t n_per_row) {
    if (!src || !dst || nrows < 0 || n_per_row <= 0) return B200MOE_ERR_INVALID_ARG;
    const uint8_t * s = static_cast<const uint8_t *>(src);
    if (type == TYPE_NVFP4) {
        if (n_per_row % 64) return B200MOE_ERR_INVALID_ARG;
        for (int64_t b = 0; b < nrows * n_per_row / 64; ++b) {
            const uint8_t * blk = s + b * 36;
            for (int sb = 0; sb < 4; ++sb) {
                const float d = ue4m3_half_to_f32(blk[sb]);
                for (int j = 0; j < 8; ++j) {
                    dst[b * 64 + sb * 16 + j] = k_fp4_values[blk[4 + sb * 8 + j] & 15] * d;
                    dst[b * 64 + sb * 16 + j + 8] = k_fp4_values[blk[4 + sb * 8 + j] >> 4] * d;
                }
            }
        }
        return B200MOE_OK;
    }
    if (type == TYPE_Q3_K) {
        if (n_per_row % 256) return B200MOE_ERR_INVALID_ARG;
        for (int64_t b = 0; b < nrows * n_per_row / 256; ++b) {
            const uint8_t * blk = s + b * 110;
            uint32_t sw[3], sc[4];
            memcpy(sw, blk + 96, 12);
            q3k_unpack_scales(sw[0], sw[1], sw[2], sc);
            uint16_t hb;
            memcpy(&hb, blk + 108, 2);
            // half -> float on the host
            const uint32_t sign = (uint32_t) (hb & 0x8000) << 16, ex = (hb >> 10) & 31, mn = hb & 1023;
            float d;
            if (ex == 0) d = std::ldexp((float) mn, -24);
            else if (ex == 31) d = INFINITY;
            else { uint32_t u = ((ex + 112) << 23) | (mn << 13); memcpy(&d, &u, 4); }
            if (sign) d = -d;
            for (int idx = 0; idx < 256; ++idx) {
                const int half = idx >> 7, shift = (idx >> 5) & 3, l = idx & 31;
                const int lo = (blk[32 + 32 * half + l] >> (2 * shift)) & 3;
                const int hbit = (blk[l] >> (4 * half + shift)) & 1;
                const float dl = d * (float) q3k_scale_at(sc, idx >> 4);
                dst[b * 256 + idx] = dl * (float) (lo - (hbit ? 0 : 4));
            }
        }
        return B200MOE_OK;
    }
    return B200MOE_ERR_UNSUPPORTED;
}

// ---- compute

int b200moe_route(b200moe_ctx * ctx, const b200moe_layer * l, const void * x, int x_type, int32_t T, int32_t * ids, float * weights,
                  const b200moe_observe * ob, void * stream) {
    int rc = validate_layer(ctx, l, true, false);
    if (rc) return rc;
    if (T == 0) return B200MOE_OK;
    if (!x || !ids || !weights || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or negative token count");
    if (x_type != TYPE_F32 && x_type != TYPE_BF16) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "activations must be F32 or BF16");
    if (T == 0) return B200MOE_OK;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    layer_overlap(ctx, (int64_t) T * l->n_expert_used, l->n_expert);
    if ((rc = ensure_plan(ctx, l->n_embd, l->n_latent ? l->n_latent : l->n_embd, l->n_expert, l->n_expert_used, l->n_ff, l->wtype, T))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_type == TYPE_F32) return route_impl<float>(ctx, l, static_cast<const float *>(x), T, ids, weights, ob, false, st);
    return route_impl<__nv_bfloat16>(ctx, l, static_cast<const __nv_bfloat16 *>(x), T, ids, weights, ob, false, st);
}

int b200moe_mul_mat_id(b200moe_ctx * ctx, int wtype, const void * as, int64_t ne00, int64_t ne01, int64_t n_as, const float * b, int64_t ne11,
                       const int32_t * ids, int64_t n_ids, int64_t ids_nb1, int64_t T, float * dst, void * stream) {
    if (ctx) ctx->overlap_now = false;
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (T == 0) return B200MOE_OK;
    if (!as || !b || !ids || !dst) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer");
    if (ne00 <= 0 || ne01 <= 0 || n_as <= 0 || ne11 <= 0 || n_ids <= 0 || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "non-positive size");
    if (n_ids > 32) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "more than 32 ids per token");
    if (n_ids % ne11) return fail(ctx, B200MOE_ERR_INVALID_ARG, "ids->ne[0] must be a multiple of b->ne[1]");  // ggml.c:3406
    if (ids_nb1 % 4 || ids_nb1 < n_ids * 4) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad ids row stride");
    if ((uintptr_t) as & 15) return fail(ctx, B200MOE_ERR_INVALID_ARG, "expert tensor must be 16-byte aligned");
    if (!gemv_supported(wtype, ne00) || ne01 % 8 || n_as > 1024) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no kernel for type %d, K=%lld", wtype, (long long) ne00);
    if (T == 0) return B200MOE_OK;
    if (T * n_ids > (1 << 30)) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "too many routed rows");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // plan: treat as a layer with n_embd = n_in = ne00, rows = T * max(n_ids, ne11)
    const int k = (int) n_ids;
    int rc = ensure_plan(ctx, (int) ne00, (int) ne00, (int) std::max<int64_t>(n_as, 8), k, (int) ne00, wtype, (int) T);
    if (rc) return rc;
    Plan & p = ctx->plan;
    const int rows = (int) (T * n_ids);
    // activations: T*ne11 rows of ne00; plan.hq holds T*k rows of width n_ff (= ne00 here), ne11 <= k
    if ((rc = launch_quantize<float>(ctx, b, ne00, p.hq, (int) (T * ne11), (int) ne00, wtype, st))) return rc;
    CUDA_TRY(ctx, cudaMemsetAsync(p.groups.counts, 0, sizeof(int) * n_as, st));
    count_ids_kernel<<<(rows + 255) / 256, 256, 0, st>>>(ids, ids_nb1 / 4, (int) n_ids, (int) T, (int) n_as, p.ids, p.groups.counts, p.groups.pos, ctx->d_err);
    if ((rc = check_launch(ctx, "count_ids"))) return rc;
    if ((rc = launch_group(ctx, p.ids, (int) n_as, rows, st))) return rc;
    GemvParams g = gemv_params(ctx, as, nullptr, nullptr, nullptr, p.hq, dst, (int) ne01, (int) n_ids, (int) ne11, (int) n_as);
    return launch_gemv<false>(ctx, wtype, (int) ne00, g, tokens_per_pass(rows, (int) n_as), st);
}

int b200moe_mul_mat(b200moe_ctx * ctx, int wtype, const void * w, int64_t ne00, int64_t ne01, const float * x, int64_t T, const float * scale,
                    float * dst, void * stream) {
    if (ctx) ctx->overlap_now = false;
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (T == 0) return B200MOE_OK;
    if (!w || !x || !dst || ne00 <= 0 || ne01 <= 0 || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or non-positive size");
    if ((uintptr_t) w & 15) return fail(ctx, B200MOE_ERR_INVALID_ARG, "weight tensor must be 16-byte aligned");
    if (!gemv_supported(wtype, ne00) || ne01 % 8) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "no kernel for type %d, K=%lld", wtype, (long long) ne00);
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = ensure_plan(ctx, (int) ne00, (int) ne00, 8, 1, (int) ne00, wtype, (int) T);
    if (rc) return rc;
    return dense_matvec(ctx, wtype, w, scale, x, ctx->plan.xq, (int) ne00, (int) ne01, (int) T, dst, st);
}

// The two shared projections of a latent layer as calls of their own (the expert-parallel layer runs them on the token's rank).
int b200moe_latent_down(b200moe_ctx * ctx, const b200moe_layer * l, const void * x, int x_type, int32_t T, float * xl, void * stream) {
    int rc = validate_layer(ctx, l, false, false);
    if (rc) return rc;
    if (!l->n_latent || !l->lat_down) return fail(ctx, B200MOE_ERR_INVALID_ARG, "layer has no latent down-projection");
    if (T == 0) return B200MOE_OK;
    if (!x || !xl || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or negative token count");
    if (x_type != TYPE_F32 && x_type != TYPE_BF16) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "activations must be F32 or BF16");
    if ((uintptr_t) l->lat_down & 15) return fail(ctx, B200MOE_ERR_INVALID_ARG, "quantised tensors must be 16-byte aligned");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ctx->overlap_now = false;
    if ((rc = ensure_plan(ctx, l->n_embd, l->n_latent, l->n_expert, l->n_expert_used, l->n_ff, l->wtype, T))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Plan & p = ctx->plan;
    const float * xf32 = static_cast<const float *>(x);
    if (x_type == TYPE_BF16) {
        const size_t n = (size_t) T * l->n_embd;
        bf16_to_f32_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), p.xf, n);
        if ((rc = check_launch(ctx, "bf16_to_f32"))) return rc;
        xf32 = p.xf;
    }
    // the caller re-quantises the latent rows for the experts: their quantised form stays the reference's
    return dense_matvec(ctx, l->wtype, l->lat_down, l->lat_down_scale, xf32, p.xq, l->n_embd, l->n_latent, T, xl, st, true);
}

int b200moe_latent_up(b200moe_ctx * ctx, const b200moe_layer * l, const float * m, int32_t T, float * out, void * stream) {
    int rc = validate_layer(ctx, l, false, false);
    if (rc) return rc;
    if (!l->n_latent || !l->lat_up) return fail(ctx, B200MOE_ERR_INVALID_ARG, "layer has no latent up-projection");
    if (T == 0) return B200MOE_OK;
    if (!m || !out || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or negative token count");
    if ((uintptr_t) l->lat_up & 15) return fail(ctx, B200MOE_ERR_INVALID_ARG, "quantised tensors must be 16-byte aligned");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ctx->overlap_now = false;
    if ((rc = ensure_plan(ctx, l->n_embd, l->n_latent, l->n_expert, l->n_expert_used, l->n_ff, l->wtype, T))) return rc;
    return dense_matvec(ctx, l->wtype, l->lat_up, l->lat_up_scale, m, ctx->plan.moq, l->n_latent, l->n_embd, T, out, static_cast<cudaStream_t>(stream));
}

int b200moe_combine(b200moe_ctx * ctx, const float * y, const float * weights, float * out, int64_t n, int64_t k, int64_t T, void * stream) {
    if (ctx) ctx->overlap_now = false;
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (T == 0) return B200MOE_OK;
    if (!y || !weights || !out || n <= 0 || k <= 0 || T < 0 || n % 4) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer, non-positive size or width not a multiple of 4");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    dim3 grid((unsigned) ((n / 4 + 255) / 256), (unsigned) T);
    combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(y, weights, out, (int) n, (int) k, (int) T);
    return check_launch(ctx, "combine");
}

int b200moe_gather_rows(b200moe_ctx * ctx, const float * src, int64_t src_rows, const int32_t * idx, float * dst, int64_t n_rows, int64_t width,
                        void * stream) {
    if (ctx) ctx->overlap_now = false;
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (n_rows == 0) return B200MOE_OK;
    if (!src || !idx || !dst || n_rows < 0 || src_rows <= 0 || width <= 0 || width % 4) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer, bad size or width not a multiple of 4");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    dim3 grid((unsigned) ((width / 4 + 255) / 256), (unsigned) n_rows);
    gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const float4 *>(src), idx, reinterpret_cast<float4 *>(dst),
                                                                            (int) n_rows, (int) (width / 4), (int) src_rows);
    return check_launch(ctx, "gather_rows");
}

int b200moe_ffn(b200moe_ctx * ctx, const b200moe_layer * l, const void * x, int x_type, int32_t T, const int32_t * ids, const float * weights,
                float * out, const b200moe_observe * ob, void * stream) {
    int rc = validate_layer(ctx, l, false, true);
    if (rc) return rc;
    if (T == 0) return B200MOE_OK;
    if (!x || !ids || !weights || !out || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or negative token count");
    if (x_type != TYPE_F32 && x_type != TYPE_BF16) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "activations must be F32 or BF16");
    if (T == 0) return B200MOE_OK;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    layer_overlap(ctx, (int64_t) T * l->n_expert_used, l->n_expert);
    if ((rc = ensure_plan(ctx, l->n_embd, l->n_latent ? l->n_latent : l->n_embd, l->n_expert, l->n_expert_used, l->n_ff, l->wtype, T))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Plan & p = ctx->plan;
    const int n_in = l->n_latent ? l->n_latent : l->n_embd, k = l->n_expert_used;
    CUDA_TRY(ctx, cudaMemsetAsync(p.groups.counts, 0, sizeof(int) * l->n_expert, st));
    count_ids_kernel<<<(T * k + 255) / 256, 256, 0, st>>>(ids, k, k, T, l->n_expert, p.ids, p.groups.counts, p.groups.pos, ctx->d_err);
    if ((rc = check_launch(ctx, "count_ids"))) return rc;
    if ((rc = launch_group(ctx, p.ids, l->n_expert, T * k, st))) return rc;
    if (x_type == TYPE_F32) rc = launch_quantize<float>(ctx, static_cast<const float *>(x), n_in, p.xq, T, n_in, l->wtype, st);
    else rc = launch_quantize<__nv_bfloat16>(ctx, static_cast<const __nv_bfloat16 *>(x), n_in, p.xq, T, n_in, l->wtype, st);
    if (rc) return rc;
    rc = experts_impl(ctx, l, p.xq, p.ids, weights, T, out, ob, st);
    account(ctx, l, T);
    return rc;
}

int b200moe_layer_forward(b200moe_ctx * ctx, const b200moe_layer * l, const void * x, int x_type, int32_t T, float * out,
                          const b200moe_observe * ob, void * stream) {
    int rc = validate_layer(ctx, l);
    if (rc) return rc;
    if (T == 0) return B200MOE_OK;
    if (!x || !out || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or negative token count");
    if (x_type != TYPE_F32 && x_type != TYPE_BF16) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "activations must be F32 or BF16");
    if (T == 0) return B200MOE_OK;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    layer_overlap(ctx, (int64_t) T * l->n_expert_used, l->n_expert);
    if ((rc = b200moe_reserve(ctx, l, T))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_type == TYPE_F32) return layer_impl<float>(ctx, l, static_cast<const float *>(x), T, out, ob, st);
    return layer_impl<__nv_bfloat16>(ctx, l, static_cast<const __nv_bfloat16 *>(x), T, out, ob, st);
}

int b200moe_layer_forward_host(b200moe_ctx * ctx, const b200moe_layer * l, const void * x_host, int x_type, int32_t T, float * out_host,
                               int32_t * ids_host, float * weights_host, void * stream) {
    int rc = validate_layer(ctx, l);
    if (rc) return rc;
    if (T == 0) return B200MOE_OK;
    if (!x_host || !out_host || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or negative token count");
    if (x_type != TYPE_F32 && x_type != TYPE_BF16) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "activations must be F32 or BF16");
    if (T == 0) return B200MOE_OK;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    layer_overlap(ctx, (int64_t) T * l->n_expert_used, l->n_expert);
    if ((rc = b200moe_reserve(ctx, l, T))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Plan & p = ctx->plan;
    const size_t xbytes = (size_t) T * l->n_embd * (x_type == TYPE_F32 ? 4 : 2);
    CUDA_TRY(ctx, cudaMemcpyAsync(p.xin, x_host, xbytes, cudaMemcpyHostToDevice, st));
    if (x_type == TYPE_F32) rc = layer_impl<float>(ctx, l, static_cast<const float *>(p.xin), T, p.outb, nullptr, st);
    else rc = layer_impl<__nv_bfloat16>(ctx, l, static_cast<const __nv_bfloat16 *>(p.xin), T, p.outb, nullptr, st);
    if (rc) return rc;
    CUDA_TRY(ctx, cudaMemcpyAsync(out_host, p.outb, sizeof(float) * (size_t) T * l->n_embd, cudaMemcpyDeviceToHost, st));
    if (ids_host) CUDA_TRY(ctx, cudaMemcpyAsync(ids_host, p.ids, sizeof(int32_t) * (size_t) T * l->n_expert_used, cudaMemcpyDeviceToHost, st));
    if (weights_host) CUDA_TRY(ctx, cudaMemcpyAsync(weights_host, p.wts, sizeof(float) * (size_t) T * l->n_expert_used, cudaMemcpyDeviceToHost, st));
    return read_device_error(ctx, st);
}

// ---- expert-parallel exchange (expert_exchange.cuh) ---------------------------------------------------------------------

int64_t b200moe_ep_slot_bytes(int64_t width) { return width > 0 && width % 4 == 0 ? (width + EP_SLOT_EXTRA) * 4 : -1; }

int b200moe_ep_pack(b200moe_ctx * ctx, const float * rows, const int32_t * ids, int64_t T, int64_t k, int64_t width, int64_t n_ranks,
                    int64_t experts_per_rank, int64_t capacity, void * slots, int32_t * slot_of, int32_t * fill, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (!slots || !fill || T < 0 || k <= 0 || width <= 0 || width % 4 || n_ranks <= 0 || experts_per_rank <= 0 || capacity <= 0)
        return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or bad size");
    if (T > 0 && (!rows || !ids || !slot_of)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer");
    if (T * k > capacity * n_ranks || n_ranks * capacity > (1 << 30)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "capacity below the routed rows of this rank");
    if ((uintptr_t) rows & 15 || (uintptr_t) slots & 15) return fail(ctx, B200MOE_ERR_INVALID_ARG, "rows and slots must be 16-byte aligned");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int n_slots = (int) (n_ranks * capacity);
    ep_clear_kernel<<<(std::max<int>(n_slots, (int) n_ranks) + 255) / 256, 256, 0, st>>>(static_cast<float *>(slots), n_slots, (int) width + EP_SLOT_EXTRA,
                                                                                       (int) width, fill, (int) n_ranks);
    int rc = check_launch(ctx, "ep_clear");
    if (rc || T == 0) return rc;
    ep_pack_kernel<<<(unsigned) (T * k), 256, 0, st>>>(rows, ids, (int) (T * k), (int) k, (int) width, (int) n_ranks, (int) experts_per_rank, (int) capacity,
                                                      static_cast<float *>(slots), slot_of, fill, ctx->d_err);
    return check_launch(ctx, "ep_pack");
}

int b200moe_ep_expert_rows(b200moe_ctx * ctx, const b200moe_layer * l, const void * slots, int64_t n_slots, float * y, void * stream) {
    int rc = validate_layer(ctx, l, false, true);
    if (rc) return rc;
    if (l->n_latent) return fail(ctx, B200MOE_ERR_INVALID_ARG, "the owner's layer is the plain expert layer of the exchanged width");
    if (n_slots == 0) return B200MOE_OK;
    if (!slots || !y || n_slots < 0 || n_slots > (1 << 30)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or bad slot count");
    if ((uintptr_t) slots & 15) return fail(ctx, B200MOE_ERR_INVALID_ARG, "slots must be 16-byte aligned");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ctx->overlap_now = false;
    const int n_in = l->n_embd, R = (int) n_slots, slot_words = n_in + EP_SLOT_EXTRA;
    // one slot = one routed row of a one-slot layer
    if ((rc = ensure_plan(ctx, l->n_embd, n_in, l->n_expert, 1, l->n_ff, l->wtype, R))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Plan & p = ctx->plan;
    const float * rows = static_cast<const float *>(slots);
    const int32_t * ids = reinterpret_cast<const int32_t *>(rows + n_in);
    CUDA_TRY(ctx, cudaMemsetAsync(p.groups.counts, 0, sizeof(int) * l->n_expert, st));
    count_ids_kernel<<<(R + 255) / 256, 256, 0, st>>>(ids, slot_words, 1, R, l->n_expert, p.ids, p.groups.counts, p.groups.pos, ctx->d_err, 1);
    if ((rc = check_launch(ctx, "count_ids"))) return rc;
    if ((rc = launch_group(ctx, p.ids, l->n_expert, R, st, true))) return rc;
    // the slots' rows are quantised by whichever engine runs gate/up (empty slots hold garbage nobody reads)
    rc = experts_impl(ctx, l, p.xq, p.ids, nullptr, R, nullptr, nullptr, st, y, rows, slot_words);
    account(ctx, l, 0);
    return rc;
}

int b200moe_ep_combine(b200moe_ctx * ctx, const float * back, int64_t n_slots, const int32_t * slot_of, const float * weights, int64_t T, int64_t k,
                       int64_t width, float * out, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (T == 0) return B200MOE_OK;
    if (!back || !slot_of || !weights || !out || T < 0 || k <= 0 || width <= 0 || width % 4 || n_slots <= 0)
        return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer, bad size or width not a multiple of 4");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    dim3 grid((unsigned) ((width / 4 + 255) / 256), (unsigned) T);
    ep_combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(back, slot_of, weights, out, (int) width, (int) k, (int) T, (int) n_slots);
    return check_launch(ctx, "ep_combine");
}

// ---- single graph operators (graph_ops.cuh) ------------------------------------------------------------------------------

namespace {

bool to_view(const b200moe_tensor * t, TensorView & v, int64_t * count) {
    if (!t || !t->data) return false;
    v.data = static_cast<char *>(t->data);
    int64_t n = 1;
    for (int i = 0; i < 4; ++i) {
        if (t->ne[i] <= 0 || t->nb[i] < 0) return false;
        v.ne[i] = t->ne[i];
        v.nb[i] = t->nb[i];
        n *= t->ne[i];
    }
    if (t->nb[0] % 4) return false;
    if (count) *count = n;
    return n < ((int64_t) 1 << 40);
}

bool broadcastable(const TensorView & small, const TensorView & big) {
    for (int i = 0; i < 4; ++i) if (big.ne[i] % small.ne[i]) return false;
    return true;
}

int grid_for(int64_t n) { return (int) std::min<int64_t>((n + 255) / 256, 148 * 32); }

}  // namespace

int b200moe_op_binary(b200moe_ctx * ctx, int op, const b200moe_tensor * a, const b200moe_tensor * b, const b200moe_tensor * dst, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    TensorView va, vb, vd;
    int64_t n = 0;
    if (op < 0 || op > 2 || !to_view(a, va, nullptr) || !to_view(b, vb, nullptr) || !to_view(dst, vd, &n)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad operator or tensor");
    for (int i = 0; i < 4; ++i) if (va.ne[i] != vd.ne[i]) return fail(ctx, B200MOE_ERR_INVALID_ARG, "dst must have the shape of the first operand");
    if (!broadcastable(vb, vd)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "second operand does not repeat over the first");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    op_binary_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(op, va, vb, vd);
    return check_launch(ctx, "op_binary");
}

int b200moe_op_unary(b200moe_ctx * ctx, int op, const b200moe_tensor * a, const b200moe_tensor * dst, float p0, float p1, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    TensorView va, vd;
    int64_t n = 0;
    if (op < 0 || op > 2 || !to_view(a, va, nullptr) || !to_view(dst, vd, &n)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad operator or tensor");
    for (int i = 0; i < 4; ++i) if (va.ne[i] != vd.ne[i]) return fail(ctx, B200MOE_ERR_INVALID_ARG, "shapes differ");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    op_unary_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(op, va, vd, p0, p1);
    return check_launch(ctx, "op_unary");
}

int b200moe_op_repeat(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    TensorView va, vd;
    int64_t n = 0;
    if (!to_view(a, va, nullptr) || !to_view(dst, vd, &n) || !broadcastable(va, vd)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad tensor or shapes do not repeat");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    op_repeat_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(va, vd);
    return check_launch(ctx, "op_repeat");
}

int b200moe_op_get_rows(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * ids, const b200moe_tensor * dst, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    TensorView va, vi, vd;
    int64_t rows = 0;
    if (!to_view(a, va, nullptr) || !to_view(ids, vi, &rows) || !to_view(dst, vd, nullptr)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad tensor");
    if (vi.ne[3] != 1 || vd.ne[0] != va.ne[0] || vd.ne[1] != vi.ne[0] || vd.ne[2] != vi.ne[1] || vd.ne[3] != vi.ne[2] ||
        (va.ne[2] != vi.ne[1] && va.ne[2] != 1) || (va.ne[3] != vi.ne[2] && va.ne[3] != 1))
        return fail(ctx, B200MOE_ERR_INVALID_ARG, "get_rows shapes");
    if (va.ne[2] == 1) va.nb[2] = 0;
    if (va.ne[3] == 1) va.nb[3] = 0;
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    op_get_rows_kernel<<<(unsigned) ((rows * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(va, vi, vd, ctx->d_err);
    return check_launch(ctx, "op_get_rows");
}

int b200moe_op_sum_rows(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    TensorView va, vd;
    if (!to_view(a, va, nullptr) || !to_view(dst, vd, nullptr)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad tensor");
    if (vd.ne[0] != 1 || vd.ne[1] != va.ne[1] || vd.ne[2] != va.ne[2] || vd.ne[3] != va.ne[3]) return fail(ctx, B200MOE_ERR_INVALID_ARG, "sum_rows shapes");
    const int64_t rows = va.ne[1] * va.ne[2] * va.ne[3];
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    op_sum_rows_kernel<<<(unsigned) ((rows + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(va, vd);
    return check_launch(ctx, "op_sum_rows");
}

int b200moe_op_soft_max(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, float scale, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    TensorView va, vd;
    if (!to_view(a, va, nullptr) || !to_view(dst, vd, nullptr)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad tensor");
    for (int i = 0; i < 4; ++i) if (va.ne[i] != vd.ne[i]) return fail(ctx, B200MOE_ERR_INVALID_ARG, "shapes differ");
    if (va.ne[0] % 8 || va.ne[0] > 1024) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "soft_max rows must be multiples of 8, at most 1024 long");
    const int64_t rows = va.ne[1] * va.ne[2] * va.ne[3];
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    op_soft_max_kernel<<<(unsigned) ((rows * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(va, vd, scale);
    return check_launch(ctx, "op_soft_max");
}

int b200moe_op_argsort_desc(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    TensorView va, vd;
    if (!to_view(a, va, nullptr) || !to_view(dst, vd, nullptr)) return fail(ctx, B200MOE_ERR_INVALID_ARG, "bad tensor");
    for (int i = 0; i < 4; ++i) if (va.ne[i] != vd.ne[i]) return fail(ctx, B200MOE_ERR_INVALID_ARG, "shapes differ");
    if (va.ne[0] > 1024) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "argsort rows of at most 1024 values");
    const int64_t rows = va.ne[1] * va.ne[2] * va.ne[3];
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    op_argsort_desc_kernel<<<(unsigned) rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(va, vd);
    return check_launch(ctx, "op_argsort");
}

// dst[e, t] = dot(w[:, e], x[:, t]) in ggml_vec_dot_f32's summation order (the router matmul's kernel without a router behind it)
int b200moe_op_mul_mat_f32(b200moe_ctx * ctx, const float * w, int64_t ne00, int64_t ne01, const float * x, int64_t T, float * dst, void * stream) {
    if (!ctx) return B200MOE_ERR_INVALID_ARG;
    if (T == 0) return B200MOE_OK;
    if (!w || !x || !dst || ne00 <= 0 || ne01 <= 0 || T < 0) return fail(ctx, B200MOE_ERR_INVALID_ARG, "null pointer or non-positive size");
    if (ne00 % 32) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "F32 matmul rows must be multiples of 32 long");
    if (ne01 * T > ((int64_t) 1 << 30)) return fail(ctx, B200MOE_ERR_UNSUPPORTED, "result too large");
    CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    return launch_logits_any<float>(ctx, w, nullptr, x, dst, (int) ne00, (int) ne01, (int) T, nullptr, 0, static_cast<cudaStream_t>(stream));
}

// ---- probe of the block-scaled FP4 instruction (fp4_probe.cuh) -----------------------------------------------------------

int b200moe_probe_fp4_tile(int device, const uint8_t * a_codes, const uint8_t * b_codes, const uint8_t * sfa, const uint8_t * sfb, float * d_host) {
    if (!a_codes || !b_codes || !sfa || !sfb || !d_host) return B200MOE_ERR_INVALID_ARG;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return B200MOE_ERR_NO_DEVICE; }
    if (device < 0 || device >= n || cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return B200MOE_ERR_INVALID_ARG; }
    std::vector<uint8_t> tiles(PROBE_TILE_BYTES);
    fp4_probe_pack(a_codes, b_codes, sfa, sfb, tiles.data());
    uint8_t * d_tiles = nullptr;
    float * d_out = nullptr;
    int * d_err = nullptr;
    int rc = B200MOE_OK, herr = 0;
    if (cudaMalloc(&d_tiles, PROBE_TILE_BYTES) != cudaSuccess || cudaMalloc(&d_out, sizeof(float) * 128 * PROBE_NB) != cudaSuccess ||
        cudaMalloc(&d_err, sizeof(int)) != cudaSuccess) rc = B200MOE_ERR_ALLOC;
    if (!rc && (cudaMemcpy(d_tiles, tiles.data(), PROBE_TILE_BYTES, cudaMemcpyHostToDevice) != cudaSuccess || cudaMemset(d_err, 0, sizeof(int)) != cudaSuccess ||
                cudaFuncSetAttribute(fp4_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM) != cudaSuccess)) rc = B200MOE_ERR_CUDA;
    if (!rc) {
        fp4_probe_kernel<<<1, 128, PROBE_SMEM>>>(d_tiles, d_out, 0, PROBE_NB, 1, d_err);
        if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(d_host, d_out, sizeof(float) * 128 * PROBE_NB, cudaMemcpyDeviceToHost) != cudaSuccess ||
            cudaMemcpy(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) rc = B200MOE_ERR_CUDA;
        else if (herr) rc = B200MOE_ERR_DEVICE_CHECK;
    }
    cudaGetLastError();
    cudaFree(d_tiles); cudaFree(d_out); cudaFree(d_err);
    return rc;
}

int b200moe_probe_fp4_rate(int device, int n_mma, int n_acc, int rounds, double * tflops) {
    if (!tflops || n_mma < 8 || n_mma > 256 || n_mma % 8 || n_acc < 1 || n_acc * n_mma + 48 > 512 || rounds < 1 || rounds > (1 << 22)) return B200MOE_ERR_INVALID_ARG;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return B200MOE_ERR_NO_DEVICE; }
    if (device < 0 || device >= n || cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return B200MOE_ERR_INVALID_ARG; }
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); return B200MOE_ERR_CUDA; }
    if (prop.major != 10) return B200MOE_ERR_UNSUPPORTED;
    // arbitrary operands: ones with unit scales (the rate does not depend on the values)
    std::vector<uint8_t> a(128 * 256, 2), b(PROBE_NB * 256, 2), sfa(128 * 16, 0x38), sfb(PROBE_NB * 16, 0x38), tiles(PROBE_TILE_BYTES);
    fp4_probe_pack(a.data(), b.data(), sfa.data(), sfb.data(), tiles.data());
    uint8_t * d_tiles = nullptr;
    int * d_err = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = B200MOE_OK, herr = 0;
    if (cudaMalloc(&d_tiles, PROBE_TILE_BYTES) != cudaSuccess || cudaMalloc(&d_err, sizeof(int)) != cudaSuccess) rc = B200MOE_ERR_ALLOC;
    if (!rc && (cudaMemcpy(d_tiles, tiles.data(), PROBE_TILE_BYTES, cudaMemcpyHostToDevice) != cudaSuccess || cudaMemset(d_err, 0, sizeof(int)) != cudaSuccess ||
                cudaFuncSetAttribute(fp4_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM) != cudaSuccess ||
                cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)) rc = B200MOE_ERR_CUDA;
    if (!rc) {
        const int sms = prop.multiProcessorCount;
        fp4_probe_kernel<<<sms, 128, PROBE_SMEM>>>(d_tiles, nullptr, std::max(1, rounds / 50), n_mma, n_acc, d_err);   // warm-up
        cudaEventRecord(e0);
        fp4_probe_kernel<<<sms, 128, PROBE_SMEM>>>(d_tiles, nullptr, rounds, n_mma, n_acc, d_err);
        cudaEventRecord(e1);
        float ms = 0.0f;
        if (cudaDeviceSynchronize() != cudaSuccess || cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess ||
            cudaMemcpy(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) rc = B200MOE_ERR_CUDA;
        else if (herr) rc = B200MOE_ERR_DEVICE_CHECK;
        else *tflops = 2.0 * 128 * n_mma * 64 * 4.0 * n_acc * (double) rounds * sms / (ms * 1e-3) / 1e12;
    }
    cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(d_tiles); cudaFree(d_err);
    return rc;
}

// ---- routing with no allocation at all -----------------------------------------------------------------
// Scratch for the router logits lives in the library image.  In HOST code the name below is only a stand-in for
// the symbol, not a device address, so the address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_logits[B200MOE_NOALLOC_MAX_LOGITS];
static float * g_noalloc_logits_ptr[64] = {};

static int noalloc_fail(char * buf, size_t len, int code, const char * msg) {
    if (buf && len) snprintf(buf, len, "%s", msg);
    return code;
}

int b200moe_route_noalloc(int device, const b200moe_layer * l, const void * x, int x_type, int32_t T, int32_t * ids, float * weights,
                          void * stream, char * errbuf, size_t errbuf_len) {
    if (errbuf && errbuf_len) errbuf[0] = 0;
    if (!l) return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_INVALID_ARG, "layer is null");
    if (T == 0) return B200MOE_OK;
    if (T < 0 || !x || !ids || !weights || !l->router_w) return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_INVALID_ARG, "null pointer or negative token count");
    if (device < 0 || device >= 64) return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_INVALID_ARG, "device ordinal out of range");
    if (x_type != TYPE_F32 && x_type != TYPE_BF16) return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_UNSUPPORTED, "activations must be F32 or BF16");
    const int E = l->n_expert, K = l->n_expert_used, H = l->n_embd;
    if (E <= 0 || K <= 0 || H <= 0 || K > E) return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_INVALID_ARG, "bad layer dimensions");
    if (K > 32 || E > 1024 || E % 8 || H % 32) return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_UNSUPPORTED, "need k <= 32, n_expert % 8 == 0 and <= 1024, n_embd % 32 == 0");
    if ((int64_t) T * E > B200MOE_NOALLOC_MAX_LOGITS) {
        char msg[160];
        snprintf(msg, sizeof msg, "n_tokens * n_expert = %lld exceeds the built-in scratch of %d floats", (long long) T * E, B200MOE_NOALLOC_MAX_LOGITS);
        return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_UNSUPPORTED, msg);
    }
    if (cudaSetDevice(device) != cudaSuccess) { cudaGetLastError(); return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_CUDA, "cudaSetDevice failed"); }
    if (!g_noalloc_logits_ptr[device]) {  // set-up, once per device, with that device current
        float * ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **) &ptr, g_noalloc_logits);
        if (e != cudaSuccess || !ptr) { cudaGetLastError(); return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_CUDA, cudaGetErrorString(e)); }
        g_noalloc_logits_ptr[device] = ptr;
    }
    float * logits = g_noalloc_logits_ptr[device];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    constexpr int TT = 4;
    const int64_t warps = (int64_t) E * ((T + TT - 1) / TT);
    const int lblocks = (int) ((warps * 32 + 255) / 256);
    if (x_type == TYPE_F32)
        router_logits_kernel<TT, float><<<lblocks, 256, 0, st>>>(l->router_w, l->router_bias, static_cast<const float *>(x), logits, H, E, T, nullptr, 0);
    else
        router_logits_kernel<TT, __nv_bfloat16><<<lblocks, 256, 0, st>>>(l->router_w, l->router_bias, static_cast<const __nv_bfloat16 *>(x), logits, H, E, T, nullptr, 0);
    const int sblocks = (T * 32 + 255) / 256;
#define SEL(EPL) route_select_kernel<EPL><<<sblocks, 256, 0, st>>>(logits, E, K, T, ids, weights, nullptr, nullptr, nullptr)
    if (E <= 32) SEL(1);
    else if (E <= 64) SEL(2);
    else if (E <= 128) SEL(4);
    else if (E <= 256) SEL(8);
    else if (E <= 512) SEL(16);
    else SEL(32);
#undef SEL
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return noalloc_fail(errbuf, errbuf_len, B200MOE_ERR_CUDA, cudaGetErrorString(e));
    return B200MOE_OK;
}

}  // extern "C"
