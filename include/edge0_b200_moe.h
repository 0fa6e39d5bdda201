/* edge0_b200_moe.h — C ABI of the B200 (sm_100a) quantised MoE-FFN path.
 *
 * Drop-in for the one hot path edge0-infer runs through ggml: router top-k, token->expert gather,
 * Q3_K / NVFP4 expert gate/up/down matmuls (ggml MUL_MAT_ID), SwiGLU and the weighted combine.
 * Plain pointers and sizes only; every function returns a b200moe_status (0 = success), validates
 * its arguments on the host before any launch and never aborts the process.  All tensor pointers
 * are DEVICE pointers unless the name ends in _host.  Layouts are ggml's (ne[0] fastest) and the
 * quantised blocks are ggml's block_q3_K / block_nvfp4 bytes, unchanged.
 *
 * Citations name the reference interface each entry point stands in for
 * (paths inside the Edge0 repository).
 */
#ifndef EDGE0_B200_MOE_H
#define EDGE0_B200_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200MOE_API __attribute__((visibility("default")))
#else
#define B200MOE_API
#endif

typedef struct b200moe_ctx b200moe_ctx;

/* values equal ggml_type (edge0-infer/third_party/ggml/include/ggml.h:398-430) */
enum b200moe_type { B200MOE_TYPE_F32 = 0, B200MOE_TYPE_Q3_K = 11, B200MOE_TYPE_BF16 = 30, B200MOE_TYPE_NVFP4 = 40 };

/* mirrors ggml_status (SUCCESS / FAILED / ALLOC_FAILED) plus argument errors that ggml asserts on */
enum b200moe_status {
    B200MOE_OK = 0,
    B200MOE_ERR_INVALID_ARG = 1,  /* null pointer, negative size, shape the op contract forbids */
    B200MOE_ERR_UNSUPPORTED = 2,  /* well-formed, but no kernel for this type / width */
    B200MOE_ERR_ALLOC = 3,        /* device scratch could not be allocated */
    B200MOE_ERR_CUDA = 4,         /* a CUDA call or launch failed; b200moe_last_error has the text */
    B200MOE_ERR_DEVICE_CHECK = 5, /* a kernel's own bounded wait or index check gave up */
    B200MOE_ERR_NO_DEVICE = 6
};

/* One MoE FFN layer's weights: what Builder::route / Builder::ffn look up by name
 * (edge0-infer/src/models/edge0_35b/forward.cpp:262-271, 300-311).
 *   router_w    F32 [n_embd, n_expert]            blk.N.ffn_gate_inp.weight
 *   router_bias F32 [n_expert] or NULL            added to the logits before the softmax
 *   gate/up     wtype [n_in, n_ff, n_expert]      blk.N.ffn_{gate,up}_exps.weight   (n_in = n_latent ? n_latent : n_embd)
 *   down        wtype [n_ff, n_in, n_expert]      blk.N.ffn_down_exps.weight
 *   *_scale     F32 [n_expert] or NULL            NVFP4 per-expert tensor scale, applied to the matmul result
 *                                                 (pattern at third_party/ggml/src/ggml-cuda/ggml-cuda.cu:3655-3673)
 *   lat_down    wtype [n_embd, n_latent]          shared projection into the latent width (n_latent > 0 only;
 *   lat_up      wtype [n_latent, n_embd]          semantics of edge0-strata/src/latent/latent_moe.cpp:38-92, one group)
 */
typedef struct b200moe_layer {
    int32_t n_embd;
    int32_t n_latent;      /* 0: experts work at n_embd */
    int32_t n_expert;
    int32_t n_expert_used; /* top-k */
    int32_t n_ff;
    int32_t wtype;         /* b200moe_type of gate/up/down (and lat_*) */
    const float * router_w;
    const float * router_bias;
    const void  * gate;
    const void  * up;
    const void  * down;
    const float * gate_scale;
    const float * up_scale;
    const float * down_scale;
    const void  * lat_down;
    const void  * lat_up;
    const float * lat_down_scale; /* F32 [1] or NULL */
    const float * lat_up_scale;   /* F32 [1] or NULL */
    /* shared expert with its sigmoid gate (forward.cpp:312-314): out += down_shexp(silu(gate_shexp x) * up_shexp x) * sigmoid(gate_inp_shexp . x).
     * All NULL / 0 when the layer has none; plain (non-latent) layers only.  Tensors of type wtype, [n_ff_shexp][n_embd] and
     * [n_embd][n_ff_shexp] rows; gate_inp_shexp F32 [n_embd].  The reference multiplies these without tensor scales. */
    const void  * gate_shexp;
    const void  * up_shexp;
    const void  * down_shexp;
    const float * gate_inp_shexp;
    int32_t n_ff_shexp;
    int32_t reserved_;
} b200moe_layer;

/* Optional observation outputs, named after the reference's ForwardRequest::observe labels
 * (forward.cpp:752-761).  Any pointer may be NULL. */
typedef struct b200moe_observe {
    float   * ffn_moe_logits;       /* F32 [n_expert, T] */
    float   * ffn_moe_probs;        /* F32 [n_expert, T] */
    int32_t * ffn_moe_topk;         /* I32 [k, T]        */
    float   * ffn_moe_weights_norm; /* F32 [k, T]        */
    float   * ffn_moe_hidden;       /* F32 [n_ff, k, T]  silu(gate)*up         */
    float   * ffn_moe_down;         /* F32 [n_in, k, T]  down, before weights  */
    float   * ffn_shexp_gated;      /* F32 [n_embd, T]   shared expert times its sigmoid gate (layers that have one) */
} b200moe_observe;

/* per-call counters (reference: WeightActivity / DecodeTiming, include/edge0/weight_activity.h, timing.h) */
typedef struct b200moe_counters {
    int64_t tokens;
    int64_t experts_touched;  /* distinct experts with at least one routed row */
    int64_t weight_bytes;     /* expert + router bytes the kernels streamed   */
    int64_t kernel_launches;
    int64_t fixup_overflow;   /* values the exact re-quantisation fix-up marked but could not list (its list holds a quarter of
                                 `hidden`): they kept the tensor-core result.  Updated by b200moe_synchronize.  Non-zero only for
                                 degenerate inputs such as blocks of equal values */
} b200moe_counters;

/* ---- lifetime (reference: ggml_backend_dev_init / ggml_backend_free through
 *      BackendFacility::create, edge0-infer/src/platform/backend.cpp:95-129) */
B200MOE_API int  b200moe_create(int device, b200moe_ctx ** out);
B200MOE_API void b200moe_destroy(b200moe_ctx * ctx);
/* Size the context's device scratch for up to max_tokens tokens of this layer shape (reference:
 * ggml_gallocr workspace sizing in exec::build_plan, edge0-infer/src/exec/execution.cpp:303-311).
 * Called implicitly by the compute entry points when the scratch is too small. */
B200MOE_API int  b200moe_reserve(b200moe_ctx * ctx, const b200moe_layer * layer, int32_t max_tokens);
B200MOE_API const char * b200moe_last_error(const b200moe_ctx * ctx);
B200MOE_API const char * b200moe_status_string(int status);
B200MOE_API int  b200moe_device_memory(int device, size_t * free_bytes, size_t * total_bytes); /* ggml_backend_dev_memory */
B200MOE_API int  b200moe_get_counters(const b200moe_ctx * ctx, b200moe_counters * out);
B200MOE_API int  b200moe_synchronize(b200moe_ctx * ctx, void * stream); /* ggml_backend_synchronize */

/* Which kernels run the expert matmuls (reference: model option switches such as `routing` / `experts`,
 * edge0-infer/docs/configuration.md:62-72; plain struct-style option, no environment variables).  Three engines exist:
 *   integer   dp4a kernels that follow the reference's fp32 summation order: bit-identical to the CPU path
 *   FP4       tcgen05 kind::mxf4nvf4 (block-scaled FP4 MMA, UE4M3 scale per 16): NVFP4 rows exactly as they lie in memory,
 *             activations as exact digit planes of the reference's int8 grid; differs from the integer engine only by fp32
 *             accumulation (~5e-6 of RMS on `hidden`); one pass over an expert's weights per 14 routed rows: batched decode
 *   f16       tcgen05 kind::f16: weights dequantised to fp16, activations as fp16 hi + lo (~1.4e-4 of RMS on `hidden`); one pass
 *             per 128 routed rows: prefill
 * The reference re-quantises `hidden` to int8 before `down`, which turns a tensor-core gate/up's error into a few flipped
 * values; the "fix-up" recomputes every value of `hidden` within a safe margin of a rounding boundary or of its block's maximum
 * with the integer engine's arithmetic, so the quantised `hidden` is the reference's own.
 *   0  default.  Up to 16 routed rows (one or two tokens at top-8): integer (bit-identical).  Fewer than 24 routed rows per
 *      expert on average: FP4 for gate/up and down (output within ~3e-3 of RMS at 256 tokens; latent layers, which re-quantise
 *      once more after `down`, add the fix-up).  More: f16 for gate/up and down, with the fix-up beyond 4096 routed rows;
 *      latent layers add the fix-up and keep `down` on the integer engine.  Types or widths an engine has no kernel for
 *      (Q3_K; n_ff not a multiple of 128; n_in not a multiple of 256 for FP4, of 128 for f16) fall back to integer.
 *      Dense products (b200moe_mul_mat, the latent projections) of NVFP4 matrices with at least 4 tokens use the FP4 engine
 *      under paths 0, 2, 3, 4, 6 and 8, the integer engine otherwise.
 *   1  integer everywhere: the whole layer is bit-identical to the reference CPU path
 *   2  f16 wherever the type and widths allow, no fix-up: output error growing to 1e-2 of RMS at 4096 tokens
 *   3  integer gate/up, f16 down
 *   4  as 2 plus the fix-up after gate/up: what remains is the ~1e-5 of the `down` GEMM
 *   5  f16 gate/up + fix-up, integer down: bit-identical whenever the fix-up's margin holds
 *   6  FP4 gate/up and down, no fix-up
 *   7  FP4 gate/up + fix-up, integer down: bit-identical whenever the fix-up's margin holds
 *   8  FP4 gate/up + fix-up, FP4 down
 * Paths 6-8 fail with B200MOE_ERR_UNSUPPORTED when the layer is not NVFP4 with n_ff % 128 == 0 and n_in % 256 == 0. */
B200MOE_API int  b200moe_set_expert_path(b200moe_ctx * ctx, int path);

/* Launch overlap (no counterpart in the reference; comparable to a backend's own stream options).  OFF by default.  When on, calls
 * in the batched-decode regime (fewer than 24 routed rows per expert on average; larger calls always launch serially) launch the
 * small kernels and the integer expert kernels of one layer as programmatic dependents of one another, so a kernel's launch and
 * set-up (barriers, tables) run alongside the tail of its predecessor; every kernel waits for its predecessor to finish before it
 * reads or writes global memory.  The tensor-core kernels are never launched this way and never release their dependents early:
 * nothing becomes resident beside a kernel that holds tensor memory.  Helps eagerly launched steps (+7 % through
 * b200moe_layer_forward_host when measured on the integer path), not CUDA-graph replay. */
B200MOE_API int  b200moe_set_launch_overlap(b200moe_ctx * ctx, int enable);
/* Per-kernel device timing (reference: DecodeTiming with an injectable clock, include/edge0/timing.h:4-9).
 * When enabled, every expert-matmul launch is bracketed by CUDA events on its stream; b200moe_kernel_times
 * waits for them and returns, for kind 0 (fused gate+up+SwiGLU), kind 1 (single indexed matmul / down) and kind 2 (dense
 * products: b200moe_mul_mat, the latent projections), the number of launches and their summed duration since the last call.
 * Do not enable it while a stream is being captured. */
B200MOE_API int  b200moe_enable_kernel_timing(b200moe_ctx * ctx, int enable);
B200MOE_API int  b200moe_kernel_times(b200moe_ctx * ctx, int64_t launches[3], double total_ms[3]);

/* ---- data formats (reference: ggml_row_size, ggml.h:761; quantize_row_nvfp4_ref, ggml-quants.c:384-417;
 *      dequantize_row_q3_K / _nvfp4, ggml-quants.c:1305-1353, 589-612).  Host memory. */
B200MOE_API int64_t b200moe_row_size(int type, int64_t n);
/* 1 when b200moe_mul_mat_id / b200moe_mul_mat have a kernel for rows of ne00 values of this type (what a backend's supports_op asks) */
B200MOE_API int  b200moe_mul_mat_id_width_ok(int type, int64_t ne00);
B200MOE_API int  b200moe_quantize_nvfp4_host(const float * src, void * dst, int64_t nrows, int64_t n_per_row);
B200MOE_API int  b200moe_dequantize_host(int type, const void * src, float * dst, int64_t nrows, int64_t n_per_row);

/* ---- expert packs of edge0-strata (tools/iq_pack.py, docs/NVFP4.md:44-47; layout: NativeExpertLayout,
 *      include/strata/kernels/iq_kernels.hpp:53-60): experts.bin holds one blob per expert,
 *          [gate rows (n_ff x n_embd) | up rows (n_ff x n_embd) | down rows (n_embd x n_ff)] as raw block_nvfp4 rows
 *          + a 16-byte tail {s_gate, s_up, s_down, 0} (fp32),
 *      because the GGUF has no room for the per-tensor scales.  The rows are the bytes the kernels read: loading is three
 *      copies per expert into the [n_expert][rows][row_bytes] tensors of b200moe_layer plus the tails into its three scale
 *      arrays - no repacking.  `blobs` is host memory, expert e at blobs + e * blob_stride (blob_stride >= blob bytes).
 *      to_device = 0: the destinations are host memory too; 1: device memory, copied on `stream`, which the call synchronises
 *      before it returns (the blobs may be freed afterwards). */
B200MOE_API int64_t b200moe_expert_blob_bytes_nvfp4(int32_t n_embd, int32_t n_ff);
B200MOE_API int  b200moe_unpack_expert_blobs_nvfp4(const void * blobs, int64_t blob_stride, int32_t n_expert, int32_t n_embd, int32_t n_ff,
                                                   void * gate, void * up, void * down, float * gate_scale, float * up_scale,
                                                   float * down_scale, int to_device, void * stream);

/* ---- GGUF model files (reference: edge0-infer reads its weights through ggml's gguf API, src/model/asset_index.cpp; format:
 *      third_party/ggml/docs/gguf.md).  Host code.  The file is mapped read-only and tensors are handed out as pointers into the
 *      mapping, in ggml's block layout - the layout the kernels read, so a layer loads with one copy per tensor and no repacking.
 *      b200moe_gguf_moe_layer fills a b200moe_layer with HOST pointers to the MoE FFN tensors of block `layer` as edge0-infer names
 *      them (forward.cpp:262-314: blk.N.ffn_gate_inp.weight, ffn_gate_exps / ffn_up_exps / ffn_down_exps .weight, optionally
 *      exp_probs_b.bias and the four shared-expert tensors); n_expert_used <= 0 reads <general.architecture>.expert_used_count
 *      (models/edge0_35b/assets.cpp:63-66).  The caller copies the tensors to the device (their sizes: b200moe_gguf_tensor) and
 *      passes device pointers to the compute entry points; the mapping must stay open until those copies are done. */
typedef struct b200moe_gguf b200moe_gguf;
B200MOE_API int  b200moe_gguf_open(const char * path, b200moe_gguf ** out, char * err, size_t err_len);
B200MOE_API void b200moe_gguf_close(b200moe_gguf * g);
B200MOE_API int64_t b200moe_gguf_n_tensors(const b200moe_gguf * g);
/* B200MOE_ERR_INVALID_ARG: no such tensor; B200MOE_ERR_UNSUPPORTED: a ggml type this library does not read (type and ne are still set) */
B200MOE_API int  b200moe_gguf_tensor(const b200moe_gguf * g, const char * name, int32_t * type, int64_t ne[4], const void ** data, uint64_t * nbytes);
B200MOE_API int  b200moe_gguf_metadata_u64(const b200moe_gguf * g, const char * key, uint64_t * value);
B200MOE_API int  b200moe_gguf_moe_layer(const b200moe_gguf * g, int32_t layer, int32_t n_expert_used, b200moe_layer * out, char * err, size_t err_len);

/* ---- compute.  `stream` is a cudaStream_t (NULL = default stream); calls are asynchronous on it. */

/* Builder::route (forward.cpp:262-271) = mul_mat(F32) -> soft_max -> argsort_top_k -> get_rows ->
 * sum_rows -> clamp(2^-14) -> div.  x: x_type (F32 or BF16) [n_embd, T].
 * ids I32 [k, T] (expert indices, descending probability); weights F32 [k, T].
 * Reads router_w / router_bias only: the expert pointers of `layer` may be NULL here (the dimensions must still be valid). */
B200MOE_API int b200moe_route(b200moe_ctx * ctx, const b200moe_layer * layer, const void * x, int x_type,
                              int32_t n_tokens, int32_t * ids, float * weights,
                              const b200moe_observe * observe, void * stream);

/* ggml_mul_mat_id (ggml.c:3392-3416; CPU kernel ggml-cpu/ggml-cpu.c:1550-1740).
 *   as   wtype [ne00, ne01, n_as]   b  F32 [ne00, ne11, T]   ids I32 [n_ids, T], row stride ids_nb1 bytes
 *   dst  F32 [ne01, n_ids, T];  row (id, t) uses b[:, id % ne11, t] quantised to the type's vec_dot_type.
 * ids may index expert slots rather than experts (edge0-infer/src/weights/expert_slots.h:13-18). */
B200MOE_API int b200moe_mul_mat_id(b200moe_ctx * ctx, int wtype, const void * as, int64_t ne00, int64_t ne01, int64_t n_as,
                                   const float * b, int64_t ne11, const int32_t * ids, int64_t n_ids, int64_t ids_nb1,
                                   int64_t n_tokens, float * dst, void * stream);

/* ggml_mul_mat with a quantised weight matrix (ggml-cpu/ggml-cpu.c:1255-1468): dst F32 [ne01, T] = W [ne00, ne01] . x F32 [ne00, T],
 * x quantised to the type's vec_dot_type first; optional fp32 scale[1] multiplies the result (NVFP4 tensor scale).
 * Used for the shared latent projections of the expert-parallel layer. */
B200MOE_API int b200moe_mul_mat(b200moe_ctx * ctx, int wtype, const void * w, int64_t ne00, int64_t ne01, const float * x, int64_t n_tokens,
                                const float * scale, float * dst, void * stream);

/* The two shared projections of a latent layer as calls of their own (edge0-strata/src/latent/latent_moe.cpp:38-92: xl = D x before
 * the experts, y = U m behind the combine); the expert-parallel layer runs them on the token's rank.  x: [n_embd, T] in x_type;
 * xl F32 [n_latent, T]; m F32 [n_latent, T]; out F32 [n_embd, T].  The latent rows are re-quantised by whoever runs the experts:
 * whatever engine computes them, their quantised (Q8_0) form is the reference's (exact fix-up behind the FP4 engine). */
B200MOE_API int b200moe_latent_down(b200moe_ctx * ctx, const b200moe_layer * layer, const void * x, int x_type, int32_t n_tokens, float * xl,
                                    void * stream);
B200MOE_API int b200moe_latent_up(b200moe_ctx * ctx, const b200moe_layer * layer, const float * m, int32_t n_tokens, float * out, void * stream);

/* The tail of Builder::ffn (forward.cpp:308-310): out[:, t] = sum over slots s = 0..k-1, in that order, of y[:, s, t] * weights[s, t].
 * y F32 [n, k, T], weights F32 [k, T], out F32 [n, T]. */
B200MOE_API int b200moe_combine(b200moe_ctx * ctx, const float * y, const float * weights, float * out, int64_t n, int64_t k, int64_t n_tokens,
                                void * stream);

/* ggml_get_rows on F32 rows (ggml-cpu/ops.cpp get_rows): dst[r, :] = src[idx[r], :]; used to pack rows for token dispatch and to put
 * returned rows back into slot order.  width must be a multiple of 4. */
B200MOE_API int b200moe_gather_rows(b200moe_ctx * ctx, const float * src, int64_t src_rows, const int32_t * idx, float * dst, int64_t n_rows,
                                    int64_t width, void * stream);

/* ---- expert-parallel exchange.  The reference has no multi-GPU form of the latent layer (edge0-strata/src/latent/latent_moe.cpp:38-92
 * runs on one device; its peer experts are staged through the host, src/core/peer_experts.cpp:186-192), so these three entry
 * points replace nothing: they are the device side of an all-to-all whose split sizes never depend on the routing.
 *   Expert e lives on rank e / experts_per_rank.  Every rank sends every peer `capacity` SLOTS (capacity >= the rank's routed
 *   rows T * k, its worst case), so one equal-split all-to-all of n_ranks * capacity slots moves the rows and a second one of
 *   n_ranks * capacity result rows brings them back, with no count read on the host between routing and the collective.
 *   A slot is (width + 4) * 4 bytes (b200moe_ep_slot_bytes): the F32 row, the expert id local to the destination rank, padding;
 *   id -1 marks an empty slot. */
B200MOE_API int64_t b200moe_ep_slot_bytes(int64_t width);
/* rows F32 [width, T], ids I32 [k, T] (global expert ids) -> slots [n_ranks][capacity] ordered by destination rank, slot_of I32 [k, T]
 * (where routed row (t, s) went: dest * capacity + position), fill I32 [n_ranks] scratch (rows per destination afterwards). */
B200MOE_API int b200moe_ep_pack(b200moe_ctx * ctx, const float * rows, const int32_t * ids, int64_t n_tokens, int64_t k, int64_t width,
                                int64_t n_ranks, int64_t experts_per_rank, int64_t capacity, void * slots, int32_t * slot_of, int32_t * fill,
                                void * stream);
/* The owner's side: `layer` holds this rank's experts as a plain layer of the exchanged width (n_embd = width, n_latent = 0,
 * n_expert = experts_per_rank; router_w may be NULL).  Every non-empty slot is one routed row: y[slot] = down_e(silu(gate_e x) * up_e x),
 * the arithmetic of b200moe_ffn with one slot of weight 1.  y F32 [width, n_slots]; rows of empty slots are left untouched. */
B200MOE_API int b200moe_ep_expert_rows(b200moe_ctx * ctx, const b200moe_layer * layer, const void * slots, int64_t n_slots, float * y,
                                       void * stream);
/* Back on the token's rank: out[:, t] = sum over s = 0..k-1, in that order, of back[:, slot_of[s, t]] * weights[s, t]
 * (the tail of Builder::ffn, forward.cpp:308-310, behind an index).  back F32 [width, n_slots]. */
B200MOE_API int b200moe_ep_combine(b200moe_ctx * ctx, const float * back, int64_t n_slots, const int32_t * slot_of, const float * weights,
                                   int64_t n_tokens, int64_t k, int64_t width, float * out, void * stream);

/* Builder::ffn with given routing (forward.cpp:300-311): gate/up mul_mat_id -> silu*up -> down mul_mat_id ->
 * * weights -> sum over slots in slot order.  x: [n_in, T] in x_type; out F32 [n_in, T].
 * Reads the expert tensors only: router_w and the latent projections of `layer` may be NULL here. */
B200MOE_API int b200moe_ffn(b200moe_ctx * ctx, const b200moe_layer * layer, const void * x, int x_type, int32_t n_tokens,
                            const int32_t * ids, const float * weights, float * out,
                            const b200moe_observe * observe, void * stream);

/* route + (latent down) + ffn + (latent up): the whole layer on device buffers.  out F32 [n_embd, T]. */
B200MOE_API int b200moe_layer_forward(b200moe_ctx * ctx, const b200moe_layer * layer, const void * x, int x_type,
                                      int32_t n_tokens, float * out, const b200moe_observe * observe, void * stream);

/* Same through HOST buffers: copies x in, runs the layer, copies out (and ids/weights when non-NULL) back and
 * waits.  This is what a caller holding host tensors pays (exec::Plan::set_inputs / read_output =
 * ggml_backend_tensor_set / _get, edge0-infer/src/exec/execution.cpp:343,421). */
B200MOE_API int b200moe_layer_forward_host(b200moe_ctx * ctx, const b200moe_layer * layer, const void * x_host, int x_type,
                                           int32_t n_tokens, float * out_host, int32_t * ids_host, float * weights_host,
                                           void * stream);

/* ---- the small F32 operators around the MoE sub-graphs, one call per ggml op, for graph nodes that are not part of a fused
 * pattern (reference: the CPU backend's operators, ggml-cpu/ops.cpp; what exec::Plan needs a backend to run for every node it
 * said it supports, edge0-infer/src/exec/execution.cpp:256-260).  Tensors are described as ggml does: ne[] elements, nb[] byte
 * strides.  add / mul / div (second operand repeated over the first), clamp, repeat, get_rows and sum_rows are bit-identical to
 * the CPU operators; soft_max and silu are for rows that are multiples of 8 long (beyond, the reference finishes with libm's
 * expf); sigmoid evaluates the reference's expf as the double-precision exponential rounded to float (the correctly rounded value
 * but for rare double-rounding cases); argsort is descending with equal values in index
 * order (the reference leaves their order unspecified). */
typedef struct b200moe_tensor {
    void *  data;
    int64_t ne[4];
    int64_t nb[4];
} b200moe_tensor;
enum { B200MOE_OP_ADD = 0, B200MOE_OP_MUL = 1, B200MOE_OP_DIV = 2 };
enum { B200MOE_OP_SILU = 0, B200MOE_OP_SIGMOID = 1, B200MOE_OP_CLAMP = 2 };   /* clamp: p0 = min, p1 = max */
B200MOE_API int b200moe_op_binary(b200moe_ctx * ctx, int op, const b200moe_tensor * a, const b200moe_tensor * b, const b200moe_tensor * dst,
                                  void * stream);
B200MOE_API int b200moe_op_unary(b200moe_ctx * ctx, int op, const b200moe_tensor * a, const b200moe_tensor * dst, float p0, float p1, void * stream);
B200MOE_API int b200moe_op_repeat(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, void * stream);
B200MOE_API int b200moe_op_get_rows(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * ids, const b200moe_tensor * dst, void * stream);
B200MOE_API int b200moe_op_sum_rows(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, void * stream);
B200MOE_API int b200moe_op_soft_max(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, float scale, void * stream);
B200MOE_API int b200moe_op_argsort_desc(b200moe_ctx * ctx, const b200moe_tensor * a, const b200moe_tensor * dst, void * stream);
/* ggml_mul_mat of two F32 matrices in ggml_vec_dot_f32's summation order (ggml-cpu/vec.cpp:11): dst [ne01, T] = w [ne00, ne01] . x [ne00, T] */
B200MOE_API int b200moe_op_mul_mat_f32(b200moe_ctx * ctx, const float * w, int64_t ne00, int64_t ne01, const float * x, int64_t n_tokens, float * dst,
                                       void * stream);

/* ---- probe of the block-scaled FP4 tensor-core instruction (tcgen05.mma kind::mxf4nvf4, UE4M3 scale per 16 values; the reference's only
 * Blackwell kernel is the warp-level form of it, ggml-cuda/mma.cuh:1186-1214).  Not part of the layer: it pins the operand formats
 * the FP4 engine relies on and measures the denominator of "% of FP4 peak".  Both allocate and free their own device memory.
 *   tile: D[128][256] (host, F32) = A[128][256] . B[256][256]^T with one E2M1 code per byte in a_codes / b_codes (row-major, K = 256)
 *         and one UE4M3 byte per 16 values in sfa [128][16] / sfb [256][16].
 *   rate: dense TFLOP/s of `rounds` x 4 x n_acc instructions (M = 128, N = n_mma, K = 64) per SM that alternate between n_acc
 *         accumulators, operands resident in shared memory, every SM busy.  n_mma % 8 == 0, n_acc * n_mma + 48 <= 512. */
B200MOE_API int b200moe_probe_fp4_tile(int device, const uint8_t * a_codes, const uint8_t * b_codes, const uint8_t * sfa, const uint8_t * sfb,
                                       float * d_host);
B200MOE_API int b200moe_probe_fp4_rate(int device, int n_mma, int n_acc, int rounds, double * tflops);

/* Routing without any allocation.  (No counterpart in the reference: its backends always own a workspace.)
 *
 * For callers that must not trigger cudaMalloc: code running inside a latency-critical serving loop, inside a
 * memory pool that has handed the whole device to someone else, or on a thread that is not allowed to take the
 * allocator's lock.  It computes exactly what b200moe_route computes (same kernels, same bits), but keeps the
 * intermediate router logits in a fixed array that is part of the library image instead of context scratch, and it
 * needs no b200moe_ctx.
 *
 * Limit: n_tokens * n_expert <= B200MOE_NOALLOC_MAX_LOGITS (32768 floats = 128 KiB, e.g. 256 tokens x 128 experts).
 * Every GPU that loads the library holds that array until the process exits.  Larger requests are rejected with
 * B200MOE_ERR_UNSUPPORTED; nothing is launched.
 *
 * The first call on each device looks up the array's device address (one cudaGetSymbolAddress, which may load the
 * module): make that first call outside of any stream capture.  All calls on a device share the one array: it is
 * fully overwritten by each call (nothing has to start at zero), and two calls whose kernels overlap on the GPU
 * (different streams, no ordering between them) race on it - serialise them.
 * `device` is the CUDA device ordinal of the pointers; it is made current.  errbuf (may be NULL) receives a
 * message when the status is not B200MOE_OK. */
#define B200MOE_NOALLOC_MAX_LOGITS 32768
B200MOE_API int b200moe_route_noalloc(int device, const b200moe_layer * layer, const void * x, int x_type, int32_t n_tokens,
                                      int32_t * ids, float * weights, void * stream, char * errbuf, size_t errbuf_len);

#ifdef __cplusplus
}
#endif
#endif /* EDGE0_B200_MOE_H */
