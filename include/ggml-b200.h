/* ggml-b200.h — ggml backend that runs the quantised MoE-FFN sub-graphs on a B200 through the C ABI of
 * edge0_b200_moe.h.
 *
 * It plugs in where edge0-infer picks a ggml backend device (BackendFacility::create,
 * edge0-infer/src/platform/backend.cpp:95-129) and implements ggml's backend interface
 * (third_party/ggml/src/ggml-backend-impl.h: ggml_backend_reg_i, ggml_backend_device_i,
 * ggml_backend_buffer_type_i, ggml_backend_buffer_i, ggml_backend_i).
 *
 * Scope: the graphs Builder::route and Builder::ffn emit (src/models/edge0_35b/forward.cpp:262-271, 300-311),
 * optionally with a per-expert bias on the router logits, the NVFP4 per-expert scale pattern
 * (reshape -> repeat -> get_rows -> mul after a MUL_MAT_ID, ggml-cuda/ggml-cuda.cu:3655-3673), a dense quantised
 * MUL_MAT (optionally times a one-element scale) and CONT of a row-strided tensor.  graph_compute recognises those
 * sub-graphs and runs each as one fused call; a graph with any other compute node is refused with
 * GGML_STATUS_FAILED (nothing is silently computed elsewhere).  ggml_backend_sched therefore has to give this
 * backend whole route / ffn sub-graphs, which is how the reference schedules them (one device per layer).
 */
#ifndef GGML_B200_H
#define GGML_B200_H

#include "ggml.h"
#include "ggml-backend.h"

#ifdef __cplusplus
extern "C" {
#endif

#define GGML_B200_NAME "B200"

/* registry with one device per visible CUDA device of compute capability 10.x */
GGML_BACKEND_API ggml_backend_reg_t ggml_backend_b200_reg(void);

/* a backend (stream) on CUDA device `device`; NULL when the device is absent or not sm_100 */
GGML_BACKEND_API ggml_backend_t ggml_backend_b200_init(int device);
GGML_BACKEND_API bool ggml_backend_is_b200(ggml_backend_t backend);

/* device-memory buffer type of `device` */
GGML_BACKEND_API ggml_backend_buffer_type_t ggml_backend_b200_buffer_type(int device);

/* expert kernel policy, see b200moe_set_expert_path (0 default, 1 integer kernels only = bit-identical to the CPU backend) */
GGML_BACKEND_API int ggml_backend_b200_set_expert_path(ggml_backend_t backend, int path);

/* what the last graph_compute did: fused route groups, fused ffn groups, dense matmuls, other nodes run one by one,
 * results that went through backend scratch because their graph memory was still in use when they were computed */
struct ggml_b200_graph_stats {
    int n_route;
    int n_ffn;
    int n_dense;
    int n_single;
    int n_nodes;
    int n_deferred;
};
GGML_BACKEND_API int ggml_backend_b200_graph_stats(ggml_backend_t backend, struct ggml_b200_graph_stats * out);

/* text of the last failure of this backend ("" when none) */
GGML_BACKEND_API const char * ggml_backend_b200_last_error(ggml_backend_t backend);

#ifdef __cplusplus
}
#endif
#endif /* GGML_B200_H */
