/* TEST INFRASTRUCTURE: CPU restatement of the reference's quantised MoE-FFN path.
 * Only tests, the smoke check and the benchmark's cpu_baseline leg may use it; the
 * product library never links or calls it.  See moe_oracle.c for the reference citations. */
#ifndef MOE_ORACLE_H
#define MOE_ORACLE_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_TYPE_F32 = 0, ORC_TYPE_Q3_K = 11, ORC_TYPE_NVFP4 = 40 };

/* Same field order as ref_moe_args in ref_driver.cpp so one Python struct serves both. */
typedef struct orc_moe_args {
    int32_t H, L, E, K, I, T;
    int32_t wtype;
    int32_t n_threads;   /* ignored: the restatement is scalar, single-threaded */
    int32_t repeats;     /* timed repetitions after the first evaluation */
    int32_t latent;
    const float * x;
    const float * router_w;
    const float * router_bias;
    const void  * gate;
    const void  * up;
    const void  * down;
    const float * s_gate;
    const float * s_up;
    const float * s_down;
    const void  * lat_d;
    const void  * lat_u;
    const float * s_lat_d;
    const float * s_lat_u;
    float   * logits;
    float   * probs;
    int32_t * ids;
    float   * weights;
    float   * hidden;
    float   * down_out;
    float   * moe_out;
    float   * out;
    double  * ms_best;
    double  * ms_median;
    /* shared expert with its sigmoid gate (edge0-infer/src/models/edge0_35b/forward.cpp:312-314); all null / 0 when the layer has none.
     * Non-latent layers only. */
    const void  * sh_gate;      /* [I_sh][H] quantised rows */
    const void  * sh_up;        /* [I_sh][H] */
    const void  * sh_down;      /* [H][I_sh] */
    const float * sh_gate_inp;  /* [H] F32 */
    float   * shexp_gated;      /* [T][H] output: shared expert times its gate, or null */
    int32_t   I_sh;
    int32_t   pad_;
} orc_moe_args;

int64_t  orc_row_size(int type, int64_t n);
float    orc_fp16_to_fp32(uint16_t h);
uint16_t orc_fp32_to_fp16(float f);
float    orc_ue4m3_to_fp32(uint8_t x);
uint8_t  orc_fp32_to_ue4m3(float x);

void orc_quantize_row_nvfp4(const float * x, void * y, int64_t k);
void orc_dequantize_row_nvfp4(const void * x, float * y, int64_t k);
void orc_dequantize_row_q3_K(const void * x, float * y, int64_t k);
int  orc_dequantize(int type, const void * src, float * dst, int64_t n);
int  orc_quantize(int type, const float * src, void * dst, int64_t nrows, int64_t n_per_row);

void orc_quantize_row_q8_0(const float * x, void * y, int64_t k);
void orc_quantize_row_q8_K(const float * x, void * y, int64_t k);
int64_t orc_quantize_activation(int wtype, const float * src, void * dst, int64_t n);

float orc_vec_dot_f32(int n, const float * x, const float * y);
float orc_vec_dot_q3_K_q8_K(int n, const void * w, const void * a);
float orc_vec_dot_nvfp4_q8_0(int n, const void * w, const void * a);
int   orc_vec_dot(int wtype, int64_t n, const void * wrow, const void * act, float * out);

float orc_expf(float x);
float orc_silu(float x);
void  orc_soft_max_row(int n, float * y, const float * x);
/* top-k of one row, descending; ties broken by ascending index.  Returns 1 when a tie
 * (equal values) touches the selection, which the reference's unstable sort leaves unspecified. */
int   orc_top_k_row(int n, int k, const float * p, int32_t * ids);

int   orc_moe_layer(const orc_moe_args * a);

#ifdef __cplusplus
}
#endif
#endif
