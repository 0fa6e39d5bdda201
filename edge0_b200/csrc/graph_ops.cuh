// The small F32 graph operators around the MoE sub-graphs, one kernel per ggml op, for graphs (or parts of graphs) that do not
// match a fused pattern: ADD / MUL / DIV with ggml's broadcasting, SILU, SIGMOID, CLAMP, SOFT_MAX, ARGSORT (descending),
// GET_ROWS, SUM_ROWS, REPEAT.  Each follows the reference CPU operator's arithmetic (ggml-cpu/ops.cpp, vec.h, vec.cpp):
//   * add, mul, div, clamp, repeat, get_rows: single correctly rounded operations or copies - bit-identical;
//   * sum_rows: sequential accumulation in double (ggml_vec_sum_f32, vec.h:1495-1505) - bit-identical;
//   * soft_max: ggml_v_expf lanes, groups of 8 summed as the AVX2 horizontal add does, groups accumulated in double, scaled by
//     (float)(1/sum) (ops.cpp:5584-5694, vec.cpp:531-551) - bit-identical for rows that are multiples of 8;
//   * silu: x / (1 + exp(-x)) with ggml_v_expf (vec.cpp:380-392, the SIMD body) - bit-identical for rows that are multiples of 8
//     (the reference finishes a ragged tail with libm's expf);
//   * sigmoid: the reference calls libm's expf per element (vec.h:936); here expf is the double-precision exponential rounded to
//     float (the correctly rounded value but for double-rounding cases rarer than 1 in 2^28);
//   * argsort: the reference's std::sort leaves the order of equal values unspecified; here equal values keep index order.
// Tensors are described as ggml describes them: ne[4] elements, nb[4] byte strides.
#pragma once
#include "common.cuh"

namespace b200moe {

struct TensorView {
    char * data;
    int64_t ne[4];
    int64_t nb[4];
};

__device__ __forceinline__ int64_t view_offset(const TensorView & t, int64_t i0, int64_t i1, int64_t i2, int64_t i3) {
    return i0 * t.nb[0] + i1 * t.nb[1] + i2 * t.nb[2] + i3 * t.nb[3];
}

enum BinaryOp : int { BIN_ADD = 0, BIN_MUL = 1, BIN_DIV = 2 };
enum UnaryOp : int { UN_SILU = 0, UN_SIGMOID = 1, UN_CLAMP = 2 };

// dst[i] = a[i] op b[i mod ne(b)] (ggml_compute_forward_add / mul / div with src1 broadcast over src0)
__global__ void __launch_bounds__(256) op_binary_kernel(int op, TensorView a, TensorView b, TensorView d) {
    const int64_t n = d.ne[0] * d.ne[1] * d.ne[2] * d.ne[3];
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t i0 = i % d.ne[0], r1 = i / d.ne[0], i1 = r1 % d.ne[1], r2 = r1 / d.ne[1], i2 = r2 % d.ne[2], i3 = r2 / d.ne[2];
        const float x = *reinterpret_cast<const float *>(a.data + view_offset(a, i0, i1, i2, i3));
        const float y = *reinterpret_cast<const float *>(b.data + view_offset(b, i0 % b.ne[0], i1 % b.ne[1], i2 % b.ne[2], i3 % b.ne[3]));
        const float r = op == BIN_ADD ? __fadd_rn(x, y) : op == BIN_MUL ? __fmul_rn(x, y) : __fdiv_rn(x, y);
        *reinterpret_cast<float *>(d.data + view_offset(d, i0, i1, i2, i3)) = r;
    }
}

__global__ void __launch_bounds__(256) op_unary_kernel(int op, TensorView a, TensorView d, float p0, float p1) {
    const int64_t n = d.ne[0] * d.ne[1] * d.ne[2] * d.ne[3];
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t i0 = i % d.ne[0], r1 = i / d.ne[0], i1 = r1 % d.ne[1], r2 = r1 / d.ne[1], i2 = r2 % d.ne[2], i3 = r2 / d.ne[2];
        const float x = *reinterpret_cast<const float *>(a.data + view_offset(a, i0, i1, i2, i3));
        float r;
        if (op == UN_SILU) r = ggml_silu(x);
        else if (op == UN_SIGMOID) r = __fdiv_rn(1.0f, __fadd_rn(1.0f, (float) exp((double) -x)));
        else r = x < p0 ? p0 : (x > p1 ? p1 : x);
        *reinterpret_cast<float *>(d.data + view_offset(d, i0, i1, i2, i3)) = r;
    }
}

// dst[i] = a[i mod ne(a)] (ggml_compute_forward_repeat)
__global__ void __launch_bounds__(256) op_repeat_kernel(TensorView a, TensorView d) {
    const int64_t n = d.ne[0] * d.ne[1] * d.ne[2] * d.ne[3];
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t i0 = i % d.ne[0], r1 = i / d.ne[0], i1 = r1 % d.ne[1], r2 = r1 / d.ne[1], i2 = r2 % d.ne[2], i3 = r2 / d.ne[2];
        *reinterpret_cast<float *>(d.data + view_offset(d, i0, i1, i2, i3)) =
            *reinterpret_cast<const float *>(a.data + view_offset(a, i0 % a.ne[0], i1 % a.ne[1], i2 % a.ne[2], i3 % a.ne[3]));
    }
}

// dst[:, i10, i11, i12] = a[:, ids[i10, i11, i12], i11, i12] (ggml_compute_forward_get_rows_f32); one warp per row; bad ids are reported
__global__ void __launch_bounds__(256) op_get_rows_kernel(TensorView a, TensorView ids, TensorView d, int * err) {
    const int64_t rows = ids.ne[0] * ids.ne[1] * ids.ne[2];
    const int64_t w = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= rows) return;
    const int64_t i10 = w % ids.ne[0], i11 = (w / ids.ne[0]) % ids.ne[1], i12 = w / (ids.ne[0] * ids.ne[1]);
    const int32_t r = *reinterpret_cast<const int32_t *>(ids.data + i10 * ids.nb[0] + i11 * ids.nb[1] + i12 * ids.nb[2]);
    if (r < 0 || r >= a.ne[1]) { if (lane == 0) report_error(err, DEV_ERR_BAD_EXPERT_ID); return; }
    const char * src = a.data + (int64_t) r * a.nb[1] + i11 * a.nb[2] + i12 * a.nb[3];
    char * dst = d.data + i10 * d.nb[1] + i11 * d.nb[2] + i12 * d.nb[3];
    for (int64_t i = lane; i < a.ne[0]; i += 32) *reinterpret_cast<float *>(dst + i * d.nb[0]) = *reinterpret_cast<const float *>(src + i * a.nb[0]);
}

// dst[0, i1, i2, i3] = (float) sum in double over i0, in index order; one thread per row
__global__ void __launch_bounds__(256) op_sum_rows_kernel(TensorView a, TensorView d) {
    const int64_t rows = a.ne[1] * a.ne[2] * a.ne[3];
    const int64_t r = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int64_t i1 = r % a.ne[1], i2 = (r / a.ne[1]) % a.ne[2], i3 = r / (a.ne[1] * a.ne[2]);
    const char * src = a.data + view_offset(a, 0, i1, i2, i3);
    double s = 0.0;
    for (int64_t i = 0; i < a.ne[0]; ++i) s += (double) *reinterpret_cast<const float *>(src + i * a.nb[0]);
    *reinterpret_cast<float *>(d.data + view_offset(d, 0, i1, i2, i3)) = (float) s;
}

// soft_max over rows of n <= 1024 elements, n % 8 == 0 (no mask, max_bias 0): one warp per row, lane owns n/32-element slices
// interleaved by groups of 8 so that the reference's 8-lane groups can be summed in its order.
__global__ void __launch_bounds__(256) op_soft_max_kernel(TensorView a, TensorView d, float scale) {
    const int64_t rows = a.ne[1] * a.ne[2] * a.ne[3];
    const int64_t r = ((int64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    const int64_t i1 = r % a.ne[1], i2 = (r / a.ne[1]) % a.ne[2], i3 = r / (a.ne[1] * a.ne[2]);
    const char * src = a.data + view_offset(a, 0, i1, i2, i3);
    char * dst = d.data + view_offset(d, 0, i1, i2, i3);
    const int n = (int) a.ne[0];
    // element e lives on lane (e / 8) % 32 ... keep it simple: lane l owns elements l, l + 32, ... (values), group sums via shuffles
    float mx = -INFINITY;
    for (int e = lane; e < n; e += 32) mx = fmaxf(mx, __fmul_rn(*reinterpret_cast<const float *>(src + (int64_t) e * a.nb[0]), scale));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    double sum = 0.0;
    // 32 elements per step = four groups of 8; lane l holds element base + l; group g = lanes 8g .. 8g+7
    for (int base = 0; base < n; base += 32) {
        const int e = base + lane;
        float v = 0.0f;
        if (e < n) {
            v = ggml_expf(__fsub_rn(__fmul_rn(*reinterpret_cast<const float *>(src + (int64_t) e * a.nb[0]), scale), mx));
            *reinterpret_cast<float *>(dst + (int64_t) e * d.nb[0]) = v;
        }
        // hsum of 8: (v0+v4, v1+v5, v2+v6, v3+v7) -> (r0+r2, r1+r3) -> s0+s1, evaluated on the group's lane 0
        const float r4 = __fadd_rn(__shfl_down_sync(0xffffffffu, v, 4), v);              // lanes 0..3 of a group: v[j+4] + v[j]
        const float r2 = __fadd_rn(r4, __shfl_down_sync(0xffffffffu, r4, 2));            // lanes 0,1: (r0+r2), (r1+r3)
        const float r1 = __fadd_rn(r2, __shfl_down_sync(0xffffffffu, r2, 1));            // lane 0: (r0+r2)+(r1+r3)
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const float gs = __shfl_sync(0xffffffffu, r1, 8 * g);
            if (base + 8 * g < n) sum += (double) gs;
        }
    }
    const float inv = (float) (1.0 / sum);
    __syncwarp();
    for (int e = lane; e < n; e += 32) {
        float * p = reinterpret_cast<float *>(dst + (int64_t) e * d.nb[0]);
        *p = __fmul_rn(*p, inv);
    }
}

// argsort of rows of n <= 1024 floats, descending, equal values in index order: rank by counting; one block per row
__global__ void __launch_bounds__(256) op_argsort_desc_kernel(TensorView a, TensorView d) {
    __shared__ float v[1024];
    const int64_t r = blockIdx.x;
    const int64_t i1 = r % a.ne[1], i2 = (r / a.ne[1]) % a.ne[2], i3 = r / (a.ne[1] * a.ne[2]);
    const char * src = a.data + view_offset(a, 0, i1, i2, i3);
    char * dst = d.data + view_offset(d, 0, i1, i2, i3);
    const int n = (int) a.ne[0];
    for (int i = threadIdx.x; i < n; i += blockDim.x) v[i] = *reinterpret_cast<const float *>(src + (int64_t) i * a.nb[0]);
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float x = v[i];
        int rank = 0;
        for (int j = 0; j < n; ++j) rank += (v[j] > x) || (v[j] == x && j < i);
        *reinterpret_cast<int32_t *>(dst + (int64_t) rank * d.nb[0]) = i;
    }
}

}  // namespace b200moe
