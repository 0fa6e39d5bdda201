// Routing kernels: fp32 router GEMV in the reference's summation order, activation quantisers,
// softmax + top-k + renormalise, and grouping of routed rows by expert.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace b200moe {

// Activation rows quantised the way the reference CPU backend feeds its dot products
// (vec_dot_type of the weight type): Q8_0 for NVFP4 weights, Q8_K for Q3_K weights.
// Stored as separate planes so the GEMV kernels read them with aligned vector loads:
//   q      int8  [rows][K]
//   d      float [rows][K/32]   (Q8_0: float(half(amax/127)))   or  [rows][K/256] (Q8_K: 1/iscale)
//   bsum   int16 [rows][K/16]   (Q8_K only: sums of 16 quants, used for the -4 offset of Q3_K codes)
struct ActQuant {
    int8_t *  q;
    float *   d;
    int16_t * bsum;
};

// ---- K0: router logits (+ optional bias) --------------------------------------------------------
// One warp per (expert, tile of TT tokens).  Lane l owns the reference's SIMD chain l: AVX2
// ggml_vec_dot_f32 keeps 4 accumulators x 8 lanes, element i feeding accumulator (i/8)%4 lane i%8,
// i.e. chain i%32, with FMAs in increasing i.  The cross-chain reduction follows GGML_F32x8_REDUCE:
// (a0+a2),(a1+a3) -> sum -> lanes j+(j+4) -> two horizontal adds.
template <int TT, typename XT>
__global__ void __launch_bounds__(256) router_logits_kernel(const float * __restrict__ W, const float * __restrict__ bias,
                                                           const XT * __restrict__ x, float * __restrict__ logits, int H,
                                                           int E, int T, int * __restrict__ zero_buf, int zero_n) {
    pdl_wait();
    pdl_launch_dependents();

    // block 0 also clears the per-expert counters the selection kernel accumulates into
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < zero_n; i += blockDim.x) zero_buf[i] = 0;

    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int n_tt = (T + TT - 1) / TT;
    if (warp >= E * n_tt) return;
    const int e = warp % E;
    const int t0 = (warp / E) * TT;

    float acc[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) acc[i] = 0.0f;
    const float * w = W + (size_t) e * H;
    for (int j = lane; j < H; j += 32) {
        const float wv = __ldg(w + j);
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            const int t = min(t0 + i, T - 1);
            const float xv = (float) x[(size_t) t * H + j];
            acc[i] = __fmaf_rn(wv, xv, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < TT; ++i) {
        float v = acc[i];
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));  // a0+a2 (lanes 0-7), a1+a3 (lanes 8-15)
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));   // (a0+a2)+(a1+a3)
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));   // lane j + lane j+4
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));   // hadd
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));   // hadd
        if (lane == 0 && t0 + i < T) {
            if (bias) v = __fadd_rn(v, bias[e]);
            logits[(size_t) (t0 + i) * E + e] = v;
        }
    }
}

// Register-tiled form for batches: one warp per (TE experts x TT tokens).  Every (expert, token) pair still runs the reference's
// chains - lane l owns elements l, l + 32, ... in increasing order - but a weight value now meets TT tokens and an activation value
// TE experts per load, so the kernel is bound by FMAs instead of by re-reading x once per expert from L2.
template <int TE, int TT, typename XT>
__global__ void __launch_bounds__(256) router_logits_tiled_kernel(const float * __restrict__ W, const float * __restrict__ bias,
                                                                 const XT * __restrict__ x, float * __restrict__ logits, int H, int E, int T,
                                                                 int * __restrict__ zero_buf, int zero_n) {
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < zero_n; i += blockDim.x) zero_buf[i] = 0;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int n_te = (E + TE - 1) / TE, n_tt = (T + TT - 1) / TT;
    if (warp >= n_te * n_tt) return;
    const int e0 = (warp % n_te) * TE, t0 = (warp / n_te) * TT;
    float acc[TE][TT];
#pragma unroll
    for (int a = 0; a < TE; ++a)
#pragma unroll
        for (int b = 0; b < TT; ++b) acc[a][b] = 0.0f;
    const float * wrow[TE];
    const XT * xrow[TT];
#pragma unroll
    for (int a = 0; a < TE; ++a) wrow[a] = W + (size_t) min(e0 + a, E - 1) * H;
#pragma unroll
    for (int b = 0; b < TT; ++b) xrow[b] = x + (size_t) min(t0 + b, T - 1) * H;
#pragma unroll 2
    for (int j = lane; j < H; j += 32) {
        float wv[TE], xv[TT];
#pragma unroll
        for (int a = 0; a < TE; ++a) wv[a] = __ldg(wrow[a] + j);
#pragma unroll
        for (int b = 0; b < TT; ++b) xv[b] = (float) xrow[b][j];
#pragma unroll
        for (int a = 0; a < TE; ++a)
#pragma unroll
            for (int b = 0; b < TT; ++b) acc[a][b] = __fmaf_rn(wv[a], xv[b], acc[a][b]);
    }
#pragma unroll
    for (int a = 0; a < TE; ++a)
#pragma unroll
        for (int b = 0; b < TT; ++b) {
            float v = acc[a][b];
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
            if (lane == 0 && e0 + a < E && t0 + b < T) {
                if (bias) v = __fadd_rn(v, bias[e0 + a]);
                logits[(size_t) (t0 + b) * E + e0 + a] = v;
            }
        }
}

// Shared-memory form for larger batches: a block owns (8 WE experts) x (8 WT tokens); weight and activation rows arrive in
// 128-element pieces through a three-deep cp.async ring, and every warp runs an 8 x 8 register tile out of shared memory.  The
// chains are the reference's (lane l owns elements l, l + 32, ... in increasing order), so the logits keep its bits; what changes is
// that global loads are 16 bytes wide, issued two pieces ahead, and shared by the whole tile.
// Needs H to be a multiple of 128 and 16-byte aligned rows.
constexpr int ROUTER_KC = 128, ROUTER_ST = 3;
template <int WE, int WT, typename XT>
constexpr size_t router_smem_bytes() { return (size_t) ROUTER_ST * ROUTER_KC * (8 * WE * sizeof(float) + 8 * WT * sizeof(XT)); }

__device__ __forceinline__ void cp_async16(void * smem, const void * gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t) __cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int WE, int WT, typename XT>
__global__ void __launch_bounds__(WE * WT * 32) router_logits_smem_kernel(const float * __restrict__ W, const float * __restrict__ bias,
                                                                         const XT * __restrict__ x, float * __restrict__ logits, int H, int E, int T,
                                                                         int * __restrict__ zero_buf, int zero_n) {
    constexpr int EB = 8 * WE, TB = 8 * WT, KC = ROUTER_KC, ST = ROUTER_ST, NTHR = WE * WT * 32;
    constexpr int XP = 16 / sizeof(XT);   // activation elements per 16-byte piece
    extern __shared__ __align__(16) uint8_t router_smem[];
    float (*ws)[EB][KC] = reinterpret_cast<float (*)[EB][KC]>(router_smem);
    XT (*xs)[TB][KC] = reinterpret_cast<XT (*)[TB][KC]>(router_smem + (size_t) ST * EB * KC * sizeof(float));
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < zero_n; i += NTHR) zero_buf[i] = 0;
    const int n_eb = (E + EB - 1) / EB;
    const int e0 = (blockIdx.x % n_eb) * EB, t0 = (blockIdx.x / n_eb) * TB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int we = (warp % WE) * 8, wt = (warp / WE) * 8;
    const int n_chunks = H / KC;

    auto load_chunk = [&](int c) {
        const int s = c % ST;
        for (int i = threadIdx.x; i < EB * (KC / 4); i += NTHR) {
            const int r = i / (KC / 4), q = i % (KC / 4);
            cp_async16(&ws[s][r][q * 4], W + (size_t) min(e0 + r, E - 1) * H + (size_t) c * KC + q * 4);
        }
        for (int i = threadIdx.x; i < TB * (KC / XP); i += NTHR) {
            const int r = i / (KC / XP), q = i % (KC / XP);
            cp_async16(&xs[s][r][q * XP], x + (size_t) min(t0 + r, T - 1) * H + (size_t) c * KC + q * XP);
        }
    };
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = 0.0f;
#pragma unroll
    for (int c = 0; c < ST - 1; ++c) {
        if (c < n_chunks) load_chunk(c);
        cp_async_commit();
    }
    for (int c = 0; c < n_chunks; ++c) {
        cp_async_wait<ST - 2>();   // piece c has landed (one younger group may still be in flight)
        __syncthreads();           // ... for every thread, and everybody is done with the stage the next load overwrites
        if (c + ST - 1 < n_chunks) load_chunk(c + ST - 1);
        cp_async_commit();
        const int s = c % ST;
#pragma unroll
        for (int kk = 0; kk < KC / 32; ++kk) {
            float wv[8], xv[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) wv[a] = ws[s][we + a][kk * 32 + lane];
#pragma unroll
            for (int b = 0; b < 8; ++b) xv[b] = (float) xs[s][wt + b][kk * 32 + lane];
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int b = 0; b < 8; ++b) acc[a][b] = __fmaf_rn(wv[a], xv[b], acc[a][b]);
        }
    }
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            float v = acc[a][b];
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
            const int e = e0 + we + a, t = t0 + wt + b;
            if (lane == 0 && e < E && t < T) {
                if (bias) v = __fadd_rn(v, bias[e]);
                logits[(size_t) t * E + e] = v;
            }
        }
}

// ---- activation quantisers -------------------------------------------------------------------------
// Q8_0 as the reference's AVX2 quantize_row_q8_0 (ggml-cpu/arch/x86/quants.c:302-367): d = amax/127 kept
// as half, multiplier 127/amax in fp32, round to nearest even.  One warp per 32-element block... here one
// thread per element, a warp per block.
template <typename XT>
__device__ __forceinline__ void quantize_q8_0_block(const XT * __restrict__ src, int8_t * __restrict__ q, float * __restrict__ d,
                                                   int lane) {
    const float v = (float) src[lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float dd = __fdiv_rn(amax, 127.0f);
    const float id = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    q[lane] = (int8_t) __float2int_rn(__fmul_rn(v, id));
    if (lane == 0) *d = __half2float(__float2half_rn(dd));
}

// Q8_K as quantize_row_q8_K_ref (ggml-quants.c:2768-2805): the FIRST element with the largest |x| sets
// iscale = -127/x; q = min(127, nearest_int(iscale*x)); d = 1/iscale; bsums over 16.
// One warp per 256-element block, 8 elements per lane (lane owns elements 8*lane .. 8*lane+7).
template <typename XT>
__device__ __forceinline__ void quantize_q8_K_block(const XT * __restrict__ src, int8_t * __restrict__ q, float * __restrict__ d,
                                                   int16_t * __restrict__ bsum, int lane) {
    float v[8];
    float amax = 0.0f, mx = 0.0f;
    int arg = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[i] = (float) src[lane * 8 + i];
        const float a = fabsf(v[i]);
        if (a > amax) { amax = a; mx = v[i]; arg = lane * 8 + i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
        if (oa > amax || (oa == amax && oi < arg)) { amax = oa; mx = om; arg = oi; }
    }
    if (amax == 0.0f) {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[lane * 8 + i] = 0;
        if ((lane & 1) == 0) bsum[lane >> 1] = 0;
        if (lane == 0) *d = 0.0f;
        return;
    }
    const float iscale = __fdiv_rn(-127.0f, mx);
    int s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int qi = __float2int_rn(__fmul_rn(iscale, v[i]));
        qi = min(127, qi);
        q[lane * 8 + i] = (int8_t) qi;
        s += qi;
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    if ((lane & 1) == 0) bsum[lane >> 1] = (int16_t) s;
    if (lane == 0) *d = __fdiv_rn(1.0f, iscale);
}

// rows x K activations -> ActQuant planes.  kind: 0 = Q8_0 (32-blocks), 1 = Q8_K (256-blocks).
// src row r starts at src + r*src_stride.
template <typename XT>
__global__ void __launch_bounds__(256) quantize_act_kernel(const XT * __restrict__ src, int64_t src_stride, ActQuant dst, int rows,
                                                          int K, int kind) {
    pdl_wait();
    pdl_launch_dependents();

    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (kind == 0) {
        const int nb = K / 32;
        if (warp >= rows * nb) return;
        const int r = warp / nb, b = warp % nb;
        quantize_q8_0_block(src + (size_t) r * src_stride + b * 32, dst.q + (size_t) r * K + b * 32, dst.d + (size_t) r * nb + b, lane);
    } else {
        const int nb = K / 256;
        if (warp >= rows * nb) return;
        const int r = warp / nb, b = warp % nb;
        quantize_q8_K_block(src + (size_t) r * src_stride + b * 256, dst.q + (size_t) r * K + b * 256, dst.d + (size_t) r * nb + b,
                            dst.bsum + (size_t) r * (K / 16) + b * 16, lane);
    }
}

// Router logits and activation quantisation in one launch (decode path): blocks [0, n_logit_blocks) compute logits,
// the rest quantise x for the expert matmuls.  Both only read x.
template <int TT, typename XT>
__global__ void __launch_bounds__(256) route_front_kernel(const float * __restrict__ W, const float * __restrict__ bias,
                                                         const XT * __restrict__ x, float * __restrict__ logits, int H, int E, int T,
                                                         int * __restrict__ zero_buf, int zero_n, int n_logit_blocks, ActQuant dst,
                                                         int kind) {
    pdl_wait();
    pdl_launch_dependents();

    if ((int) blockIdx.x < n_logit_blocks) {
        if (blockIdx.x == 0)
            for (int i = threadIdx.x; i < zero_n; i += blockDim.x) zero_buf[i] = 0;
        const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
        const int lane = threadIdx.x & 31;
        const int n_tt = (T + TT - 1) / TT;
        if (warp >= E * n_tt) return;
        const int e = warp % E;
        const int t0 = (warp / E) * TT;
        float acc[TT];
#pragma unroll
        for (int i = 0; i < TT; ++i) acc[i] = 0.0f;
        const float * w = W + (size_t) e * H;
        // The FMA chain of a lane is sequential by definition of the reference's order, but its loads are not:
        // fetch CH steps of weights and activations at once, then run the chain over them.
        constexpr int CH = TT == 1 ? 32 : 8;
        for (int j0 = lane; j0 < H; j0 += 32 * CH) {
            float wv[CH], xv[TT][CH];
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int j = j0 + 32 * c;
                wv[c] = j < H ? __ldg(w + j) : 0.0f;
#pragma unroll
                for (int i = 0; i < TT; ++i) {
                    const int t = min(t0 + i, T - 1);
                    xv[i][c] = j < H ? (float) x[(size_t) t * H + j] : 0.0f;
                }
            }
#pragma unroll
            for (int c = 0; c < CH; ++c)
                if (j0 + 32 * c < H) {
#pragma unroll
                    for (int i = 0; i < TT; ++i) acc[i] = __fmaf_rn(wv[c], xv[i][c], acc[i]);
                }
        }
#pragma unroll
        for (int i = 0; i < TT; ++i) {
            float v = acc[i];
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
            if (lane == 0 && t0 + i < T) {
                if (bias) v = __fadd_rn(v, bias[e]);
                logits[(size_t) (t0 + i) * E + e] = v;
            }
        }
        return;
    }
    const int warp = (((int) blockIdx.x - n_logit_blocks) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (kind == 0) {
        const int nb = H / 32;
        if (warp >= T * nb) return;
        const int r = warp / nb, b = warp % nb;
        quantize_q8_0_block(x + (size_t) r * H + b * 32, dst.q + (size_t) r * H + b * 32, dst.d + (size_t) r * nb + b, lane);
    } else {
        const int nb = H / 256;
        if (warp >= T * nb) return;
        const int r = warp / nb, b = warp % nb;
        quantize_q8_K_block(x + (size_t) r * H + b * 256, dst.q + (size_t) r * H + b * 256, dst.d + (size_t) r * nb + b,
                            dst.bsum + (size_t) r * (H / 16) + b * 16, lane);
    }
}

// ---- K1: softmax + top-k + renormalise, one warp per token ---------------------------------------------
// soft_max (ggml-cpu/ops.cpp:5584-5694, vec.cpp:531-551): exp via ggml_v_expf, groups of 8 summed in fp32 as
// ((v0+v4)+(v2+v6))+((v1+v5)+(v3+v7)), groups accumulated in double, p = exp * (float)(1/sum).
// top-k = argsort descending, first k (ggml.c:5441-5455); equal values: lower index first.
// weights = p[ids] / max((float)sum_double(p[ids]), 2^-14) (forward.cpp:268-269).
// Also counts rows per expert and remembers each row's arrival position for the grouping kernel.
template <int EPL>  // experts per lane; E <= 32*EPL, E % 8 == 0
__device__ __forceinline__ void route_select_token(const float * __restrict__ logits, int E, int K, int t, int lane,
                                                   int32_t * __restrict__ ids, float * __restrict__ weights,
                                                   float * __restrict__ probs_out, int * __restrict__ counts,
                                                   int * __restrict__ pos) {
    const float * l = logits + (size_t) t * E;

    // lane owns experts e = lane*EPL + i  (contiguous, so a group of 8 experts sits in 8/EPL lanes or one lane)
    float p[EPL];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = lane * EPL + i;
        p[i] = e < E ? l[e] : -INFINITY;
        mx = fmaxf(mx, p[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int e = lane * EPL + i;
        p[i] = e < E ? ggml_expf(__fsub_rn(p[i], mx)) : 0.0f;
    }
    // group-of-8 sums in the reference's order, then the double accumulation over groups in index order
    double sum = 0.0;
    for (int g = 0; g < E / 8; ++g) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int e = g * 8 + j;
            const int owner = e / EPL, slot = e % EPL;
            float val = 0.0f;
#pragma unroll
            for (int i = 0; i < EPL; ++i)
                if (i == slot) val = p[i];
            v[j] = __shfl_sync(0xffffffffu, val, owner);
        }
        const float r0 = __fadd_rn(v[4], v[0]), r1 = __fadd_rn(v[5], v[1]), r2 = __fadd_rn(v[6], v[2]), r3 = __fadd_rn(v[7], v[3]);
        sum += (double) __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
    }
    const float inv = (float) (1.0 / sum);
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        p[i] = __fmul_rn(p[i], inv);
        const int e = lane * EPL + i;
        if (probs_out && e < E) probs_out[(size_t) t * E + e] = p[i];
    }

    // iterative arg-max, K rounds; ties -> lower expert index
    float sel_p = 0.0f;
    int sel_e = -1;
    double wsum = 0.0;
    uint32_t taken = 0;  // bit i: p[i] already selected
    for (int k = 0; k < K; ++k) {
        float best = -1.0f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = lane * EPL + i;
            if (e < E && !((taken >> i) & 1u) && p[i] > best) { best = p[i]; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (best_e / EPL == lane) taken |= 1u << (best_e % EPL);
        if (lane == k) { sel_p = best; sel_e = best_e; }
        wsum += (double) best;  // sum_rows accumulates in double in slot order (ggml-cpu/vec.h:1495-1505)
    }
    float den = (float) wsum;
    den = fmaxf(den, 6.103515625e-5f);
    if (lane < K) {
        // NaN logits leave no candidate; keep the index in range so nothing downstream is addressed with it
        sel_e = sel_e < 0 ? 0 : (sel_e >= E ? E - 1 : sel_e);
        ids[(size_t) t * K + lane] = sel_e;
        weights[(size_t) t * K + lane] = __fdiv_rn(sel_p, den);
        if (counts) pos[(size_t) t * K + lane] = atomicAdd(&counts[sel_e], 1);
    }
}

template <int EPL>
__global__ void __launch_bounds__(256) route_select_kernel(const float * __restrict__ logits, int E, int K, int T,
                                                          int32_t * __restrict__ ids, float * __restrict__ weights,
                                                          float * __restrict__ probs_out, int * __restrict__ counts,
                                                          int * __restrict__ pos) {
    pdl_wait();
    pdl_launch_dependents();

    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (t >= T) return;
    route_select_token<EPL>(logits, E, K, t, threadIdx.x & 31, ids, weights, probs_out, counts, pos);
}

// ---- K2: grouping ----------------------------------------------------------------------------------------
// Group descriptor produced for the expert kernels (reference: matrix_rows / matrix_row_counts in
// ggml_compute_forward_mul_mat_id, ggml-cpu/ggml-cpu.c:1648-1663):
//   offsets[e]   first slot of expert e in perm, offsets[E] = total rows
//   perm[i]      routed row index (token*K + slot) placed i-th
//   active[a]    a-th expert that has at least one row; n_active in meta[0], total rows in meta[1]
constexpr int TOKEN_TILE_ROWS = 14;   // routed rows per token tile of the FP4 tensor-core kernels (7 digit planes each)

struct Groups {
    int * counts;   // [E]
    int * offsets;  // [E+1]
    int * pos;      // [rows]
    int * perm;     // [rows]
    int * active;   // [E]
    int * meta;     // [4]
    int * cost;     // [4][E+1]: rows 0-2: prefix over active experts of the work per weight row for the nt = 1, 2, 4 kernels;
                    // row 3, indexed by EXPERT id: index of the expert's first token tile (prefix of ceil(rows / TOKEN_TILE_ROWS))
};

// Block-wide: counts must be final and visible to this block.
// allow_empty: ids equal to -1 mark routed rows that do not exist (empty slots of an expert-parallel exchange): they are in no group.
__device__ __forceinline__ void group_scan_body(Groups g, const int32_t * __restrict__ ids, int E, int rows, int * err, int * sh, bool allow_empty = false) {
    int * off = sh;
    int * act = sh + (E + 1);  // act[a] = a-th active expert (also written to g.active)
    int * cnt = sh + (2 * E + 1);  // counts, fetched by the whole block at once (the scan below would wait for memory 32 at a time)
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) cnt[e] = g.counts[e];
    __syncthreads();
    if (tid < 32) {
        // warp 0: exclusive scan of counts, compaction of active experts and the three work prefixes, 32 experts a step
        int run = 0, na = 0, c1 = 0, c2 = 0, c4 = 0, tl = 0;
        for (int base = 0; base < E; base += 32) {
            const int e = base + tid;
            const int n = e < E ? cnt[e] : 0;
            // work per weight row: nt=1 kernels: one pass per routed row; nt=4 kernels: 3 per pass (decode) + 2 per routed row
            int incl = n, w2 = (n + 1) / 2, w4 = 3 * ((n + 3) / 4) + 2 * n;
            int i2 = w2, i4 = w4, it = (n + TOKEN_TILE_ROWS - 1) / TOKEN_TILE_ROWS;
            const int wt = it;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int a = __shfl_up_sync(0xffffffffu, incl, o), b = __shfl_up_sync(0xffffffffu, i2, o), c = __shfl_up_sync(0xffffffffu, i4, o);
                const int d = __shfl_up_sync(0xffffffffu, it, o);
                if (tid >= o) { incl += a; i2 += b; i4 += c; it += d; }
            }
            if (e < E) { off[e] = run + incl - n; g.cost[3 * (E + 1) + e] = tl + it - wt; }
            const unsigned m = __ballot_sync(0xffffffffu, n > 0);
            if (n > 0) {
                const int a = na + __popc(m & ((1u << tid) - 1));
                act[a] = e;
                g.active[a] = e;
                g.cost[a] = c1 + incl - n;
                g.cost[(E + 1) + a] = c2 + i2 - w2;
                g.cost[2 * (E + 1) + a] = c4 + i4 - w4;
            }
            run += __shfl_sync(0xffffffffu, incl, 31);
            c1 += __shfl_sync(0xffffffffu, incl, 31);
            c2 += __shfl_sync(0xffffffffu, i2, 31);
            c4 += __shfl_sync(0xffffffffu, i4, 31);
            tl += __shfl_sync(0xffffffffu, it, 31);
            na += __popc(m);
        }
        if (tid == 0) {
            off[E] = run;
            g.cost[na] = c1; g.cost[(E + 1) + na] = c2; g.cost[2 * (E + 1) + na] = c4; g.cost[3 * (E + 1) + E] = tl;
            g.meta[0] = na;
            g.meta[1] = run;
            if (allow_empty ? run > rows : run != rows) report_error(err, DEV_ERR_BAD_SHAPE);
        }
    }
    __syncthreads();
    for (int e = tid; e <= E; e += blockDim.x) g.offsets[e] = off[e];
    for (int r = tid; r < rows; r += blockDim.x) {
        const int e = ids[r];
        if (allow_empty && e == -1) continue;
        if (e < 0 || e >= E) { report_error(err, DEV_ERR_BAD_EXPERT_ID); continue; }
        g.perm[off[e] + g.pos[r]] = r;
    }
}

// The grouping of a dense product: every one of the T rows belongs to the single group 0 (one launch instead of the
// count / scan pair; same tables as group_scan_body leaves for E = 1).
__global__ void __launch_bounds__(256) one_group_kernel(Groups g, int32_t * __restrict__ ids, int T) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T) { ids[t] = 0; g.perm[t] = t; }
    if (t == 0) {
        g.counts[0] = T;
        g.offsets[0] = 0; g.offsets[1] = T;
        g.active[0] = 0;
        g.meta[0] = 1; g.meta[1] = T;
        g.cost[0] = 0; g.cost[1] = T;
        g.cost[2] = 0; g.cost[3] = (T + 1) / 2;
        g.cost[4] = 0; g.cost[5] = 3 * ((T + 3) / 4) + 2 * T;
        g.cost[6] = 0; g.cost[7] = (T + TOKEN_TILE_ROWS - 1) / TOKEN_TILE_ROWS;
    }
}

// Single block.  counts must be final (selection kernel finished).
__global__ void __launch_bounds__(1024) group_scan_kernel(Groups g, const int32_t * __restrict__ ids, int E, int rows, int * err, int allow_empty) {
    pdl_wait();
    pdl_launch_dependents();

    extern __shared__ int sh[];  // [E+1] offsets, [E] active experts, [E] counts
    group_scan_body(g, ids, E, rows, err, sh, allow_empty != 0);
}

// Small batches: selection for every token and the grouping in ONE single-block launch (one warp per token, looping).
template <int EPL>
__global__ void __launch_bounds__(1024) route_select_group_kernel(const float * __restrict__ logits, int E, int K, int T,
                                                                 int32_t * __restrict__ ids, float * __restrict__ weights,
                                                                 float * __restrict__ probs_out, Groups g, int * err) {
    pdl_wait();
    pdl_launch_dependents();

    extern __shared__ int sh[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int t = warp; t < T; t += nw) route_select_token<EPL>(logits, E, K, t, lane, ids, weights, probs_out, g.counts, g.pos);
    __syncthreads();  // global writes of this block (counts, pos, ids) are visible to the whole block afterwards
    group_scan_body(g, ids, E, T * K, err, sh);
}

// Counting pass for routing that was not produced by route_select_kernel (ids given by the caller,
// possibly as a strided view: row t starts at ids + t*ids_stride).  Writes compact ids as well.
__global__ void __launch_bounds__(256) count_ids_kernel(const int32_t * __restrict__ ids, int64_t ids_stride, int n_ids, int T, int E,
                                                       int32_t * __restrict__ ids_compact, int * __restrict__ counts,
                                                       int * __restrict__ pos, int * err, int allow_empty = 0) {
    pdl_wait();
    pdl_launch_dependents();

    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_ids * T) return;
    const int t = r / n_ids, s = r % n_ids;
    const int e = ids[(size_t) t * ids_stride + s];
    ids_compact[r] = e;
    if (allow_empty && e == -1) { pos[r] = 0; return; }
    if (e < 0 || e >= E) { report_error(err, DEV_ERR_BAD_EXPERT_ID); pos[r] = 0; return; }
    pos[r] = atomicAdd(&counts[e], 1);
}

}  // namespace b200moe
