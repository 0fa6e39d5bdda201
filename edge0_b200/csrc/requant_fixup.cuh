// Exact re-quantisation behind the tensor-core gate/up GEMM.
//
// The reference quantises `hidden` to Q8_0 before the down projection: per block of 32, d = amax / 127 and
// q = round(h * 127 / amax).  The tensor-core GEMM returns h with a small error (its fp32 accumulation aligns products
// to ~15 bits); almost every q is unaffected, but a value that sits within that error of a rounding boundary - or of its
// block's maximum, which sets the scale of all 32 - can flip, and the reference's own arithmetic amplifies one flipped
// int8 into ~1e-2 of the output RMS.  Instead of bounding the tail, remove it:
//   1. requant_mark_kernel   lists every (routed row, feature) whose rounding is not decided by a safe margin, and the
//                            candidates for a block's maximum when the block scale itself is not decided by that margin;
//   2. requant_fix_kernel    recomputes exactly those values with the integer lane chains of expert_gemv.cuh (the
//                            reference's own summation order) and patches `hidden`;
//   3. the ordinary quantiser then sees exact values wherever the outcome depends on them, so the int8 `hidden` - and with
//      the integer down kernel the whole layer - is the reference's, bit for bit, as long as the GEMM's error stays
//      inside the margin (a few per cent of the values are recomputed; the margin is ~10x the largest error measured).
// What has to be exact is the QUANTISED block, not the fp32 values: q = round(h * 127 / amax) and d = half(amax / 127).  The
// block maximum (one value in 32) therefore needs recomputing only when something hangs on its last bits: when amax / 127 lies
// within the error of a rounding boundary of fp16 (d in doubt), or when some value of the block sits close to an int8 rounding
// boundary (a recomputed value that close is only decided once amax is exact too).  Blocks with neither keep the GEMM's maximum.
// With the FP4 engine's margin about 1.3 % of the values are listed, with the f16 engine's about 6 %.
// The list holds a quarter of all values; when more are marked (degenerate inputs such as blocks of equal values), the surplus
// stays as the GEMM produced it and the overflow is counted (FixList::overflow, reported through b200moe_get_counters).
#pragma once
#include "expert_gemv.cuh"

namespace b200moe {

struct FixList {
    int2 * items;      // (routed row, feature)
    int * count;       // number of items marked; items beyond `capacity` were not stored
    int capacity;
    unsigned long long * overflow;   // running total of marked items that did not fit (or null)
};

// Is x > 0 within a relative distance rel of a point where rounding to fp16 changes its result (the midpoint between two
// neighbouring fp16 numbers)?
__device__ __forceinline__ bool near_half_rounding_boundary(float x, float rel) {
    const float lo = __half2float(__float2half_rd(x)), hi = __half2float(__float2half_ru(x));
    if (lo == hi) return false;                     // exactly representable: half a spacing away from both midpoints
    return fabsf(x - 0.5f * (lo + hi)) <= rel * x;
}

// One warp per (routed row, block of 32 features).
//   step_margin : distance from a rounding boundary, in quantisation steps, below which a value is recomputed
//   rel_margin  : relative distance from the block maximum below which a value counts as a candidate for it; the same
//                 relative uncertainty of the scale widens the step margin of large values
//   perm        : routed rows sorted by expert.  Warps walk (feature block, sorted row) with the row fastest, so values that need
//                 the same weight rows (same expert, same 32 features) are listed next to each other and the recomputation
//                 finds those rows in cache instead of fetching 2 x row_bytes from HBM per value.
//   meta[1]     : number of routed rows that are in a group (fewer than `rows` when an exchange left slots empty)
__global__ void __launch_bounds__(256) requant_mark_kernel(const float * __restrict__ hid, const int * __restrict__ perm, const int * __restrict__ meta,
                                                          int rows, int n_ff, float step_margin, float rel_margin, FixList list) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int nb = n_ff / 32;
    if (warp >= rows * nb || warp % rows >= meta[1]) return;
    const int b = warp / rows, r = perm[warp % rows];
    const float v = hid[(size_t) r * n_ff + b * 32 + lane];
    const float a = fabsf(v);
    float amax = a;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bool risky = false;
    if (amax > 0.0f) {
        const float id = 127.0f / amax;
        const float t = a * id;                                   // 0 .. 127
        const float dist = fabsf((t - floorf(t)) - 0.5f);         // distance from the rounding boundary, in steps
        // the block scale half(amax / 127) is in doubt only near an fp16 rounding boundary: then every candidate for the maximum counts
        risky = dist < step_margin + t * rel_margin;
    }
    // the maximum's candidates: when the block scale is in doubt, or when a value of the block is recomputed (its rounding is only
    // decided against the exact maximum)
    const bool need_max = __any_sync(0xffffffffu, risky) || (amax > 0.0f && near_half_rounding_boundary(amax / 127.0f, 2.0f * rel_margin));
    risky = risky || (need_max && amax > 0.0f && a >= amax * (1.0f - rel_margin));
    const uint32_t m = __ballot_sync(0xffffffffu, risky);
    if (m == 0) return;
    int base = 0;
    if (lane == 0) {
        base = atomicAdd(list.count, __popc(m));
        const int over = base + __popc(m) - max(base, list.capacity);
        if (over > 0 && list.overflow) atomicAdd(list.overflow, (unsigned long long) over);
    }
    base = __shfl_sync(0xffffffffu, base, 0);
    if (risky) {
        const int slot = base + __popc(m & ((1u << lane) - 1));
        if (slot < list.capacity) list.items[slot] = make_int2(r, b * 32 + lane);
    }
}

struct FixParams {
    const uint8_t * w0;        // gate [n_as][n_ff][row_bytes]
    const uint8_t * w1;        // up
    const float * scale0;
    const float * scale1;
    ActQuant act;              // quantised activations of the tokens: q [tokens][K], d [tokens][K/32]
    const int32_t * ids;       // expert of every routed row
    int n_ids;                 // routed rows per token (activation row of routed row r is r / n_ids)
    int n_ff;
    int n_as;
    float * hid;               // [rows][n_ff], patched in place
    FixList list;
    int * err;
};

// 8 lanes per listed value (the reference's 8 SIMD lanes), 4 values per warp at a time.  Each group runs the same chains as
// the integer GEMV, so the patched value is the reference's, bit for bit; weight rows and activations are read straight from
// global memory (the activations and most weight rows are L2-resident right after the GEMM), and latency is hidden by
// occupancy instead of a staging ring - the listed values are scattered, there is nothing to stream.
template <int K>
__global__ void __launch_bounds__(256) requant_fix_kernel(const FixParams p) {
    constexpr int ROW_BYTES = K / 64 * NVFP4_BLOCK_BYTES;
    __shared__ float ue_tab[256];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = lane & 7, rgrp = lane >> 3;
    ue_tab[tid] = ue4m3_half_to_f32(tid);
    __syncthreads();
    const int n = min(*p.list.count, p.list.capacity);
    const int groups_per_grid = gridDim.x * 32;
    // warp-uniform trip count: every lane runs the chains (their shuffles use the full mask); idle groups redo item 0
    for (int base = (blockIdx.x * 8 + warp) * 4; base < n; base += groups_per_grid) {
        const int i = base + rgrp;
        const bool valid = i < n;
        const int2 it = p.list.items[valid ? i : 0];
        const int r = it.x, f = it.y;
        int e = p.ids[r];
        if (e < 0 || e >= p.n_as) { report_error(p.err, DEV_ERR_BAD_EXPERT_ID); e = 0; }
        const int tok = r / p.n_ids;
        const uint8_t * g_row = p.w0 + ((size_t) e * p.n_ff + f) * ROW_BYTES;
        const uint8_t * u_row = p.w1 + ((size_t) e * p.n_ff + f) * ROW_BYTES;
        float g[1], u[1];
        lane_chain_split<K>(g_row, L, reinterpret_cast<const uint8_t *>(p.act.q + (size_t) tok * K), p.act.d + (size_t) tok * (K / 32), ue_tab, g);
        lane_chain_split<K>(u_row, L, reinterpret_cast<const uint8_t *>(p.act.q + (size_t) tok * K), p.act.d + (size_t) tok * (K / 32), ue_tab, u);
        if (valid && L == 0) {
            const float sc0 = p.scale0 ? p.scale0[e] : 1.0f, sc1 = p.scale1 ? p.scale1[e] : 1.0f;
            const float v = __fmul_rn(g[0], sc0);
            p.hid[(size_t) r * p.n_ff + f] = __fmul_rn(ggml_silu(v), __fmul_rn(u[0], sc1));
        }
    }
}

// The same for ONE dense matrix (a latent projection whose result is re-quantised): listed value (token, feature) =
// round_fp32(dot(W[feature], x_hat[token]) * scale), the arithmetic of the integer matvec followed by its scale pass.
struct FixSingleParams {
    const uint8_t * w;         // [n_out][row_bytes]
    const float * scale;       // one value or null
    ActQuant act;              // q [tokens][K], d [tokens][K/32]
    int n_out;
    float * y;                 // [tokens][n_out], patched in place
    FixList list;
};

template <int K>
__global__ void __launch_bounds__(256) requant_fix_single_kernel(const FixSingleParams p) {
    constexpr int ROW_BYTES = K / 64 * NVFP4_BLOCK_BYTES;
    __shared__ float ue_tab[256];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = lane & 7, rgrp = lane >> 3;
    ue_tab[tid] = ue4m3_half_to_f32(tid);
    __syncthreads();
    const int n = min(*p.list.count, p.list.capacity);
    const int groups_per_grid = gridDim.x * 32;
    for (int base = (blockIdx.x * 8 + warp) * 4; base < n; base += groups_per_grid) {
        const int i = base + rgrp;
        const bool valid = i < n;
        const int2 it = p.list.items[valid ? i : 0];
        const int tok = it.x, f = it.y;
        float g[1];
        lane_chain_split<K>(p.w + (size_t) f * ROW_BYTES, L, reinterpret_cast<const uint8_t *>(p.act.q + (size_t) tok * K), p.act.d + (size_t) tok * (K / 32),
                            ue_tab, g);
        if (valid && L == 0) p.y[(size_t) tok * p.n_out + f] = p.scale ? __fmul_rn(g[0], p.scale[0]) : g[0];
    }
}

}  // namespace b200moe
