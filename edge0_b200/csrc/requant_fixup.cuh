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

// One warp per (routed row, 128 features): a lane holds four neighbouring values, eight lanes one block of 32.
//   step_margin : distance from a rounding boundary, in quantisation steps, below which a value is recomputed
//   rel_margin  : relative distance from the block maximum below which a value counts as a candidate for it; the same
//                 relative uncertainty of the scale widens the step margin of large values
//   perm        : routed rows sorted by expert.  Warps walk (feature chunk, sorted row) with the row fastest, so values that need
//                 the same weight rows (same expert, same features) are listed next to each other and the recomputation
//                 finds those rows in cache instead of fetching 2 x row_bytes from HBM per value.
//   meta[1]     : number of routed rows that are in a group (fewer than `rows` when an exchange left slots empty)
// n_ff must be a multiple of 128 and the rows 16-byte aligned.
__global__ void __launch_bounds__(256) requant_mark_kernel(const float * __restrict__ hid, const int * __restrict__ perm, const int * __restrict__ meta,
                                                          int rows, int n_ff, float step_margin, float rel_margin, FixList list) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int chunks = n_ff / 128;
    if (warp >= rows * chunks || warp % rows >= meta[1]) return;
    const int c = warp / rows, r = perm[warp % rows];
    const int f0 = c * 128 + lane * 4;
    const float4 v4 = *reinterpret_cast<const float4 *>(hid + (size_t) r * n_ff + f0);
    const float a[4] = { fabsf(v4.x), fabsf(v4.y), fabsf(v4.z), fabsf(v4.w) };
    float amax = fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // the block's eight lanes
    bool risky[4] = { false, false, false, false };
    if (amax > 0.0f) {
        const float id = 127.0f / amax;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float t = a[j] * id;                                // 0 .. 127
            const float dist = fabsf((t - floorf(t)) - 0.5f);         // distance from the rounding boundary, in steps
            risky[j] = dist < step_margin + t * rel_margin;
        }
    }
    // the maximum's candidates: when the block scale half(amax / 127) is in doubt (near an fp16 rounding boundary), or when a value of
    // the block is recomputed (its rounding is only decided against the exact maximum)
    const uint32_t any = __ballot_sync(0xffffffffu, risky[0] || risky[1] || risky[2] || risky[3]);
    const bool block_any = ((any >> (lane & 24)) & 0xffu) != 0;
    const bool need_max = block_any || (amax > 0.0f && near_half_rounding_boundary(amax / 127.0f, 2.0f * rel_margin));
    int n_mine = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        risky[j] = risky[j] || (need_max && amax > 0.0f && a[j] >= amax * (1.0f - rel_margin));
        n_mine += risky[j] ? 1 : 0;
    }
    int incl = n_mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (total == 0) return;
    int base = 0;
    if (lane == 0) {
        base = atomicAdd(list.count, total);
        const int over = base + total - max(base, list.capacity);
        if (over > 0 && list.overflow) atomicAdd(list.overflow, (unsigned long long) over);
    }
    base = __shfl_sync(0xffffffffu, base, 0);
    int slot = base + incl - n_mine;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (risky[j]) {
            if (slot < list.capacity) list.items[slot] = make_int2(r, f0 + j);
            ++slot;
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

// One warp per listed value (lane_chain_warp): the reference's 8 SIMD lanes run the fp32 chain, all 32 lanes fetch and decode, so
// every load of a value is in flight at once and the kernel's time is a few memory round trips, not one per group of blocks.
// The patched value is the reference's, bit for bit; weight rows and activations are read straight from global memory (the
// activations and most weight rows are L2-resident right after the GEMM) - the listed values are scattered, there is nothing to
// stream.
template <int K>
__global__ void __launch_bounds__(256) requant_fix_kernel(const FixParams p) {
    constexpr int ROW_BYTES = K / 64 * NVFP4_BLOCK_BYTES;
    __shared__ float ue_tab[256];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    ue_tab[tid] = ue4m3_half_to_f32(tid);
    __syncthreads();
    const int n = min(*p.list.count, p.list.capacity);
    for (int i = blockIdx.x * 8 + warp; i < n; i += gridDim.x * 8) {
        const int2 it = p.list.items[i];
        const int r = it.x, f = it.y;
        int e = p.ids[r];
        if (e < 0 || e >= p.n_as) { report_error(p.err, DEV_ERR_BAD_EXPERT_ID); e = 0; }
        const int tok = r / p.n_ids;
        const uint8_t * q = reinterpret_cast<const uint8_t *>(p.act.q + (size_t) tok * K);
        const float * d = p.act.d + (size_t) tok * (K / 32);
        const float g = lane_chain_warp<K>(p.w0 + ((size_t) e * p.n_ff + f) * ROW_BYTES, lane, q, d, ue_tab);
        const float u = lane_chain_warp<K>(p.w1 + ((size_t) e * p.n_ff + f) * ROW_BYTES, lane, q, d, ue_tab);
        if (lane == 0) {
            const float sc0 = p.scale0 ? p.scale0[e] : 1.0f, sc1 = p.scale1 ? p.scale1[e] : 1.0f;
            const float v = __fmul_rn(g, sc0);
            p.hid[(size_t) r * p.n_ff + f] = __fmul_rn(ggml_silu(v), __fmul_rn(u, sc1));
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
    ue_tab[tid] = ue4m3_half_to_f32(tid);
    __syncthreads();
    const int n = min(*p.list.count, p.list.capacity);
    for (int i = blockIdx.x * 8 + warp; i < n; i += gridDim.x * 8) {
        const int2 it = p.list.items[i];
        const int tok = it.x, f = it.y;
        const float g = lane_chain_warp<K>(p.w + (size_t) f * ROW_BYTES, lane, reinterpret_cast<const uint8_t *>(p.act.q + (size_t) tok * K),
                                           p.act.d + (size_t) tok * (K / 32), ue_tab);
        if (lane == 0) p.y[(size_t) tok * p.n_out + f] = p.scale ? __fmul_rn(g, p.scale[0]) : g;
    }
}

}  // namespace b200moe
