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
// block maximum (one value in 32) therefore needs recomputing only when something hangs on its last bits:
//   * amax / 127 lies within the error of a rounding boundary of fp16 (d in doubt): the mark kernel lists the candidates;
//   * a RECOMPUTED value still sits so close to an int8 rounding boundary that the maximum's own error decides it (a fifth of
//     the recomputed values - they were listed for being close): the fix kernel notices that itself and puts the block's
//     candidates on a second list, which a second pass of the same kernel recomputes.
// Blocks with neither keep the GEMM's maximum.  With the FP4 engine's margin under 1 % of the values are listed.
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
    // the maximum's candidates: when the block scale half(amax / 127) is in doubt (near an fp16 rounding boundary).  (A recomputed
    // value whose rounding hangs on the maximum's last bits is dealt with by the fix kernel.)
    const bool need_max = amax > 0.0f && near_half_rounding_boundary(amax / 127.0f, 2.0f * rel_margin);
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
    FixList more;              // candidates for block maxima found while fixing (items null: this is the second pass, find none)
    int * err;
    float rel_margin;          // the mark kernel's: relative uncertainty of a block maximum the GEMM left
};

// 8 lanes per listed value (the reference's 8 SIMD lanes), 4 values per warp at a time.  Each group runs the same chains as
// the integer GEMV, so the patched value is the reference's, bit for bit.  The listed values are scattered - nothing streams - so
// every warp fetches the two weight rows of its four values with bulk copies into its own piece of shared memory (whole rows in
// one request each instead of a few words per dependent load) and waits once; the activations are L2-resident and read directly.
// Latency is hidden by the other warps of the SM.
template <int K>
constexpr size_t requant_fix_smem_bytes() { return (size_t) 8 * 4 * 2 * (K / 64 * NVFP4_BLOCK_BYTES); }

template <int K>
__global__ void __launch_bounds__(256) requant_fix_kernel(const FixParams p) {
    constexpr int ROW_BYTES = K / 64 * NVFP4_BLOCK_BYTES;
    static_assert(ROW_BYTES % 16 == 0, "bulk copies move multiples of 16 bytes");
    extern __shared__ __align__(128) uint8_t fix_rows[];   // [8 warps][4 values][gate row, up row]
    __shared__ float ue_tab[256];
    __shared__ uint64_t bars[8];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = lane & 7, rgrp = lane >> 3;
    ue_tab[tid] = ue4m3_half_to_f32(tid);
    if (tid < 8) mbar_init(&bars[tid], 1);
    mbar_fence_init();
    __syncthreads();
    uint8_t * const rows_smem = fix_rows + (size_t) (warp * 4 + rgrp) * 2 * ROW_BYTES;
    const int n = min(*p.list.count, p.list.capacity);
    const int groups_per_grid = gridDim.x * 32;
    uint32_t parity = 0;
    // warp-uniform trip count: every lane runs the chains (their shuffles use the full mask); idle groups redo item 0
    for (int base = (blockIdx.x * 8 + warp) * 4; base < n; base += groups_per_grid) {
        const int i = base + rgrp;
        const bool valid = i < n;
        const int2 it = p.list.items[valid ? i : 0];
        const int r = it.x, f = it.y;
        int e = p.ids[r];
        if (e < 0 || e >= p.n_as) { report_error(p.err, DEV_ERR_BAD_EXPERT_ID); e = 0; }
        const int tok = r / p.n_ids;
        if (lane == 0) mbar_arrive_expect_tx(&bars[warp], 4 * 2 * ROW_BYTES);
        if (L == 0) {
            bulk_g2s(rows_smem, p.w0 + ((size_t) e * p.n_ff + f) * ROW_BYTES, ROW_BYTES, &bars[warp]);
            bulk_g2s(rows_smem + ROW_BYTES, p.w1 + ((size_t) e * p.n_ff + f) * ROW_BYTES, ROW_BYTES, &bars[warp]);
        }
        const bool landed = mbar_wait_bounded(&bars[warp], parity);
        if (!__all_sync(0xffffffffu, landed)) {                     // warp-uniform: the chains below shuffle with the full mask
            report_error(p.err, DEV_ERR_BARRIER_TIMEOUT);
            mbar_wait_bounded(&bars[warp], parity, 200000000ull);   // bounded drain before the shared memory goes away
            break;
        }
        parity ^= 1u;
        const uint8_t * g_row = rows_smem;
        const uint8_t * u_row = rows_smem + ROW_BYTES;
        float g[1], u[1];
        lane_chain_split_pair<K>(g_row, u_row, L, reinterpret_cast<const uint8_t *>(p.act.q + (size_t) tok * K), p.act.d + (size_t) tok * (K / 32), ue_tab,
                                 g[0], u[0]);
        const float sc0 = p.scale0 ? p.scale0[e] : 1.0f, sc1 = p.scale1 ? p.scale1[e] : 1.0f;
        const float hv = __fmul_rn(ggml_silu(__fmul_rn(g[0], sc0)), __fmul_rn(u[0], sc1));   // the same in all 8 lanes of the group
        float * hrow = p.hid + (size_t) r * p.n_ff;
        if (valid && L == 0) hrow[f] = hv;
        // Is the rounding of the exact value decided whatever the last bits of the block maximum are?  The group's 8 lanes read
        // the block (4 values each; values another group patches meanwhile are within the margin either way).  If not, the
        // candidates for the maximum go on the second list.
        if (p.more.items) {
            const int fb = f & ~31;
            const float4 nb = *reinterpret_cast<const float4 *>(hrow + fb + 4 * L);
            const float av[4] = { fabsf(nb.x), fabsf(nb.y), fabsf(nb.z), fabsf(nb.w) };
            float am = fmaxf(fmaxf(av[0], av[1]), fmaxf(av[2], av[3]));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
            am = fmaxf(am, fabsf(hv));
            if (valid && am > 0.0f) {
                const float t = fabsf(hv) * (127.0f / am);
                if (fabsf((t - floorf(t)) - 0.5f) < t * p.rel_margin + 2e-5f) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (av[j] >= am * (1.0f - p.rel_margin) && fb + 4 * L + j != f) {
                            const int slot = atomicAdd(p.more.count, 1);
                            if (slot < p.more.capacity) p.more.items[slot] = make_int2(r, fb + 4 * L + j);
                            else if (p.more.overflow) atomicAdd(p.more.overflow, 1ull);
                        }
                }
            }
        }
        __syncwarp();   // all lanes are done with the staged rows before the next round's copies land on them
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
    float rel_margin;          // as in FixParams
};

// One warp per listed value here (lane_chain_warp): the list of a dense product is short and its rows long (K up to 4096), so the
// kernel's time is one value's latency; with every load of the row in flight at once that is a few memory round trips.
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
        const uint8_t * q = reinterpret_cast<const uint8_t *>(p.act.q + (size_t) tok * K);
        const float * d = p.act.d + (size_t) tok * (K / 32);
        const float g = lane_chain_warp<K>(p.w + (size_t) f * ROW_BYTES, lane, q, d, ue_tab);
        const float yv = p.scale ? __fmul_rn(g, p.scale[0]) : g;
        float * yrow = p.y + (size_t) tok * p.n_out;
        if (lane == 0) yrow[f] = yv;
        // the block of 32 this value is quantised with: is its rounding decided whatever the last bits of the block maximum are?
        const int fb = f & ~31;
        const float mine = yrow[fb + lane];
        float am = fabsf(mine);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        am = fmaxf(am, fabsf(yv));
        if (am > 0.0f) {
            const float t = fabsf(yv) * (127.0f / am);
            if (fabsf((t - floorf(t)) - 0.5f) < t * p.rel_margin + 2e-5f) {
                // rare: recompute every candidate for the block maximum (warp-uniform: all lanes hold the same yv and am)
                uint32_t cands = __ballot_sync(0xffffffffu, fabsf(mine) >= am * (1.0f - p.rel_margin) && fb + lane != f);
                while (cands) {
                    const int c = __ffs(cands) - 1;
                    cands &= cands - 1;
                    const float gc = lane_chain_warp<K>(p.w + (size_t) (fb + c) * ROW_BYTES, lane, q, d, ue_tab);
                    if (lane == 0) yrow[fb + c] = p.scale ? __fmul_rn(gc, p.scale[0]) : gc;
                }
            }
        }
    }
}

}  // namespace b200moe
