// Grouped expert GEMV for decode / batched decode: streams only the routed experts' quantised rows
// from HBM through a shared-memory ring filled by 1-D bulk async copies (TMA), decodes in registers,
// integer dot products against the int8 activation grid of the reference, warp-shuffle reductions.
//
// One kernel template serves
//   DUAL = true : gate and up projections of the same rows + SwiGLU epilogue  -> hidden[row][n_out]
//   DUAL = false: one indexed matmul (ggml MUL_MAT_ID semantics)               -> dst[row][n_out]
// "row" is a routed row: token*n_ids + slot.
//
// Work distribution: the rows of all active experts form one flat list (active expert a, output row r);
// every CTA of the persistent grid takes an equal contiguous span of it, so HBM bytes per SM are equal
// whatever the routing looks like.  A span is walked in chunks of at most ROWS_PER_STAGE rows of one
// expert; chunk c lives in ring stage c % STAGES.
#pragma once
#include "common.cuh"
#include "formats.cuh"
#include "router.cuh"

namespace b200moe {

struct GemvParams {
    const uint8_t * w0;   // DUAL: gate experts; else the expert tensor  [n_as][n_out][row_bytes]
    const uint8_t * w1;   // DUAL: up experts
    const float * scale0; // per-expert fp32 scale applied to w0's result (or null)
    const float * scale1;
    ActQuant act;         // quantised activation planes, row index = (row / n_ids) * ne11 + (row % n_ids) % ne11
    const int * offsets;  // [n_as + 1]
    const int * perm;     // [rows]
    const int * active;   // [n_as]
    const int * meta;     // meta[0] = number of active experts
    const int * cost;     // [3][n_as+1] work prefixes (see Groups::cost)
    float * out;          // [rows][n_out]
    int n_out;
    int n_ids;
    int ne11;
    int n_as;
    int * err;
};

template <int WT, int K>
struct GemvCfg {
    static constexpr int UNITS = K / 32;
    static constexpr int LPR = (UNITS % 32 == 0) ? 32 : (UNITS % 16 == 0) ? 16 : (UNITS % 8 == 0) ? 8 : 0;  // lanes per row
    static_assert(LPR != 0, "K must be a multiple of 256");
    static constexpr int UPL = UNITS / LPR;  // units per lane
    static constexpr int RPP = 32 / LPR;     // rows per warp pass
    static constexpr int ROW_BYTES = WT == TYPE_NVFP4 ? K / 64 * 36 : K / 256 * 110;
    static constexpr int GRAN = (ROW_BYTES % 16 == 0) ? 1 : 8;  // span granularity in rows (16-byte rule of bulk copies)
    static constexpr int NWARPS = 16;
    // passes per warp per stage chosen so a (single-tensor) stage is roughly 16-32 KB
    static constexpr int PASSES = (ROW_BYTES * RPP * NWARPS >= 12288) ? 1 : (ROW_BYTES * RPP * NWARPS >= 6144) ? 2 : 4;
    static constexpr int ROWS_PER_STAGE = NWARPS * RPP * PASSES;
    static constexpr int TENSOR_STAGE_BYTES = ROWS_PER_STAGE * ROW_BYTES;
    static_assert(TENSOR_STAGE_BYTES % 16 == 0, "stage must keep 16-byte alignment");
    static_assert(WT != TYPE_Q3_K || UPL <= 4, "unsupported width");
};

// ---- per-token activation registers of one lane --------------------------------------------------------
template <int WT, int UPL>
struct LaneAct {
    uint32_t q[UPL][8];  // NVFP4: permuted to the decode order; Q3_K: natural order
    float d[UPL];        // NVFP4: Q8_0 block scale; Q3_K: Q8_K super-block scale
    int bs[UPL];         // Q3_K: bsums of sub-blocks 2p, 2p+1 packed as two int16
};

template <int WT, int K>
__device__ __forceinline__ void load_lane_act(LaneAct<WT, GemvCfg<WT, K>::UPL> & a, const ActQuant & act, int act_row, int lir, bool valid) {
    using C = GemvCfg<WT, K>;
#pragma unroll
    for (int i = 0; i < C::UPL; ++i) {
        const int u = i * C::LPR + lir;  // units of a lane are strided by LPR: neighbouring lanes read neighbouring units
        uint32_t w[8];
        if (valid) {
            const int4 * src = reinterpret_cast<const int4 *>(act.q + (size_t) act_row * K + u * 32);
            const int4 v0 = __ldg(src), v1 = __ldg(src + 1);
            w[0] = v0.x; w[1] = v0.y; w[2] = v0.z; w[3] = v0.w; w[4] = v1.x; w[5] = v1.y; w[6] = v1.z; w[7] = v1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = 0;
        }
        if (WT == TYPE_NVFP4) {
            fp4_permute_act16(&w[0], &a.q[i][0]);
            fp4_permute_act16(&w[4], &a.q[i][4]);
            a.d[i] = valid ? __ldg(act.d + (size_t) act_row * (K / 32) + u) : 0.0f;
            a.bs[i] = 0;
        } else {
            // Q3_K unit (sb, p): needs elements 128*j + 32*s + 4p..4p+3 of super-block sb -> that is one word out
            // of each 32-element group; they are NOT contiguous, so fetch them individually.
            const int sb = u >> 3, p = u & 7;
            const int8_t * base = act.q + (size_t) act_row * K + sb * 256 + 4 * p;
#pragma unroll
            for (int j = 0; j < 8; ++j) a.q[i][j] = valid ? __ldg(reinterpret_cast<const uint32_t *>(base + 32 * j)) : 0u;
            a.d[i] = valid ? __ldg(act.d + (size_t) act_row * (K / 256) + sb) : 0.0f;
            a.bs[i] = valid ? __ldg(reinterpret_cast<const int *>(act.bsum + (size_t) act_row * (K / 16) + sb * 16 + 2 * p)) : 0;
        }
    }
}

__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t * p) {  // 2-byte aligned 32-bit load from shared memory
    const uint16_t * h = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t) h[0] | ((uint32_t) h[1] << 16);
}

// Lane-partial dot products of one weight row against NT tokens.
template <int WT, int K, int NT>
__device__ __forceinline__ void row_partial(const uint8_t * __restrict__ row, int lir, const LaneAct<WT, GemvCfg<WT, K>::UPL> (&acts)[NT],
                                            const float * __restrict__ ue_tab, float (&acc)[NT]) {
    using C = GemvCfg<WT, K>;
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.0f;
#pragma unroll
    for (int i = 0; i < C::UPL; ++i) {
        const int u = i * C::LPR + lir;
        if (WT == TYPE_NVFP4) {
            const uint8_t * blk = row + (u >> 1) * NVFP4_BLOCK_BYTES;
            const int hf = u & 1;
            const uint32_t dw = *reinterpret_cast<const uint32_t *>(blk);
            const uint32_t * qs = reinterpret_cast<const uint32_t *>(blk + 4 + 16 * hf);
            const uint32_t w0 = qs[0], w1 = qs[1], w2 = qs[2], w3 = qs[3];
            const float s0 = ue_tab[(dw >> (16 * hf)) & 0xff];
            const float s1 = ue_tab[(dw >> (16 * hf + 8)) & 0xff];
            const Fp4Word a0 = fp4_decode_word(w0), a1 = fp4_decode_word(w1), b0 = fp4_decode_word(w2), b1 = fp4_decode_word(w3);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const uint32_t * q = acts[t].q[i];
                int pa = dot4((int) a0.pos_a, (int) q[0], 0);
                pa = dot4((int) a0.pos_b, (int) q[1], pa);
                pa = dot4((int) a1.pos_a, (int) q[2], pa);
                pa = dot4((int) a1.pos_b, (int) q[3], pa);
                int na = dot4((int) a0.neg_a, (int) q[0], 0);
                na = dot4((int) a0.neg_b, (int) q[1], na);
                na = dot4((int) a1.neg_a, (int) q[2], na);
                na = dot4((int) a1.neg_b, (int) q[3], na);
                int pb = dot4((int) b0.pos_a, (int) q[4], 0);
                pb = dot4((int) b0.pos_b, (int) q[5], pb);
                pb = dot4((int) b1.pos_a, (int) q[6], pb);
                pb = dot4((int) b1.pos_b, (int) q[7], pb);
                int nb = dot4((int) b0.neg_a, (int) q[4], 0);
                nb = dot4((int) b0.neg_b, (int) q[5], nb);
                nb = dot4((int) b1.neg_a, (int) q[6], nb);
                nb = dot4((int) b1.neg_b, (int) q[7], nb);
                const float dy = acts[t].d[i];
                acc[t] = fmaf(s0 * dy, small_int_to_float(pa - na), acc[t]);
                acc[t] = fmaf(s1 * dy, small_int_to_float(pb - nb), acc[t]);
            }
        } else {
            const int sb = u >> 3, p = u & 7;
            const uint8_t * blk = row + sb * Q3K_BLOCK_BYTES;  // 2-byte aligned
            const uint32_t hm = lds_u32_a2(blk + 4 * p);
            const uint32_t qs0 = lds_u32_a2(blk + 32 + 4 * p);
            const uint32_t qs1 = lds_u32_a2(blk + 64 + 4 * p);
            uint32_t sc[4];
            q3k_unpack_scales(lds_u32_a2(blk + 96), lds_u32_a2(blk + 100), lds_u32_a2(blk + 104), sc);
            const float dw = __half2float(*reinterpret_cast<const __half *>(blk + 108));
            const int c0 = q3k_scale_at(sc, 2 * p), c1 = q3k_scale_at(sc, 2 * p + 1);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                int isum = q3k_unit_dot(qs0, qs1, hm, sc, p, acts[t].q[i]);
                const int bs = acts[t].bs[i];
                isum -= 4 * (c0 * (int) (int16_t) (bs & 0xffff) + c1 * (int) (int16_t) (bs >> 16));
                acc[t] = fmaf(dw * acts[t].d[i], small_int_to_float(isum), acc[t]);
            }
        }
    }
}

// chunk walker shared by the producer thread and the consumers
struct Chunk {
    int a;      // index into active[]
    int r0;     // first output row
    int n;      // rows
};
struct ChunkWalker {
    int u, u_end, units_per_expert, gran, max_rows;
    __device__ __forceinline__ bool next(Chunk & c) {
        if (u >= u_end) return false;
        const int a = u / units_per_expert;
        const int uu = u - a * units_per_expert;
        int n_units = min(u_end - u, units_per_expert - uu);
        n_units = min(n_units, max_rows / gran);
        c.a = a;
        c.r0 = uu * gran;
        c.n = n_units * gran;
        u += n_units;
        return true;
    }
};

template <int WT, int K, bool DUAL, int NT, int STAGES>
__global__ void __launch_bounds__(GemvCfg<WT, K>::NWARPS * 32, 1) expert_gemv_kernel(const GemvParams p) {
    using C = GemvCfg<WT, K>;
    constexpr int NTENS = DUAL ? 2 : 1;
    constexpr int STAGE_BYTES = C::TENSOR_STAGE_BYTES * NTENS;

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t * ring = smem;                                                   // STAGES * STAGE_BYTES
    uint64_t * full = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);  // STAGES barriers
    float * ue_tab = reinterpret_cast<float *>(full + STAGES);               // 256 floats (NVFP4 only)
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int lir = lane % C::LPR;   // lane in row group
    const int rgrp = lane / C::LPR;  // which of the RPP rows of a pass

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
        s_abort = 0;
    }
    if (WT == TYPE_NVFP4)
        for (int i = tid; i < 256; i += blockDim.x) ue_tab[i] = ue4m3_half_to_f32(i);
    __syncthreads();

    const int n_active = p.meta[0];
    const int upe = p.n_out / C::GRAN;                       // span units per expert
    const long long total = (long long) n_active * upe;
    ChunkWalker cons, prod;
    // Span boundaries balance WORK, not rows: a weight row of an expert with n routed rows costs ceil(n/NT) passes.
    // Boundary i sits at work i/grid of the total; both neighbours compute it the same way, so spans tile exactly.
    __shared__ int s_span[2];
    if (tid < 2) {
        const int * cw = p.cost + (NT == 1 ? 0 : NT == 2 ? 1 : 2) * (p.n_as + 1);
        const long long total_work = (long long) cw[n_active] * upe;
        const long long c = total_work * (blockIdx.x + tid) / gridDim.x;
        int lo = 0, hi = n_active;  // largest a with cw[a]*upe <= c
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((long long) cw[mid] * upe <= c) lo = mid; else hi = mid;
        }
        int u;
        if (n_active == 0) u = 0;
        else if (blockIdx.x + tid == gridDim.x) u = (int) total;
        else {
            const int per = max(cw[lo + 1] - cw[lo], 1);
            const long long uu = (c - (long long) cw[lo] * upe) / per;
            u = lo * upe + (int) (uu < (long long) upe ? uu : (long long) upe);
        }
        s_span[tid] = u;
    }
    __syncthreads();
    cons.u = s_span[0];
    cons.u_end = s_span[1];
    cons.units_per_expert = upe;
    cons.gran = C::GRAN;
    cons.max_rows = C::ROWS_PER_STAGE;
    prod = cons;

    auto issue = [&](const Chunk & c, int stage) {
        const int e = p.active[c.a];
        const uint32_t bytes = (uint32_t) c.n * C::ROW_BYTES;
        uint8_t * dst = ring + (size_t) stage * STAGE_BYTES;
        mbar_arrive_expect_tx(&full[stage], bytes * NTENS);
        const size_t off = ((size_t) e * p.n_out + c.r0) * C::ROW_BYTES;
        bulk_g2s(dst, p.w0 + off, bytes, &full[stage]);
        if (DUAL) bulk_g2s(dst + C::TENSOR_STAGE_BYTES, p.w1 + off, bytes, &full[stage]);
    };

    int issued = 0;
    if (tid == 0) {
        Chunk c;
        for (int s = 0; s < STAGES; ++s)
            if (prod.next(c)) { issue(c, s); ++issued; }
    }

    LaneAct<WT, C::UPL> acts[NT];
    int loaded_e = -1, loaded_tc = -1;

    Chunk ck;
    int ci = 0;
    bool failed = false;
    while (cons.next(ck)) {
        const int stage = ci % STAGES;
        const uint32_t parity = (uint32_t) (ci / STAGES) & 1u;
        if (!mbar_wait_bounded(&full[stage], parity)) {
            report_error(p.err, DEV_ERR_BARRIER_TIMEOUT);
            s_abort = 1;
        }
        if (__syncthreads_or(s_abort)) { failed = true; break; }

        const int e = p.active[ck.a];
        const int row_beg = p.offsets[e], n_e = p.offsets[e + 1] - row_beg;
        const uint8_t * st = ring + (size_t) stage * STAGE_BYTES;
        const float sc0 = p.scale0 ? p.scale0[e] : 1.0f;
        const float sc1 = (DUAL && p.scale1) ? p.scale1[e] : 1.0f;

        for (int tc = 0; tc * NT < n_e; ++tc) {
            int rows[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int i = tc * NT + t;
                rows[t] = i < n_e ? p.perm[row_beg + i] : -1;
            }
            if (loaded_e != e || loaded_tc != tc) {
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const int r = rows[t];
                    const int arow = r >= 0 ? (r / p.n_ids) * p.ne11 + (r % p.n_ids) % p.ne11 : 0;
                    load_lane_act<WT, K>(acts[t], p.act, arow, lir, r >= 0);
                }
                loaded_e = e;
                loaded_tc = tc;
            }
#pragma unroll 1
            for (int ps = 0; ps < C::PASSES; ++ps) {
                const int lr = (ps * C::NWARPS + warp) * C::RPP + rgrp;  // row within the stage
                const bool row_ok = lr < ck.n;
                const uint8_t * wrow = st + (size_t) (row_ok ? lr : 0) * C::ROW_BYTES;
                float g[NT], uacc[NT];
                row_partial<WT, K, NT>(wrow, lir, acts, ue_tab, g);
                if (DUAL) row_partial<WT, K, NT>(wrow + C::TENSOR_STAGE_BYTES, lir, acts, ue_tab, uacc);
                group_reduce<NT, C::LPR>(g, lir);
                if (DUAL) group_reduce<NT, C::LPR>(uacc, lir);
                const int tv = group_reduce_owner_value<NT, C::LPR>(lir);
                constexpr int LOWMASK = (C::LPR / NT) - 1;  // lanes sharing the same value; the one with low bits 0 writes
                if (row_ok && (lir & LOWMASK) == 0) {
                    int r = -1;
#pragma unroll
                    for (int t = 0; t < NT; ++t)
                        if (t == tv) r = rows[t];
                    if (r >= 0) {
                        float v = g[0] * sc0;
                        if (DUAL) {
                            const float uv = uacc[0] * sc1;
                            v = __fmul_rn(ggml_silu(v), uv);
                        }
                        p.out[(size_t) r * p.n_out + ck.r0 + lr] = v;
                    }
                }
            }
        }
        __syncthreads();  // everyone is done reading this stage
        if (tid == 0) {
            Chunk c;
            if (prod.next(c)) { issue(c, stage); ++issued; }
        }
        ++ci;
    }

    if (failed && tid == 0) {
        // bounded drain of copies still in flight before the block (and its shared memory) goes away
        for (int k = ci; k < issued; ++k) mbar_wait_bounded(&full[k % STAGES], (uint32_t) (k / STAGES) & 1u, 200000000ull);
    }
}

// ring depth: four stages unless that would not fit in shared memory
template <int WT, int K, bool DUAL>
constexpr int gemv_stages() {
    constexpr int stage = GemvCfg<WT, K>::TENSOR_STAGE_BYTES * (DUAL ? 2 : 1);
    return (4 * stage <= 200 * 1024) ? 4 : (3 * stage <= 200 * 1024) ? 3 : 2;
}

template <int WT, int K, bool DUAL, int STAGES>
constexpr size_t gemv_smem_bytes() {
    return (size_t) STAGES * GemvCfg<WT, K>::TENSOR_STAGE_BYTES * (DUAL ? 2 : 1) + STAGES * 8 + 256 * 4 + 64;
}

// ---- weighted combine: out[t][i] = sum over slots in slot order of y[t*k+s][i] * w[t][s] (forward.cpp:308-310)
__global__ void __launch_bounds__(256) combine_kernel(const float * __restrict__ y, const float * __restrict__ w, float * __restrict__ out,
                                                     int n, int k, int T) {
    const int i4 = blockIdx.x * blockDim.x + threadIdx.x;  // float4 index within a token row
    const int t = blockIdx.y;
    if (i4 * 4 >= n || t >= T) return;
    const float4 * yr = reinterpret_cast<const float4 *>(y + (size_t) t * k * n) + i4;
    const float * wr = w + (size_t) t * k;
    float4 a = yr[0];
    const float w0 = wr[0];
    a.x = __fmul_rn(a.x, w0); a.y = __fmul_rn(a.y, w0); a.z = __fmul_rn(a.z, w0); a.w = __fmul_rn(a.w, w0);
    for (int s = 1; s < k; ++s) {
        const float4 b = yr[(size_t) s * (n / 4)];
        const float ws = wr[s];
        a.x = __fadd_rn(a.x, __fmul_rn(b.x, ws));
        a.y = __fadd_rn(a.y, __fmul_rn(b.y, ws));
        a.z = __fadd_rn(a.z, __fmul_rn(b.z, ws));
        a.w = __fadd_rn(a.w, __fmul_rn(b.w, ws));
    }
    reinterpret_cast<float4 *>(out + (size_t) t * n)[i4] = a;
}

}  // namespace b200moe
