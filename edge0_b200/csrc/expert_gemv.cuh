// Grouped expert GEMV for decode / batched decode: streams only the routed experts' quantised rows from HBM through
// a shared-memory ring filled by 1-D bulk async copies (TMA), integer dot products against the reference's int8
// activation grid, and fp32 accumulation in EXACTLY the order of the reference's AVX2 kernels, so every dot product
// is bit-identical to the CPU path (and with it every later re-quantisation of activations).
//
// How the reference sums (ggml-cpu/arch/x86/quants.c, AVX2 branches): eight fp32 lanes; lane L collects, block after
// block, fma(scale, (float) p_L, acc_L) where p_L is the integer dot of a fixed group of 4 elements per 32
// (NVFP4: group L of each Q8_0 block; Q3_K: elements 4L..4L+3 of every 32-group of the super-block, scale-weighted and
// summed over the super-block first); the eight lanes are folded at the end as ((a0+a4)+(a2+a6))+((a1+a5)+(a3+a7)).
// Here 8 GPU lanes play the 8 AVX lanes of one weight row (4 rows per warp), each running its chain over K in
// order; three xor-shuffles reproduce the fold.
//
// One kernel template serves
//   DUAL = true : gate and up projections of the same rows + SwiGLU epilogue  -> hidden[row][n_out]
//   DUAL = false: one indexed matmul (ggml MUL_MAT_ID semantics)               -> dst[row][n_out]
// "row" is a routed row: token*n_ids + slot.
//
// Work distribution: the rows of all active experts form one flat list (active expert a, output row r); every CTA of
// the persistent grid takes a contiguous span of equal WORK (rows x passes over the expert's routed rows).  A span is
// walked in chunks of at most ROWS_PER_STAGE rows of one expert; chunk c lives in ring stage c % STAGES.
#pragma once
#include <type_traits>

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
    const float * act_f32; // or (NVFP4 only): the fp32 activations [rows][K], quantised to Q8_0 while they are staged (act unused)
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
    int w_stride;         // rows between consecutive experts' matrices: n_out, or 0 when every group uses the same matrix
    int * err;
};

template <int WT, int K, int NW = 8>
struct GemvCfg {
    static constexpr int LPR = 8;            // lanes per row = the reference's 8 SIMD lanes
    static constexpr int RPP = 4;            // rows per warp pass
    static constexpr int ROW_BYTES = WT == TYPE_NVFP4 ? K / 64 * 36 : K / 256 * 110;
    static constexpr int GRAN = (ROW_BYTES % 16 == 0) ? 1 : 8;  // span granularity in rows (16-byte rule of bulk copies)
    static constexpr int NWARPS = NW;        // 8; 4 for the one-or-two-token kernel (several small CTAs per SM)
    // passes per warp per stage chosen so a (single-tensor) stage is roughly 12-40 KB
    static constexpr int PASSES = (ROW_BYTES * RPP * NWARPS >= 12288) ? 1 : (ROW_BYTES * RPP * NWARPS >= 6144) ? 2 : 4;
    static constexpr int ROWS_PER_STAGE = NWARPS * RPP * PASSES;
    static constexpr int TENSOR_STAGE_BYTES = ROWS_PER_STAGE * ROW_BYTES;
    static_assert(TENSOR_STAGE_BYTES % 16 == 0, "stage must keep 16-byte alignment");
    // activations of one token in shared memory: K int8, then the block scales as floats (padded to 16 bytes)
    static constexpr int ACT_D = WT == TYPE_NVFP4 ? K / 32 : K / 256;
    static constexpr int ACT_TOKEN_BYTES = K + ((ACT_D * 4 + 15) / 16) * 16;
};

__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t * p) {  // 2-byte aligned 32-bit load from shared memory
    const uint16_t * h = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t) h[0] | ((uint32_t) h[1] << 16);
}

// One SIMD lane (L = 0..7) of the reference's dot product of one weight row with NT activation rows.
//   row   : the quantised weight row in shared memory
//   acts  : the activations of NTS rows, token-interleaved: words [K/4][NTS] of int8x4, then block scales [ACT_D][NTS];
//           the first NT of the NTS rows are used
template <int N, typename T>
__device__ __forceinline__ void load_vec(T (&dst)[N], const T * src) {
    static_assert(sizeof(T) == 4, "32-bit elements");
    if (N == 4) {
        const uint4 v = *reinterpret_cast<const uint4 *>(src);
        memcpy(&dst[0], &v, 16);
    } else if (N == 2) {
        const uint2 v = *reinterpret_cast<const uint2 *>(src);
        memcpy(&dst[0], &v, 8);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) dst[i] = src[i];
    }
}

template <int WT, int K, int NT, int NTS>
__device__ __forceinline__ void lane_chain(const uint8_t * __restrict__ row, int L, const uint8_t * __restrict__ acts,
                                           const float * __restrict__ ue_tab, float (&acc)[NT]) {
    using C = GemvCfg<WT, K>;
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.0f;
    if (WT == TYPE_NVFP4) {
        // lane L: sub-block (L>>2) of each half block, elements 4*(L&3) .. +3 of it = the low (L&3 < 2) or high nibbles of
        // one qs word; they meet word L of the Q8_0 block.  ggml_vec_dot_nvfp4_q8_0, ggml-cpu/arch/x86/quants.c:1004-1062.
        const int sub_in_half = L >> 2, mp = L & 3;
        const int word_off = 4 + 8 * sub_in_half + 4 * (mp & 1);
        const int nib_shift = 4 * (mp >> 1);
#pragma unroll 2
        for (int b = 0; b < K / 64; ++b) {
            const uint8_t * blk = row + b * NVFP4_BLOCK_BYTES;
            const uint32_t dw = *reinterpret_cast<const uint32_t *>(blk);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const uint32_t w = *reinterpret_cast<const uint32_t *>(blk + 16 * hf + word_off);
                const uint32_t t4 = (w >> nib_shift) & 0x0f0f0f0fu;          // four codes, one per byte
                const uint32_t u = t4 | (t4 >> 4);
                const uint32_t sel = byte_perm(u, 0u, 0x4420u);              // the four codes packed into 16 bits (bytes 0 and 2 of u)
                const uint32_t pos = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel);
                const uint32_t neg = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel ^ 0x8888u);
                // signed bytes: a byte of `neg` is a magnitude 0..12, 0x80 - it never borrows, the xor drops the guard bit
                const uint32_t code = pos | ((0x80808080u - neg) ^ 0x80808080u);
                const float sw = ue_tab[(dw >> (8 * (2 * hf + sub_in_half))) & 0xff];
                const int unit = 2 * b + hf;
                // activations are stored [unit][lane word][token] and [unit][token]: one vector load serves all NT rows
                uint32_t aw[NT];
                float dy[NT];
                load_vec<NT>(aw, reinterpret_cast<const uint32_t *>(acts) + (size_t) (unit * 8 + L) * NTS);
                load_vec<NT>(dy, reinterpret_cast<const float *>(acts + (size_t) K * NTS) + (size_t) unit * NTS);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const int p = dot4((int) code, (int) aw[t], 0);
                    acc[t] = __fmaf_rn(__fmul_rn(sw, dy[t]), small_int_to_float(p), acc[t]);
                }
            }
        }
    } else {
        // lane L: byte columns 4L..4L+3 of every super-block; integer sum over the super-block with the signed 6-bit
        // sub-block scales, then one fma with d_w*d_x.  ggml_vec_dot_q3_K_q8_K, ggml-cpu/arch/x86/quants.c:1766-1880.
        const int hi = L >= 4 ? 1 : 0;
#pragma unroll 1
        for (int sb = 0; sb < K / 256; ++sb) {
            const uint8_t * blk = row + sb * Q3K_BLOCK_BYTES;  // 2-byte aligned
            const uint32_t hm = lds_u32_a2(blk + 4 * L);
            const uint32_t qs0 = lds_u32_a2(blk + 32 + 4 * L);
            const uint32_t qs1 = lds_u32_a2(blk + 64 + 4 * L);
            uint32_t sc[4];
            q3k_unpack_scales(lds_u32_a2(blk + 96), lds_u32_a2(blk + 100), lds_u32_a2(blk + 104), sc);
            const float dw = __half2float(*reinterpret_cast<const __half *>(blk + 108));
            int sumi[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) sumi[t] = 0;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t w = j ? qs1 : qs0;
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const int bit = 4 * j + s;
                    const uint32_t lo2 = (w >> (2 * s)) & 0x03030303u;
                    const uint32_t hb4 = bit >= 2 ? ((hm >> (bit - 2)) & 0x04040404u) : ((hm << (2 - bit)) & 0x04040404u);
                    // codes 0..7 -> signed -4..3 in every byte without borrows between bytes
                    const uint32_t code = (((lo2 | hb4) | 0x80808080u) - 0x04040404u) ^ 0x80808080u;
                    const int scale = q3k_scale_at(sc, 8 * j + 2 * s + hi);
                    uint32_t aw[NT];
                    load_vec<NT>(aw, reinterpret_cast<const uint32_t *>(acts) + (size_t) (sb * 64 + 8 * (4 * j + s) + L) * NTS);
#pragma unroll
                    for (int t = 0; t < NT; ++t) sumi[t] += scale * dot4((int) code, (int) aw[t], 0);
                }
            }
            float dx[NT];
            load_vec<NT>(dx, reinterpret_cast<const float *>(acts + (size_t) K * NTS) + (size_t) sb * NTS);
#pragma unroll
            for (int t = 0; t < NT; ++t) acc[t] = __fmaf_rn(__fmul_rn(dx[t], dw), small_int_to_float(sumi[t]), acc[t]);
        }
    }
    // hsum_float_8: (a4+a0, a5+a1, a6+a2, a7+a3) -> (r0+r2, r1+r3) -> s0+s1
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float v = acc[t];
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
        acc[t] = v;
    }
}

// decode of four NVFP4 codes (one per byte of t4's nibbles) to signed int8 (twice the E2M1 value)
__device__ __forceinline__ uint32_t nvfp4_codes_to_s8(uint32_t w, int nib_shift) {
    const uint32_t t4 = (w >> nib_shift) & 0x0f0f0f0fu;          // four codes, one per byte
    const uint32_t u = t4 | (t4 >> 4);
    const uint32_t sel = byte_perm(u, 0u, 0x4420u);              // the four codes packed into 16 bits (bytes 0 and 2 of u)
    const uint32_t pos = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel);
    const uint32_t neg = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel ^ 0x8888u);
    // signed bytes: a byte of `neg` is a magnitude 0..12, 0x80 - it never borrows, the xor drops the guard bit
    return pos | ((0x80808080u - neg) ^ 0x80808080u);
}

// lane_chain<TYPE_NVFP4> for TWO weight rows against the same activations (the gate row and the up row of a feature): the two
// chains are independent, so running them in one loop doubles the work in flight per lane - and each activation word and block
// scale is fetched once for both.  Every chain keeps its own order of operations: the results are those of two lane_chain calls.
template <int K, int NT, int NTS>
__device__ __forceinline__ void lane_chain_pair(const uint8_t * __restrict__ row0, const uint8_t * __restrict__ row1, int L,
                                                const uint8_t * __restrict__ acts, const float * __restrict__ ue_tab, float (&acc0)[NT],
                                                float (&acc1)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) acc0[t] = acc1[t] = 0.0f;
    const int sub_in_half = L >> 2, mp = L & 3;
    const int word_off = 4 + 8 * sub_in_half + 4 * (mp & 1);
    const int nib_shift = 4 * (mp >> 1);
#pragma unroll 2
    for (int b = 0; b < K / 64; ++b) {
        const uint8_t * blk0 = row0 + b * NVFP4_BLOCK_BYTES, * blk1 = row1 + b * NVFP4_BLOCK_BYTES;
        const uint32_t dw0 = *reinterpret_cast<const uint32_t *>(blk0), dw1 = *reinterpret_cast<const uint32_t *>(blk1);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const uint32_t code0 = nvfp4_codes_to_s8(*reinterpret_cast<const uint32_t *>(blk0 + 16 * hf + word_off), nib_shift);
            const uint32_t code1 = nvfp4_codes_to_s8(*reinterpret_cast<const uint32_t *>(blk1 + 16 * hf + word_off), nib_shift);
            const float sw0 = ue_tab[(dw0 >> (8 * (2 * hf + sub_in_half))) & 0xff], sw1 = ue_tab[(dw1 >> (8 * (2 * hf + sub_in_half))) & 0xff];
            const int unit = 2 * b + hf;
            uint32_t aw[NT];
            float dy[NT];
            load_vec<NT>(aw, reinterpret_cast<const uint32_t *>(acts) + (size_t) (unit * 8 + L) * NTS);
            load_vec<NT>(dy, reinterpret_cast<const float *>(acts + (size_t) K * NTS) + (size_t) unit * NTS);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                acc0[t] = __fmaf_rn(__fmul_rn(sw0, dy[t]), small_int_to_float(dot4((int) code0, (int) aw[t], 0)), acc0[t]);
                acc1[t] = __fmaf_rn(__fmul_rn(sw1, dy[t]), small_int_to_float(dot4((int) code1, (int) aw[t], 0)), acc1[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float v = acc0[t], w = acc1[t];
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
        w = __fadd_rn(w, __shfl_xor_sync(0xffffffffu, w, 4));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
        w = __fadd_rn(w, __shfl_xor_sync(0xffffffffu, w, 2));
        v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
        w = __fadd_rn(w, __shfl_xor_sync(0xffffffffu, w, 1));
        acc0[t] = v;
        acc1[t] = w;
    }
}

// The same pair for ONE activation row whose int8 values (q, K bytes) and block scales (d, K/32 floats) lie in separate arrays,
// in any address space (the layout lane_chain_split reads).
template <int K>
__device__ __forceinline__ void lane_chain_split_pair(const uint8_t * __restrict__ row0, const uint8_t * __restrict__ row1, int L,
                                                      const uint8_t * __restrict__ q, const float * __restrict__ d,
                                                      const float * __restrict__ ue_tab, float & out0, float & out1) {
    const int sub_in_half = L >> 2, mp = L & 3;
    const int word_off = 4 + 8 * sub_in_half + 4 * (mp & 1);
    const int nib_shift = 4 * (mp >> 1);
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll 4
    for (int b = 0; b < K / 64; ++b) {
        const uint8_t * blk0 = row0 + b * NVFP4_BLOCK_BYTES, * blk1 = row1 + b * NVFP4_BLOCK_BYTES;
        const uint32_t dw0 = *reinterpret_cast<const uint32_t *>(blk0), dw1 = *reinterpret_cast<const uint32_t *>(blk1);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const uint32_t code0 = nvfp4_codes_to_s8(*reinterpret_cast<const uint32_t *>(blk0 + 16 * hf + word_off), nib_shift);
            const uint32_t code1 = nvfp4_codes_to_s8(*reinterpret_cast<const uint32_t *>(blk1 + 16 * hf + word_off), nib_shift);
            const float sw0 = ue_tab[(dw0 >> (8 * (2 * hf + sub_in_half))) & 0xff], sw1 = ue_tab[(dw1 >> (8 * (2 * hf + sub_in_half))) & 0xff];
            const int unit = 2 * b + hf;
            const uint32_t aw = reinterpret_cast<const uint32_t *>(q)[unit * 8 + L];
            const float dy = d[unit];
            a0 = __fmaf_rn(__fmul_rn(sw0, dy), small_int_to_float(dot4((int) code0, (int) aw, 0)), a0);
            a1 = __fmaf_rn(__fmul_rn(sw1, dy), small_int_to_float(dot4((int) code1, (int) aw, 0)), a1);
        }
    }
    a0 = __fadd_rn(a0, __shfl_xor_sync(0xffffffffu, a0, 4));
    a1 = __fadd_rn(a1, __shfl_xor_sync(0xffffffffu, a1, 4));
    a0 = __fadd_rn(a0, __shfl_xor_sync(0xffffffffu, a0, 2));
    a1 = __fadd_rn(a1, __shfl_xor_sync(0xffffffffu, a1, 2));
    a0 = __fadd_rn(a0, __shfl_xor_sync(0xffffffffu, a0, 1));
    a1 = __fadd_rn(a1, __shfl_xor_sync(0xffffffffu, a1, 1));
    out0 = a0;
    out1 = a1;
}

// The NVFP4 chain of lane_chain for ONE activation row whose int8 values (q, K bytes) and block scales (d, K/32 floats)
// lie in separate arrays, in any address space.  Same operations in the same order as lane_chain<TYPE_NVFP4, K, 1, 1>.
template <int K>
__device__ __forceinline__ void lane_chain_split(const uint8_t * __restrict__ row, int L, const uint8_t * __restrict__ q,
                                                 const float * __restrict__ d, const float * __restrict__ ue_tab, float (&acc)[1]) {
    const int sub_in_half = L >> 2, mp = L & 3;
    const int word_off = 4 + 8 * sub_in_half + 4 * (mp & 1);
    const int nib_shift = 4 * (mp >> 1);
    float a = 0.0f;
#pragma unroll 4
    for (int b = 0; b < K / 64; ++b) {
        const uint8_t * blk = row + b * NVFP4_BLOCK_BYTES;
        const uint32_t dw = *reinterpret_cast<const uint32_t *>(blk);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            const uint32_t w = *reinterpret_cast<const uint32_t *>(blk + 16 * hf + word_off);
            const uint32_t t4 = (w >> nib_shift) & 0x0f0f0f0fu;
            const uint32_t u = t4 | (t4 >> 4);
            const uint32_t sel = byte_perm(u, 0u, 0x4420u);
            const uint32_t pos = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel);
            const uint32_t neg = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel ^ 0x8888u);
            const uint32_t code = pos | ((0x80808080u - neg) ^ 0x80808080u);
            const float sw = ue_tab[(dw >> (8 * (2 * hf + sub_in_half))) & 0xff];
            const int unit = 2 * b + hf;
            const uint32_t aw = reinterpret_cast<const uint32_t *>(q)[unit * 8 + L];
            const float dy = d[unit];
            const int p = dot4((int) code, (int) aw, 0);
            a = __fmaf_rn(__fmul_rn(sw, dy), small_int_to_float(p), a);
        }
    }
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 4));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
    acc[0] = a;
}

// The same chain run by a whole warp for ONE row: the four 8-lane groups split the half-blocks between them (group rg takes
// units rg, rg + 4, ...), every lane fetches and decodes its share with all loads in flight at once, and the fp32 chain - which
// must stay sequential to keep the reference's bits - then collects scale and dot product of every unit in order through
// shuffles.  All four groups end with the same eight partial sums; the result is valid in every lane.
template <int K>
__device__ __forceinline__ float lane_chain_warp(const uint8_t * __restrict__ row, int lane, const uint8_t * __restrict__ q,
                                                 const float * __restrict__ d, const float * __restrict__ ue_tab) {
    constexpr int UNITS = K / 32, UPL = UNITS / 4;       // half-blocks in the row, and per lane
    constexpr int BATCH = UPL < 8 ? UPL : 8;             // fetched and decoded at a time (bounds the registers)
    static_assert(UNITS % 4 == 0 && UPL % BATCH == 0, "half-blocks must split over four lane groups in whole batches");
    const int L = lane & 7, rg = lane >> 3;
    const int sub_in_half = L >> 2, mp = L & 3;
    const int word_off = 4 + 8 * sub_in_half + 4 * (mp & 1);
    const int nib_shift = 4 * (mp >> 1);
    float a = 0.0f;
#pragma unroll 1
    for (int i0 = 0; i0 < UPL; i0 += BATCH) {
        uint32_t w[BATCH], aw[BATCH], dw[BATCH];
        float dy[BATCH];
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int u = 4 * (i0 + i) + rg, b = u >> 1, hf = u & 1;
            const uint8_t * blk = row + b * NVFP4_BLOCK_BYTES;
            dw[i] = *reinterpret_cast<const uint32_t *>(blk);
            w[i] = *reinterpret_cast<const uint32_t *>(blk + 16 * hf + word_off);
            aw[i] = reinterpret_cast<const uint32_t *>(q)[u * 8 + L];
            dy[i] = d[u];
        }
        float sd[BATCH], pf[BATCH];
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int hf = rg & 1;                       // u = 4 (i0 + i) + rg
            const uint32_t t4 = (w[i] >> nib_shift) & 0x0f0f0f0fu;
            const uint32_t u8 = t4 | (t4 >> 4);
            const uint32_t sel = byte_perm(u8, 0u, 0x4420u);
            const uint32_t pos = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel);
            const uint32_t neg = byte_perm(FP4_MAG_LO, FP4_MAG_HI, sel ^ 0x8888u);
            const uint32_t code = pos | ((0x80808080u - neg) ^ 0x80808080u);
            const float sw = ue_tab[(dw[i] >> (8 * (2 * hf + sub_in_half))) & 0xff];
            sd[i] = __fmul_rn(sw, dy[i]);
            pf[i] = small_int_to_float(dot4((int) code, (int) aw[i], 0));
        }
#pragma unroll
        for (int u = 0; u < 4 * BATCH; ++u) {            // units 4 i0 .. 4 (i0 + BATCH) - 1, in order
            const int src = (u & 3) * 8 + L;
            const float sv = __shfl_sync(0xffffffffu, sd[u >> 2], src), pv = __shfl_sync(0xffffffffu, pf[u >> 2], src);
            a = __fmaf_rn(sv, pv, a);
        }
    }
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 4));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
    return a;
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

template <int WT, int K, bool DUAL, int NT, int STAGES, int NW = 8>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 1 : 4) expert_gemv_kernel(const GemvParams p) {
    using C = GemvCfg<WT, K, NW>;
    constexpr int NTENS = DUAL ? 2 : 1;
    constexpr int STAGE_BYTES = C::TENSOR_STAGE_BYTES * NTENS;
    constexpr int NTHREADS = C::NWARPS * 32;

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t * ring = smem;                                                        // STAGES * STAGE_BYTES
    uint8_t * acts = smem + STAGES * STAGE_BYTES;                                 // NT * ACT_TOKEN_BYTES (16-byte aligned)
    uint64_t * full = reinterpret_cast<uint64_t *>(acts + NT * C::ACT_TOKEN_BYTES);  // STAGES barriers
    float * ue_tab = reinterpret_cast<float *>(full + STAGES);                    // 256 floats (NVFP4 only)
    __shared__ int s_abort;
    __shared__ int s_span[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int L = lane & 7;       // SIMD lane of the reference this thread plays
    const int rgrp = lane >> 3;   // which of the 4 rows of a warp pass

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
        s_abort = 0;
    }
    if (WT == TYPE_NVFP4)
        for (int i = tid; i < 256; i += NTHREADS) ue_tab[i] = ue4m3_half_to_f32(i);
    __syncthreads();
    pdl_wait();                 // programmatic dependent launch: everything before this ran alongside the previous kernel's tail
    pdl_launch_dependents();

    const int n_active = p.meta[0];
    const int upe = p.n_out / C::GRAN;                       // span units per expert
    const long long total = (long long) n_active * upe;
    // Span boundaries balance WORK, not rows: a weight row of an expert with n routed rows costs 3 per pass (decode) + 2 per routed row.
    // Boundary i sits at work i/grid of the total; both neighbours compute it the same way, so spans tile exactly.
    if (NW != 8) {
        // one-or-two-token kernel: CTA b owns stage-sized chunk b of the flat row list - no search, no dependent loads
        if (tid < 2) {
            const long long u = (long long) (blockIdx.x + tid) * (C::ROWS_PER_STAGE / C::GRAN);
            s_span[tid] = (int) (u < total ? u : total);
        }
    } else if (tid < 2) {
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
    ChunkWalker cons, prod;
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
        const size_t off = ((size_t) e * p.w_stride + c.r0) * C::ROW_BYTES;
        bulk_g2s(dst, p.w0 + off, bytes, &full[stage]);
        if (DUAL) bulk_g2s(dst + C::TENSOR_STAGE_BYTES, p.w1 + off, bytes, &full[stage]);
    };

    int issued = 0;
    if (tid == 0) {
        Chunk c;
        for (int s = 0; s < STAGES; ++s)
            if (prod.next(c)) { issue(c, s); ++issued; }
    }

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

        // Routed rows of this expert are taken NT at a time; a remainder of 1 or 2 runs the narrower chains instead of
        // padding to NT (the weight decode is shared by the rows of a pass, the per-row work is not).
        for (int t0 = 0, tc = 0; t0 < n_e; ++tc) {
            const int left = n_e - t0;
            const int ntc = (NT >= 4 && left >= 3) ? 4 : (NT >= 2 && left >= 2) ? 2 : 1;
            int rows[NT];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int i = t0 + t;
                rows[t] = (t < ntc && i < n_e) ? p.perm[row_beg + i] : -1;
            }
            if (loaded_e != e || loaded_tc != tc) {
                // the activation rows of this pass into shared memory (all warps use the same ones)
                __syncthreads();
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    if (t >= ntc) break;
                    const int r = rows[t];
                    const int arow = r >= 0 ? (r / p.n_ids) * p.ne11 + (r % p.n_ids) % p.ne11 : 0;
                    uint32_t * dq = reinterpret_cast<uint32_t *>(acts);
                    float * dd = reinterpret_cast<float *>(acts + (size_t) K * NT);
                    if (WT == TYPE_NVFP4 && p.act_f32) {
                        // Q8_0 on the fly, the arithmetic of quantize_q8_0_block: 8 lanes hold one block of 32 (4 values each)
                        const float4 * src = reinterpret_cast<const float4 *>(p.act_f32 + (size_t) arow * K);
                        for (int i0 = 0; i0 < K / 4; i0 += NTHREADS) {
                            const int i = i0 + tid;
                            const bool in = i < K / 4;
                            const float4 v = (in && r >= 0) ? __ldg(src + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                            const float id = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
                            const uint32_t q = ((uint32_t) __float2int_rn(__fmul_rn(v.x, id)) & 0xffu) |
                                               (((uint32_t) __float2int_rn(__fmul_rn(v.y, id)) & 0xffu) << 8) |
                                               (((uint32_t) __float2int_rn(__fmul_rn(v.z, id)) & 0xffu) << 16) |
                                               (((uint32_t) __float2int_rn(__fmul_rn(v.w, id)) & 0xffu) << 24);
                            if (in) {
                                dq[(size_t) i * NT + t] = q;
                                if ((i & 7) == 0) dd[(size_t) (i >> 3) * NT + t] = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
                            }
                        }
                    } else {
                        const uint32_t * srcq = reinterpret_cast<const uint32_t *>(p.act.q + (size_t) arow * K);
                        for (int i = tid; i < K / 4; i += NTHREADS) dq[(size_t) i * NT + t] = r >= 0 ? __ldg(srcq + i) : 0u;
                        for (int i = tid; i < C::ACT_D; i += NTHREADS) dd[(size_t) i * NT + t] = r >= 0 ? __ldg(p.act.d + (size_t) arow * C::ACT_D + i) : 0.0f;
                    }
                }
                __syncthreads();
                loaded_e = e;
                loaded_tc = tc;
            }
#pragma unroll 1
            for (int ps = 0; ps < C::PASSES; ++ps) {
                const int lr = (ps * C::NWARPS + warp) * C::RPP + rgrp;  // row within the stage
                const bool row_ok = lr < ck.n;
                const uint8_t * wrow = st + (size_t) (row_ok ? lr : 0) * C::ROW_BYTES;
                float g[NT], uacc[NT];
                auto run = [&](auto ntag) {
                    constexpr int NTC = decltype(ntag)::value;
                    float gg[NTC], uu[NTC];
                    if constexpr (DUAL && WT == TYPE_NVFP4) {
                        lane_chain_pair<K, NTC, NT>(wrow, wrow + C::TENSOR_STAGE_BYTES, L, acts, ue_tab, gg, uu);
                    } else {
                        lane_chain<WT, K, NTC, NT>(wrow, L, acts, ue_tab, gg);
                        if (DUAL) lane_chain<WT, K, NTC, NT>(wrow + C::TENSOR_STAGE_BYTES, L, acts, ue_tab, uu);
                    }
#pragma unroll
                    for (int t = 0; t < NTC; ++t) { g[t] = gg[t]; uacc[t] = DUAL ? uu[t] : 0.0f; }
                };
                if (NT >= 4 && ntc == 4) run(std::integral_constant<int, (NT >= 4 ? 4 : 1)>{});
                else if (NT >= 2 && ntc == 2) run(std::integral_constant<int, (NT >= 2 ? 2 : 1)>{});
                else run(std::integral_constant<int, 1>{});
                if (row_ok && L == 0) {
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const int r = rows[t];
                        if (t < ntc && r >= 0) {
                            float v = __fmul_rn(g[t], sc0);
                            if (DUAL) v = __fmul_rn(ggml_silu(v), __fmul_rn(uacc[t], sc1));
                            p.out[(size_t) r * p.n_out + ck.r0 + lr] = v;
                        }
                    }
                }
            }
            t0 += ntc;
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
    return (4 * stage <= 190 * 1024) ? 4 : (3 * stage <= 190 * 1024) ? 3 : 2;
}

template <int WT, int K, bool DUAL, int NT, int STAGES, int NW = 8>
constexpr size_t gemv_smem_bytes() {
    return (size_t) STAGES * GemvCfg<WT, K, NW>::TENSOR_STAGE_BYTES * (DUAL ? 2 : 1) + NT * GemvCfg<WT, K, NW>::ACT_TOKEN_BYTES + STAGES * 8 +
           256 * 4 + 64;
}

// ---- weighted combine: out[t][i] = sum over slots in slot order of y[t*k+s][i] * w[t][s] (forward.cpp:308-310)
__global__ void __launch_bounds__(256) combine_kernel(const float * __restrict__ y, const float * __restrict__ w, float * __restrict__ out,
                                                     int n, int k, int T) {
    pdl_wait();
    pdl_launch_dependents();

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
