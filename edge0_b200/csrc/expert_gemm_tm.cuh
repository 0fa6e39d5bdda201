// Grouped expert GEMM for batched decode: TOKENS on the M side of the instruction, 256 weight rows on the N side.
//
// Why: on this part a tcgen05.mma (kind::f16, M = 128, K = 16) with an operand A it has not seen before takes ~175 cycles
// whatever N is (measured: the same for N = 16 and N = 256).  With weights as A (expert_gemm.cuh) every instruction covers
// 128 weight rows x 16 K positions, so the weight matrices alone fix the instruction count and an expert with four rows
// costs as much as one with a hundred.  Here the roles are the usual ones, D[token, feature] = A[token, k] * B[feature, k]:
//   * B = 256 weight rows (gate rows f..f+127 followed by up rows f..f+127, or 256 rows of `down`) x 64 K positions per stage,
//     dequantised to fp16 in the 128B-swizzled K-major layout: one instruction now covers 256 weight rows x 16 K positions;
//   * A = up to 64 routed rows of one expert, each as TWO adjacent tile rows: fp16 hi part and fp16 lo part of q * d (the
//     reference's int8 grid needs 18 bits).  Both parts therefore go through the same instruction; the epilogue adds
//     accumulator lanes 2j and 2j+1 with one shuffle.  (Weights-as-A needs a second instruction for the lo part.)
// Per stage of K = 64 this is 4 instructions instead of 16.
//
// Roles and rings are those of expert_gemm.cuh (raw-weight TMA producer, activation TMA producer, MMA issuer, TMEM owner,
// 4 epilogue warps, 16 dequant warps; every wait bounded).  The kernel is bound by shared-memory traffic (operand tile written
// once and read once by the tensor core, raw rows, activation tiles): E2M1 values are therefore decoded with byte permutes in
// registers rather than through a table in shared memory (measured: the table's loads cost more than the permutes).
#pragma once
#include "expert_gemm.cuh"

namespace b200moe {

// instruction descriptor: fp16 A and B, both K-major, fp32 accumulate, M = 128, N = 256
constexpr uint32_t UMMA_IDESC_F16_M128_N256 = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

constexpr int GEMM_TM_THREADS = 768;            // 8 role warps + 16 dequant warps
constexpr int GEMM_TM_DQ_THREADS = 512;

template <int K>
struct GemmTmCfg {
    static constexpr int TOK = 64;                                  // routed rows per tile (two tile rows each)
    static constexpr int B_TILE = 256 * 128;                        // 256 weight rows x 64 halfs
    static constexpr int A_TILE = 128 * 128;                        // 64 rows x (hi, lo) x 64 halfs
    static constexpr int STAGE = B_TILE + A_TILE;
    static constexpr int RAW_STAGE = 256 * GEMM_RAW_ROW;
    static constexpr int TS = 3;
    static constexpr int RS = 2;
    static constexpr uint32_t TMEM_COLS = 512;                      // two accumulators of 256 columns
    static_assert(K % GEMM_RAW_K == 0, "K must be a multiple of 256");
    static constexpr size_t SMEM = (size_t) TS * STAGE + (size_t) RS * RAW_STAGE + 1024;
};

// DUAL: B rows 0..127 = gate rows, 128..255 = up rows of the same 128 features; epilogue = SwiGLU.
// single: B rows = 256 consecutive rows of the one tensor (n_out must be a multiple of 256).
template <int K, bool DUAL>
__global__ void __launch_bounds__(GEMM_TM_THREADS, 1)
expert_gemm_tm_kernel(const MmaParams p, const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                      const __grid_constant__ CUtensorMap map_act) {
    using C = GemmTmCfg<K>;
    constexpr int TS = C::TS, RS = C::RS, TOK = C::TOK;
    constexpr int KC = K / GEMM_RAW_K;
    constexpr int FEAT = DUAL ? 128 : 256;          // output features per item

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t * tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint8_t * raws = tiles + (size_t) TS * C::STAGE;
    __shared__ uint64_t raw_full[RS], raw_empty[RS], tile_full[TS], tile_empty[TS], acc_full[2], acc_empty[2];
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    __shared__ uint32_t s_scale_lut[256];           // UE4M3 byte -> half2(value, value)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < RS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], GEMM_TM_DQ_THREADS / 32); }
        for (int i = 0; i < TS; ++i) { mbar_init(&tile_full[i], GEMM_TM_DQ_THREADS + 1); mbar_init(&tile_empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        mbar_fence_init();
        s_abort = 0;
    }
    if (tid < 256) {
        const __half2 h = __float2half2_rn(2.0f * ue4m3_half_to_f32(tid));   // the helper returns the value halved
        s_scale_lut[tid] = *reinterpret_cast<const uint32_t *>(&h);
    }
    if (warp == 3) {
        tmem_alloc(&s_tmem, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    pdl_wait();                 // a no-op unless the launch carried the programmatic attribute (the library never gives it to this kernel)
    // No early griddepcontrol.launch_dependents here: a dependent grid must not become resident beside a kernel that holds tensor
    // memory (wrong values were measured in that situation; dependents of this kernel start when it has finished).

    const int n_active = p.meta[0];
    const int f_tiles = p.n_out / FEAT;
    const int n_items = n_active * f_tiles;

    if (warp == 0) {
        // ---------------------------------------------------------------- raw weight producer
        if (lane == 0) {
            Ring raw;
            for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const int a = item / f_tiles, ft = item % f_tiles;
                const int e = p.active[a];
                const int n_e = p.offsets[e + 1] - p.offsets[e];
                const int row0 = e * p.n_out + ft * FEAT;
                for (int t0 = 0; t0 < n_e && !s_abort; t0 += TOK) {
                    for (int kc = 0; kc < KC; ++kc) {
                        if (!wait_or_abort<200>(&raw_empty[raw.stage], raw.phase ^ 1u, &s_abort, p.err)) break;
                        uint8_t * dst = raws + (size_t) raw.stage * C::RAW_STAGE;
                        mbar_arrive_expect_tx(&raw_full[raw.stage], C::RAW_STAGE);
                        tma_load_2d(dst, &map_w0, kc * GEMM_RAW_ROW, row0, &raw_full[raw.stage]);
                        if (DUAL) tma_load_2d(dst + 128 * GEMM_RAW_ROW, &map_w1, kc * GEMM_RAW_ROW, row0, &raw_full[raw.stage]);
                        else tma_load_2d(dst + 128 * GEMM_RAW_ROW, &map_w0, kc * GEMM_RAW_ROW, row0 + 128, &raw_full[raw.stage]);
                        raw.template advance<RS>();
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- activation producer
        if (lane == 0) {
            Ring tile;
            for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const int e = p.active[item / f_tiles];
                const int row_beg = p.offsets[e], n_e = p.offsets[e + 1] - row_beg;
                for (int t0 = 0; t0 < n_e && !s_abort; t0 += TOK) {
                    for (int ks = 0; ks < K / 64; ++ks) {
                        if (!wait_or_abort<100>(&tile_empty[tile.stage], tile.phase ^ 1u, &s_abort, p.err)) break;
                        uint8_t * st = tiles + (size_t) tile.stage * C::STAGE + C::B_TILE;
                        mbar_arrive_expect_tx(&tile_full[tile.stage], C::A_TILE);
                        tma_load_2d(st, &map_act, ks * 64, 2 * (row_beg + t0), &tile_full[tile.stage]);   // rows 2j, 2j+1 = hi, lo of routed row j
                        tile.template advance<TS>();
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            Ring tile, acc;
            for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const int e = p.active[item / f_tiles];
                const int n_e = p.offsets[e + 1] - p.offsets[e];
                for (int t0 = 0; t0 < n_e && !s_abort; t0 += TOK) {
                    if (!wait_or_abort<40>(&acc_empty[acc.stage], acc.phase ^ 1u, &s_abort, p.err)) break;
                    tc_fence_after();
                    const uint32_t d0 = tmem + (uint32_t) acc.stage * 256;
                    for (int ks = 0; ks < K / 64; ++ks) {
                        if (!wait_or_abort<40>(&tile_full[tile.stage], tile.phase, &s_abort, p.err)) break;
                        tc_fence_after();
                        const uint32_t db = DESC_LO | (smem_u32(tiles + (size_t) tile.stage * C::STAGE) >> 4);
                        const uint32_t da = db + (C::B_TILE >> 4);
                        umma_f16_lohi(d0, da, db, DESC_HI, UMMA_IDESC_F16_M128_N256, ks != 0);
#pragma unroll
                        for (int kk = 1; kk < 4; ++kk) umma_f16_acc(d0, da + 2 * kk, db + 2 * kk, DESC_HI, UMMA_IDESC_F16_M128_N256);
                        umma_commit(&tile_empty[tile.stage]);   // frees the operand stage when these MMAs have read it
                        tile.template advance<TS>();
                    }
                    umma_commit(&acc_full[acc.stage]);
                    acc.template advance<2>();
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------------------------------------------------------- epilogue
        Ring acc;
        const int q = warp & 3;                 // TMEM lane quarter this warp may read: tile rows 32q .. 32q+31
        const int tok_in_tile = (32 * q + lane) >> 1;
        for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
            const int a = item / f_tiles, ft = item % f_tiles;
            const int e = p.active[a];
            const int row_beg = p.offsets[e], n_e = p.offsets[e + 1] - row_beg;
            const float sc0 = p.scale0 ? p.scale0[e] : 1.0f;
            const float sc1 = (DUAL && p.scale1) ? p.scale1[e] : 1.0f;
            for (int t0 = 0; t0 < n_e && !s_abort; t0 += TOK) {
                const int nt = min(TOK, n_e - t0);
                // lanes leave the polling loop one by one: the vote reconverges the warp (tcgen05.ld below needs all of it)
                // and makes the outcome uniform
                if (!__all_sync(0xffffffffu, wait_or_abort<200>(&acc_full[acc.stage], acc.phase, &s_abort, p.err))) break;
                tc_fence_after();
                if (16 * q < nt) {              // this warp's 16 routed rows exist (warp-uniform)
                    const uint32_t d0 = tmem + (uint32_t) acc.stage * 256 + ((uint32_t) (q * 32) << 16);
                    const bool live = tok_in_tile < nt && !(lane & 1);
                    const int r = tok_in_tile < nt ? p.perm[row_beg + t0 + tok_in_tile] : 0;
                    float * orow = p.out + (size_t) r * p.n_out + ft * FEAT;
                    for (int cb = 0; cb < FEAT; cb += 16) {
                        float g[16], u[16];
                        tmem_ld16(d0 + cb, g);
                        if (DUAL) tmem_ld16(d0 + 128 + cb, u);
                        float4 o[4];
                        float * of = reinterpret_cast<float *>(o);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            // hi part + lo part of the same routed row sit in adjacent lanes
                            float v = __fadd_rn(g[j], __shfl_xor_sync(0xffffffffu, g[j], 1)) * sc0;
                            if (DUAL) {
                                const float w = __fadd_rn(u[j], __shfl_xor_sync(0xffffffffu, u[j], 1)) * sc1;
                                v = __fmul_rn(ggml_silu(v), w);
                            }
                            of[j] = v;
                        }
                        if (live) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) reinterpret_cast<float4 *>(orow + cb)[j] = o[j];
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc.stage]);
                acc.template advance<2>();
            }
        }
    } else if (warp >= 8) {
        // ---------------------------------------------------------------- dequantisers
        // thread = (B tile row, half of the K = 64 step): 16 warps, so that table lookups and stores of one warp overlap
        // with the arithmetic of three others on the same scheduler
        const int dq = tid - 256;
        const int drow = dq & 255, dhalf = dq >> 8;
        uint32_t b_off[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) b_off[i] = sw128_offset(drow, 4 * dhalf + i);
        const uint32_t raw_off = (uint32_t) drow * GEMM_RAW_ROW;
        Ring raw, tile;
        for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
            const int e = p.active[item / f_tiles];
            const int n_e = p.offsets[e + 1] - p.offsets[e];
            for (int t0 = 0; t0 < n_e && !s_abort; t0 += TOK) {
                for (int kc = 0; kc < KC && !s_abort; ++kc) {
                    if (!__all_sync(0xffffffffu, wait_or_abort(&raw_full[raw.stage], raw.phase, &s_abort, p.err))) break;
                    uint32_t S[4], Q[16];          // per block: the scale word and this half's 4 qs words
                    {
                        const uint4 * src = reinterpret_cast<const uint4 *>(raws + (size_t) raw.stage * C::RAW_STAGE + raw_off);
                        uint32_t R[36];            // 4 blocks of [scale word][8 qs words]
#pragma unroll
                        for (int i = 0; i < 9; ++i) {
                            const uint4 v = src[i];
                            R[4 * i] = v.x; R[4 * i + 1] = v.y; R[4 * i + 2] = v.z; R[4 * i + 3] = v.w;
                        }
#pragma unroll
                        for (int kb = 0; kb < 4; ++kb) {
                            S[kb] = dhalf ? (R[9 * kb] >> 16) : R[9 * kb];
#pragma unroll
                            for (int w = 0; w < 4; ++w) Q[4 * kb + w] = dhalf ? R[9 * kb + 5 + w] : R[9 * kb + 1 + w];
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&raw_empty[raw.stage]);
                    raw.template advance<RS>();
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        if (!__all_sync(0xffffffffu, wait_or_abort(&tile_empty[tile.stage], tile.phase ^ 1u, &s_abort, p.err))) break;
                        uint8_t * st = tiles + (size_t) tile.stage * C::STAGE;
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const uint32_t s2u = s_scale_lut[(S[kb] >> (8 * i)) & 0xff];
                            const __half2 s2 = *reinterpret_cast<const __half2 *>(&s2u);
                            const uint32_t q0 = Q[4 * kb + 2 * i], q1 = Q[4 * kb + 2 * i + 1];
                            uint32_t h[8], h0[4], h1[4];
                            fp4_word_to_half2x4(q0, h0);
                            fp4_word_to_half2x4(q1, h1);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const __half2 v0 = __hmul2(*reinterpret_cast<const __half2 *>(&h0[j]), s2);
                                const __half2 v1 = __hmul2(*reinterpret_cast<const __half2 *>(&h1[j]), s2);
                                h[j] = *reinterpret_cast<const uint32_t *>(&v0);
                                h[4 + j] = *reinterpret_cast<const uint32_t *>(&v1);
                            }
                            // 16 halfs = two 16-byte chunks: K positions of this sub-block in unpack order
                            *reinterpret_cast<uint4 *>(st + b_off[2 * i]) = make_uint4(h[0], h[1], h[2], h[3]);
                            *reinterpret_cast<uint4 *>(st + b_off[2 * i + 1]) = make_uint4(h[4], h[5], h[6], h[7]);
                        }
                        // Every writer orders its own stores against the tensor core's (async proxy) reads and then arrives
                        // itself.  (One elected arrival per warp after __syncwarp was measured to let the MMA read rows of the
                        // last-arriving warp before they were visible.)
                        fence_async_smem();
                        mbar_arrive(&tile_full[tile.stage]);
                        tile.template advance<TS>();
                    }
                }
            }
        }
    }

    // ---- teardown: everyone meets here (all waits above are bounded), then TMEM goes back
    if (s_abort) {
        // copies that were issued but never consumed land within microseconds; give them a bounded grace period
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 3) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace b200moe
