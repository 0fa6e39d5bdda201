// Warp-specialised grouped expert GEMM on tcgen05 (accumulators in TMEM) for NVFP4 weights.
//
// Same arithmetic contract as expert_mma.cuh (activations stay on the reference's int8 grid as fp16 hi + lo planes,
// NVFP4 weights exact in fp16, kind::f16 with fp32 accumulation, D[feature, token] = W[feature, k] * A[token, k]),
// but every stage of the pipeline has its own warps, so no warp ever waits for global memory:
//
//   warp 0        raw-weight producer: one thread issues tiled TMA loads of [128 feature rows][144 bytes] boxes
//                 (256 K positions per row, block_nvfp4 bytes as they lie in HBM) into a ring of raw stages
//   warp 1        activation producer: one thread issues tiled TMA loads of the fp16 hi / lo tiles (128-byte rows,
//                 SWIZZLE_128B) straight into the operand ring
//   warp 2        MMA issuer: one thread issues tcgen05.mma for each K = 64 operand stage and commits to mbarriers
//   warp 3        owns the TMEM allocation
//   warps 4-7     epilogue: tcgen05.ld of a finished accumulator, per-expert scale, SwiGLU, scatter to routed rows,
//                 overlapped with the next tile's main loop through two accumulator buffers
//   warps 8-15    dequantisers: each thread turns the 64 (gate+up) or 32 (single tensor) weights of its feature row
//                 into fp16 in the 128B-swizzled K-major operand tile
//
// Rings and their barriers (count of arrivals that complete a phase):
//   raw_full[RS]  (1 + bytes)  producer arms with the byte count      raw_empty[RS]  (8)  one arrival per dequant warp
//   tile_full[TS] (256 + 1 + bytes) dequant threads + activation producer  tile_empty[TS] (1)  tcgen05.commit
//   acc_full[2]   (1)  tcgen05.commit after the last K step           acc_empty[2]   (4)  one arrival per epilogue warp
// Every wait is bounded in time and also gives up as soon as any role has reported a failure.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "expert_mma.cuh"
#include "formats.cuh"

namespace b200moe {

__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// tiled 2-D TMA load (no multicast); x counts elements of the innermost dimension and must keep the copy 16-byte aligned
__device__ __forceinline__ void tma_load_2d(void * dst_smem, const CUtensorMap * map, int x, int y, uint64_t * bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}

// Bounded wait that also returns when another role has given up; reports a timeout itself.
// SLEEP_NS > 0: the warp sleeps between polls.  A polling warp otherwise competes for issue slots with the dequantising
// warps of its scheduler (measured: more than half of all issued instructions were polls); roles that wait most of the
// time (producers, epilogue, MMA issuer) therefore back off.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool wait_or_abort(uint64_t * bar, uint32_t parity, volatile int * abort_flag, int * err) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t i = 0; i < (1u << 30); ++i) {
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > 2000000000ull) {
                report_error(err, DEV_ERR_BARRIER_TIMEOUT);
                *abort_flag = 1;
                return false;
            }
        }
    }
    *abort_flag = 1;
    return false;
}

// The shared-memory descriptor of umma_desc_k128 split into its constant high word and the low word without the address.
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // stride between 8-row groups, version, SWIZZLE_128B
constexpr uint32_t DESC_LO = 1u << 16;                                  // leading byte offset (unused for swizzled K-major)

// D[tmem] (+)= A * B with descriptors given as (low word, shared high word); `accumulate` is a run-time flag
__device__ __forceinline__ void umma_f16_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"((uint32_t) accumulate)
        : "memory");
}
// same, always accumulating
__device__ __forceinline__ void umma_f16_acc(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc)
        : "memory");
}

struct Ring {
    int stage = 0;
    uint32_t phase = 0;
    template <int N>
    __device__ __forceinline__ void advance() {
        if (++stage == N) { stage = 0; phase ^= 1u; }
    }
};

constexpr int GEMM_THREADS = 512;
constexpr int GEMM_RAW_K = 256;                    // K positions per raw stage
constexpr int GEMM_RAW_ROW = GEMM_RAW_K / 64 * 36;  // 144 bytes of one feature row

template <int K, bool DUAL, int NT>
struct GemmCfg {
    static constexpr int NTENS = DUAL ? 2 : 1;
    static constexpr int A_TILE = 128 * 128;                        // 128 features x 64 halfs
    static constexpr int B_TILE = NT * 128;
    static constexpr int STAGE = NTENS * A_TILE + 2 * B_TILE;       // weights, activation hi, activation lo
    static constexpr int RAW_STAGE = NTENS * 128 * GEMM_RAW_ROW;
    static constexpr int BUDGET = 200 * 1024;
    static constexpr int RS = 2;
    static constexpr int TS_FIT = (BUDGET - RS * RAW_STAGE) / STAGE;
    static constexpr int TS = TS_FIT > 4 ? 4 : TS_FIT;
    static constexpr uint32_t TMEM_COLS = 2 * NTENS * NT < 32 ? 32 : 2 * NTENS * NT;
    static_assert(TS >= 2, "operand ring needs two stages");
    static_assert(K % GEMM_RAW_K == 0, "K must be a multiple of 256");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns must be a power of two up to 512");
    static constexpr size_t SMEM = (size_t) TS * STAGE + (size_t) RS * RAW_STAGE + 1024;
};

template <int K, bool DUAL, int NT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
expert_gemm_nvfp4_kernel(const MmaParams p, const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                         const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo) {
    using C = GemmCfg<K, DUAL, NT>;
    constexpr int NTENS = C::NTENS, TS = C::TS, RS = C::RS;
    constexpr int KC = K / GEMM_RAW_K;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t * tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint8_t * raws = tiles + (size_t) TS * C::STAGE;
    __shared__ uint64_t raw_full[RS], raw_empty[RS], tile_full[TS], tile_empty[TS], acc_full[2], acc_empty[2];
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;
    __shared__ uint32_t s_scale_lut[256];           // UE4M3 byte -> half2(value, value)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < RS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 8); }
        for (int i = 0; i < TS; ++i) { mbar_init(&tile_full[i], 256 + 1); mbar_init(&tile_empty[i], 1); }
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
    const int m_tiles = p.n_out / 128;
    const int n_items = n_active * m_tiles;

    if (warp == 0) {
        // ---------------------------------------------------------------- raw weight producer
        if (lane == 0) {
            Ring raw;
            for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
                const int a = item / m_tiles, mt = item % m_tiles;
                const int e = p.active[a];
                const int n_e = p.offsets[e + 1] - p.offsets[e];
                const int row0 = e * p.n_out + mt * 128;
                for (int t0 = 0; t0 < n_e && !s_abort; t0 += NT) {
                    for (int kc = 0; kc < KC; ++kc) {
                        if (!wait_or_abort<200>(&raw_empty[raw.stage], raw.phase ^ 1u, &s_abort, p.err)) break;
                        uint8_t * dst = raws + (size_t) raw.stage * C::RAW_STAGE;
                        mbar_arrive_expect_tx(&raw_full[raw.stage], C::RAW_STAGE);
                        tma_load_2d(dst, &map_w0, kc * GEMM_RAW_ROW, row0, &raw_full[raw.stage]);
                        if (DUAL) tma_load_2d(dst + 128 * GEMM_RAW_ROW, &map_w1, kc * GEMM_RAW_ROW, row0, &raw_full[raw.stage]);
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
                const int e = p.active[item / m_tiles];
                const int row_beg = p.offsets[e], n_e = p.offsets[e + 1] - row_beg;
                for (int t0 = 0; t0 < n_e && !s_abort; t0 += NT) {
                    for (int ks = 0; ks < K / 64; ++ks) {
                        if (!wait_or_abort<100>(&tile_empty[tile.stage], tile.phase ^ 1u, &s_abort, p.err)) break;
                        uint8_t * st = tiles + (size_t) tile.stage * C::STAGE + NTENS * C::A_TILE;
                        mbar_arrive_expect_tx(&tile_full[tile.stage], 2 * C::B_TILE);
                        tma_load_2d(st, &map_hi, ks * 64, row_beg + t0, &tile_full[tile.stage]);
                        tma_load_2d(st + C::B_TILE, &map_lo, ks * 64, row_beg + t0, &tile_full[tile.stage]);
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
                const int e = p.active[item / m_tiles];
                const int n_e = p.offsets[e + 1] - p.offsets[e];
                for (int t0 = 0; t0 < n_e && !s_abort; t0 += NT) {
                    const int nt = min(NT, n_e - t0);
                    const int n_mma = max(16, (nt + 15) & ~15);
                    const uint32_t idesc = umma_idesc_f16(n_mma);
                    if (!wait_or_abort<40>(&acc_empty[acc.stage], acc.phase ^ 1u, &s_abort, p.err)) break;
                    tc_fence_after();
                    const uint32_t d0 = tmem + (uint32_t) acc.stage * (NTENS * NT);
                    for (int ks = 0; ks < K / 64; ++ks) {
                        if (!wait_or_abort<40>(&tile_full[tile.stage], tile.phase, &s_abort, p.err)) break;
                        tc_fence_after();
                        // Descriptors differ only in their 14-bit start-address field (16-byte units): one 32-bit add each.
                        const uint32_t da = DESC_LO | (smem_u32(tiles + (size_t) tile.stage * C::STAGE) >> 4);
                        constexpr uint32_t OFF_A1 = C::A_TILE >> 4, OFF_BH = (NTENS * C::A_TILE) >> 4, OFF_BL = OFF_BH + (C::B_TILE >> 4);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {   // 4 x K16 = 64; 32 bytes (2 units) further along the 128-byte row each
                            if (kk == 0) umma_f16_lohi(d0, da, da + OFF_BH, DESC_HI, idesc, ks != 0);
                            else umma_f16_acc(d0, da + 2 * kk, da + OFF_BH + 2 * kk, DESC_HI, idesc);
                            umma_f16_acc(d0, da + 2 * kk, da + OFF_BL + 2 * kk, DESC_HI, idesc);
                            if (DUAL) {
                                if (kk == 0) umma_f16_lohi(d0 + NT, da + OFF_A1, da + OFF_BH, DESC_HI, idesc, ks != 0);
                                else umma_f16_acc(d0 + NT, da + OFF_A1 + 2 * kk, da + OFF_BH + 2 * kk, DESC_HI, idesc);
                                umma_f16_acc(d0 + NT, da + OFF_A1 + 2 * kk, da + OFF_BL + 2 * kk, DESC_HI, idesc);
                            }
                        }
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
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
            const int a = item / m_tiles, mt = item % m_tiles;
            const int e = p.active[a];
            const int row_beg = p.offsets[e], n_e = p.offsets[e + 1] - row_beg;
            const float sc0 = p.scale0 ? p.scale0[e] : 1.0f;
            const float sc1 = (DUAL && p.scale1) ? p.scale1[e] : 1.0f;
            const int feature = mt * 128 + q * 32 + lane;
            for (int t0 = 0; t0 < n_e && !s_abort; t0 += NT) {
                const int nt = min(NT, n_e - t0);
                // lanes leave the polling loop one by one: the vote reconverges the warp (tcgen05.ld below needs all of it)
                // and makes the outcome uniform
                if (!__all_sync(0xffffffffu, wait_or_abort<200>(&acc_full[acc.stage], acc.phase, &s_abort, p.err))) break;
                tc_fence_after();
                const uint32_t d0 = tmem + (uint32_t) acc.stage * (NTENS * NT) + ((uint32_t) (q * 32) << 16);
                for (int cb = 0; cb < nt; cb += 16) {
                    float g[16], u[16];
                    tmem_ld16(d0 + cb, g);
                    if (DUAL) tmem_ld16(d0 + NT + cb, u);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = cb + j;
                        if (t < nt) {
                            const int r = p.perm[row_beg + t0 + t];
                            float v = g[j] * sc0;
                            if (DUAL) v = __fmul_rn(ggml_silu(v), u[j] * sc1);
                            p.out[(size_t) r * p.n_out + feature] = v;
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
        const int dq = tid - 256;
        const int drow = dq & 127, dsel = dq >> 7;
        // DUAL: thread = (tensor dsel, feature row drow), all 4 sub-blocks of the K = 64 step.
        // single: thread = (half dsel of the step, feature row drow), sub-blocks 2*dsel and 2*dsel + 1.
        constexpr int NSB = DUAL ? 4 : 2;
        const int sb0 = DUAL ? 0 : dsel * 2;
        uint32_t a_off[2 * NSB];
#pragma unroll
        for (int i = 0; i < 2 * NSB; ++i) a_off[i] = ((DUAL && dsel) ? C::A_TILE : 0) + sw128_offset(drow, 2 * sb0 + i);
        const uint32_t raw_off = ((DUAL ? dsel : 0) * 128 + drow) * GEMM_RAW_ROW;
        Ring raw, tile;
        for (int item = blockIdx.x; item < n_items && !s_abort; item += gridDim.x) {
            const int e = p.active[item / m_tiles];
            const int n_e = p.offsets[e + 1] - p.offsets[e];
            for (int t0 = 0; t0 < n_e && !s_abort; t0 += NT) {
                for (int kc = 0; kc < KC && !s_abort; ++kc) {
                    if (!__all_sync(0xffffffffu, wait_or_abort(&raw_full[raw.stage], raw.phase, &s_abort, p.err))) break;
                    uint32_t R[36];                // 4 blocks of [scale word][8 qs words]
                    {
                        const uint4 * src = reinterpret_cast<const uint4 *>(raws + (size_t) raw.stage * C::RAW_STAGE + raw_off);
#pragma unroll
                        for (int i = 0; i < 9; ++i) {
                            const uint4 v = src[i];
                            R[4 * i] = v.x; R[4 * i + 1] = v.y; R[4 * i + 2] = v.z; R[4 * i + 3] = v.w;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&raw_empty[raw.stage]);
                    raw.template advance<RS>();
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        if (!__all_sync(0xffffffffu, wait_or_abort(&tile_empty[tile.stage], tile.phase ^ 1u, &s_abort, p.err))) break;
                        uint8_t * st = tiles + (size_t) tile.stage * C::STAGE;
                        const uint32_t wd = R[9 * kb] >> (8 * sb0);
#pragma unroll
                        for (int i = 0; i < NSB; ++i) {
                            const uint32_t s2u = s_scale_lut[(wd >> (8 * i)) & 0xff];
                            const __half2 s2 = *reinterpret_cast<const __half2 *>(&s2u);
                            uint32_t h[8], h0[4], h1[4];
                            // register indices must be compile-time: pick the half by selection, not by indexing
                            const uint32_t q0 = (!DUAL && dsel) ? R[9 * kb + 5 + 2 * i] : R[9 * kb + 1 + 2 * i];
                            const uint32_t q1 = (!DUAL && dsel) ? R[9 * kb + 6 + 2 * i] : R[9 * kb + 2 + 2 * i];
                            fp4_word_to_half2x4(q0, h0);
                            fp4_word_to_half2x4(q1, h1);
#pragma unroll
                            for (int w = 0; w < 4; ++w) {
                                __half2 v0 = __hmul2(*reinterpret_cast<__half2 *>(&h0[w]), s2);
                                __half2 v1 = __hmul2(*reinterpret_cast<__half2 *>(&h1[w]), s2);
                                h[w] = *reinterpret_cast<uint32_t *>(&v0);
                                h[4 + w] = *reinterpret_cast<uint32_t *>(&v1);
                            }
                            *reinterpret_cast<uint4 *>(st + a_off[2 * i]) = make_uint4(h[0], h[1], h[2], h[3]);
                            *reinterpret_cast<uint4 *>(st + a_off[2 * i + 1]) = make_uint4(h[4], h[5], h[6], h[7]);
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
    // (normal path: the epilogue has waited for every accumulator commit, which covers every MMA issued)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 3) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace b200moe
