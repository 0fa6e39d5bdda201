// Grouped expert GEMM for prefill-sized batches on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// Parity mode: activations stay on the reference's int8 grid (q * d, exactly what the CPU path multiplies with).  The
// product q * d has up to 18 significant bits, so it is carried as TWO fp16 numbers hi + lo (exact for the fp16 block
// scales of Q8_0) and each K step issues the MMA twice into the same accumulator; NVFP4 weights (E2M1 value x UE4M3 block
// scale) are exact in fp16.  The MMA is kind::f16 with fp32 accumulation, so the result differs from the integer path
// only in fp32 summation order.  (A single fp16 activation, 2^-12 relative, was measured at 3e-3 of RMS on `hidden` and
// pushed `down` past the 1e-2 bar through requantisation flips.)
//
// Operand roles are swapped with respect to the usual GEMM: D[feature, token] = W[feature, k] * A[token, k], so the
// fixed M = 128 of the instruction covers output features and N (16..128) covers however many rows an expert received.
//
// One CTA (256 threads) owns a (expert, 128-feature tile) and walks that expert's rows in tiles of up to 128:
//   per K step of 64:  every thread dequantises one (feature row, tensor) block of 64 weights straight into the
//                      128B-swizzled K-major shared-memory tile, the activation tile is copied in the same layout,
//                      one thread issues 4 (x2 for gate+up) tcgen05.mma of K = 16, commit -> mbarrier frees the stage.
//   epilogue:          tcgen05.ld of the fp32 accumulators, per-expert scale, SwiGLU (gate/up) and scatter to routed rows.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"
#include "formats.cuh"
#include "router.cuh"

namespace b200moe {

// ---- tcgen05 / TMEM wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t * smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::f16, issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// all tcgen05 operations issued so far by this thread arrive on the mbarrier when they complete
__device__ __forceinline__ void umma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp receives lane (base lane + i)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows, 128B swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((smem_addr >> 4) & 0x3fff);   // start address
    d |= (uint64_t) 1 << 16;                        // leading byte offset (unused with swizzled K-major), 16-byte units
    d |= (uint64_t) (1024 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= (uint64_t) 1 << 46;                        // descriptor version of this architecture
    d |= (uint64_t) 2 << 61;                        // SWIZZLE_128B
    return d;
}
// instruction descriptor: fp16 A and B, both K-major, fp32 accumulate, M = 128, N = n
__device__ __forceinline__ uint32_t umma_idesc_f16(int n) { return (1u << 4) | ((uint32_t) (n >> 3) << 17) | ((128u >> 4) << 24); }

// byte offset of 16-byte chunk c (0..7) of row r inside a [rows][64 halfs] tile laid out for SWIZZLE_128B
__device__ __forceinline__ uint32_t sw128_offset(int r, int c) { return (uint32_t) ((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

// ---- activations for the tensor-core path --------------------------------------------------------------------------
// fp16(q * d) of the routed rows, gathered into expert order (row i of the output is routed row perm[i]) so every expert's
// rows are contiguous.  Within each group of 16 K positions the elements are stored in the order
// [0,8,1,9,2,10,3,11,4,12,5,13,6,14,7,15], the order in which the NVFP4 nibbles of a sub-block unpack.
// One warp per (sorted row, 32-element activation block).
__global__ void __launch_bounds__(256) sorted_act_fp16_kernel(ActQuant act, const int * __restrict__ perm, int rows, int K, int n_ids,
                                                             int ne11, __half * __restrict__ out_hi, __half * __restrict__ out_lo) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int nb = K / 32;
    if (warp >= rows * nb) return;
    const int i = warp / nb, b = warp % nb;
    const int r = perm[i];
    const int arow = (r / n_ids) * ne11 + (r % n_ids) % ne11;
    const float d = act.d[(size_t) arow * nb + b];
    const int q = act.q[(size_t) arow * K + b * 32 + lane];
    const int e = lane & 15;                                  // position inside the 16-group
    const int pos = (e < 8) ? 2 * e : 2 * (e - 8) + 1;        // 0->0, 8->1, 1->2, 9->3, ...
    const float v = __fmul_rn((float) q, d);
    const __half hi = __float2half_rn(v);
    const size_t o = (size_t) i * K + b * 32 + (lane & 16) + pos;
    out_hi[o] = hi;
    out_lo[o] = __float2half_rn(__fsub_rn(v, __half2float(hi)));
}

struct MmaParams {
    const uint8_t * w0;     // [n_as][n_out][row_bytes] gate (DUAL) or the single tensor
    const uint8_t * w1;     // up (DUAL)
    const float * scale0;
    const float * scale1;
    const __half * act;     // [rows sorted by expert][K]  high part of q*d
    const __half * act_lo;  // same shape, low part
    const int * offsets;    // [n_as+1]
    const int * perm;       // [rows]
    const int * active;     // [n_as]
    const int * meta;
    float * out;            // [rows][n_out] indexed by routed row
    int n_out;
    int n_as;
    int * err;
};

constexpr int MMA_THREADS = 256;

// E2M1 magnitudes as the HIGH byte of their fp16 encoding: 0, .5, 1, 1.5 | 2, 3, 4, 6 (the low byte is zero for all of them)
constexpr uint32_t FP4_F16HI_LO = 0x3e3c3800u, FP4_F16HI_HI = 0x46444240u;

// 8 nibbles of one qs word -> 8 fp16 values (E2M1 value, signed) as four half2 words in the order
// [e0,e8] [e1,e9] [e2,e10] [e3,e11] (element j and j+8 of the sub-block share a byte).
__device__ __forceinline__ void fp4_word_to_half2x4(uint32_t w, uint32_t (&h)[4]) {
    const uint32_t wn = w ^ 0x88888888u;
    const uint32_t t = (w >> 3) & 0x11111111u;                       // sign of every nibble as 0/1
    // raw selector: positives give their byte, negatives give the replicated (zero) sign of the table byte
    const uint32_t a_lo = byte_perm(FP4_F16HI_LO, FP4_F16HI_HI, w), a_hi = byte_perm(FP4_F16HI_LO, FP4_F16HI_HI, w >> 16);
    const uint32_t c_lo = byte_perm(FP4_F16HI_LO, FP4_F16HI_HI, wn), c_hi = byte_perm(FP4_F16HI_LO, FP4_F16HI_HI, wn >> 16);
    const uint32_t s_lo = byte_perm(0x00008000u, 0u, t), s_hi = byte_perm(0x00008000u, 0u, t >> 16);
    const uint32_t b_lo = a_lo | c_lo | s_lo;                        // bytes: hi(e0) hi(e8) hi(e1) hi(e9)
    const uint32_t b_hi = a_hi | c_hi | s_hi;                        //        hi(e2) hi(e10) hi(e3) hi(e11)
    h[0] = byte_perm(b_lo, 0u, 0x1404);                              // [0, b0, 0, b1]
    h[1] = byte_perm(b_lo, 0u, 0x3424);
    h[2] = byte_perm(b_hi, 0u, 0x1404);
    h[3] = byte_perm(b_hi, 0u, 0x3424);
}

// NT = token tile (N of the instruction at most): 32 for batched decode (two CTAs per SM), 128 for prefill.
template <int K, bool DUAL, int NT>
__global__ void __launch_bounds__(MMA_THREADS, (NT <= 32 ? 2 : 1)) expert_mma_nvfp4_kernel(const MmaParams p) {
    constexpr int KS = K / 64;                      // K steps
    constexpr int ROW_BYTES = K / 64 * 36;
    constexpr int NTENS = DUAL ? 2 : 1;
    constexpr int A_TILE = 128 * 128;               // 128 rows x 64 halfs
    constexpr int B_TILE = NT * 128;
    constexpr int STAGE = NTENS * A_TILE + 2 * B_TILE;   // weights, then activation hi and lo tiles
    constexpr uint32_t TMEM_COLS = (DUAL ? 2 : 1) * NT < 32 ? 32 : (DUAL ? 2 : 1) * NT;
    constexpr int BCH = (NT * 8 + MMA_THREADS - 1) / MMA_THREADS;   // activation chunks per thread and plane
    constexpr int NSB = DUAL ? 4 : 2;                               // 16-value sub-blocks per thread and K step

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t * smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    __shared__ uint64_t bar[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ uint32_t s_scale_lut[256];           // UE4M3 byte -> half2(value, value)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(&bar[0], 1);
        mbar_init(&bar[1], 1);
        mbar_fence_init();
        s_abort = 0;
    }
    {
        const __half2 h = __float2half2_rn(2.0f * ue4m3_half_to_f32(tid));   // the helper returns the value halved
        s_scale_lut[tid] = *reinterpret_cast<const uint32_t *>(&h);
    }
    if (warp == 0) {
        tmem_alloc(&s_tmem, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    const int n_active = p.meta[0];
    const int m_tiles = p.n_out / 128;
    uint32_t commits0 = 0, commits1 = 0, waits0 = 0, waits1 = 0;   // per ring stage; every commit is matched by one wait
    bool failed = false;

    // Dequant role of this thread: feature row (tid & 127) of tensor (tid >> 7) when DUAL; when single, threads 128..255
    // take the second half (32 of the 64 values) of the same row as thread tid-128.  All shared-memory offsets of the
    // thread are fixed for the whole kernel.
    const int drow = tid & 127;
    const int dsel = tid >> 7;
    const int sb0 = DUAL ? 0 : dsel * 2;
    uint32_t a_off[2 * NSB];
#pragma unroll
    for (int i = 0; i < 2 * NSB; ++i) a_off[i] = ((DUAL && dsel) ? A_TILE : 0) + sw128_offset(drow, 2 * sb0 + i);
    uint32_t b_off[BCH];
    int b_row[BCH], b_ch[BCH];
#pragma unroll
    for (int j = 0; j < BCH; ++j) {
        const int c = tid + j * MMA_THREADS;
        b_row[j] = c >> 3;
        b_ch[j] = c & 7;
        b_off[j] = NTENS * A_TILE + sw128_offset(b_row[j], b_ch[j]);
    }

    for (int item = blockIdx.x; item < n_active * m_tiles && !failed; item += gridDim.x) {
        const int a = item / m_tiles, mt = item % m_tiles;
        const int e = p.active[a];
        const int row_beg = p.offsets[e], n_e = p.offsets[e + 1] - row_beg;
        const float sc0 = p.scale0 ? p.scale0[e] : 1.0f;
        const float sc1 = (DUAL && p.scale1) ? p.scale1[e] : 1.0f;
        const uint8_t * wsrc = ((DUAL && dsel) ? p.w1 : p.w0) + ((size_t) e * p.n_out + mt * 128 + drow) * ROW_BYTES + 8 * sb0;

        for (int t0 = 0; t0 < n_e && !failed; t0 += NT) {
            const int nt = min(NT, n_e - t0);
            const int n_mma = max(16, (nt + 15) & ~15);
            const uint32_t idesc = umma_idesc_f16(n_mma);
            const uint4 * bsrc_h[BCH];
            const uint4 * bsrc_l[BCH];
#pragma unroll
            for (int j = 0; j < BCH; ++j) {
                const size_t o = (size_t) (row_beg + t0 + min(b_row[j], nt - 1)) * K;
                bsrc_h[j] = reinterpret_cast<const uint4 *>(p.act + o) + b_ch[j];
                bsrc_l[j] = reinterpret_cast<const uint4 *>(p.act_lo + o) + b_ch[j];
            }
            // Register prefetch one K step ahead: the global loads of step ks+1 are in flight while step ks is
            // dequantised and issued, so their latency is paid once per tile instead of once per step.
            uint32_t wd_n, wq_n[2 * NSB];
            uint4 bh_n[BCH], bl_n[BCH];
            auto prefetch = [&](int ks) {
                const uint8_t * blk = wsrc + ks * 36;
                wd_n = __ldg(reinterpret_cast<const uint32_t *>(blk - 8 * sb0));
#pragma unroll
                for (int i = 0; i < 2 * NSB; ++i) wq_n[i] = __ldg(reinterpret_cast<const uint32_t *>(blk + 4) + i);
#pragma unroll
                for (int j = 0; j < BCH; ++j) {
                    bh_n[j] = __ldg(bsrc_h[j] + ks * 8);
                    bl_n[j] = __ldg(bsrc_l[j] + ks * 8);
                }
            };
            prefetch(0);
            int last_stage = 0;
            for (int ks = 0; ks < KS; ++ks) {
                const int s = ks & 1;
                uint8_t * st = smem + (size_t) s * STAGE;
                const uint32_t wd = wd_n >> (8 * sb0);
                uint32_t wq[2 * NSB];
                uint4 bh[BCH], bl[BCH];
#pragma unroll
                for (int i = 0; i < 2 * NSB; ++i) wq[i] = wq_n[i];
#pragma unroll
                for (int j = 0; j < BCH; ++j) { bh[j] = bh_n[j]; bl[j] = bl_n[j]; }
                if (ks + 1 < KS) prefetch(ks + 1);
                {   // the MMAs that last read this stage must have finished
                    const bool pending = s ? (commits1 > waits1) : (commits0 > waits0);
                    if (pending) {
                        if (!mbar_wait_bounded(&bar[s], (s ? waits1 : waits0) & 1u)) { report_error(p.err, DEV_ERR_BARRIER_TIMEOUT); s_abort = 1; }
                        if (s) ++waits1; else ++waits0;
                    }
                }
                // ---- A: dequantise this thread's sub-blocks of one weight row into the swizzled tile
#pragma unroll
                for (int i = 0; i < NSB; ++i) {
                    const uint32_t s2u = s_scale_lut[(wd >> (8 * i)) & 0xff];
                    const __half2 s2 = *reinterpret_cast<const __half2 *>(&s2u);
                    uint32_t h[8], h0[4], h1[4];
                    fp4_word_to_half2x4(wq[2 * i], h0);
                    fp4_word_to_half2x4(wq[2 * i + 1], h1);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        __half2 v0 = __hmul2(*reinterpret_cast<__half2 *>(&h0[q]), s2);
                        __half2 v1 = __hmul2(*reinterpret_cast<__half2 *>(&h1[q]), s2);
                        h[q] = *reinterpret_cast<uint32_t *>(&v0);
                        h[4 + q] = *reinterpret_cast<uint32_t *>(&v1);
                    }
                    // 16 halfs = two 16-byte chunks: K positions of this sub-block in unpack order
                    *reinterpret_cast<uint4 *>(st + a_off[2 * i]) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4 *>(st + a_off[2 * i + 1]) = make_uint4(h[4], h[5], h[6], h[7]);
                }
                // ---- B: activation rows (hi and lo) of this K step; rows past the expert's last are zero
#pragma unroll
                for (int j = 0; j < BCH; ++j) {
                    if (b_row[j] < n_mma) {
                        const bool live = b_row[j] < nt;
                        *reinterpret_cast<uint4 *>(st + b_off[j]) = live ? bh[j] : make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4 *>(st + b_off[j] + B_TILE) = live ? bl[j] : make_uint4(0, 0, 0, 0);
                    }
                }
                fence_async_smem();   // make the generic-proxy writes visible to the tensor core's reads
                tc_fence_before();
                if (__syncthreads_or(s_abort)) { failed = true; break; }
                if (tid == 0) {
                    tc_fence_after();
                    const uint32_t a0 = smem_u32(st), b0 = a0 + NTENS * A_TILE;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {   // 4 x K16 = 64; 32 bytes further along the 128-byte row each
                        const uint64_t bd = umma_desc_k128(b0 + kk * 32), bl2 = umma_desc_k128(b0 + B_TILE + kk * 32);
                        const uint64_t ad = umma_desc_k128(a0 + kk * 32);
                        umma_f16(tmem, ad, bd, idesc, (ks | kk) ? 1u : 0u);
                        umma_f16(tmem, ad, bl2, idesc, 1u);
                        if (DUAL) {
                            const uint64_t ad1 = umma_desc_k128(a0 + A_TILE + kk * 32);
                            umma_f16(tmem + NT, ad1, bd, idesc, (ks | kk) ? 1u : 0u);
                            umma_f16(tmem + NT, ad1, bl2, idesc, 1u);
                        }
                    }
                    umma_commit(&bar[s]);
                }
                if (s) ++commits1; else ++commits0;
                last_stage = s;
            }
            if (failed) break;
            // ---- epilogue: wait for the last commit (it covers every MMA of this tile)
            if (!mbar_wait_bounded(&bar[last_stage], (last_stage ? waits1 : waits0) & 1u)) { report_error(p.err, DEV_ERR_BARRIER_TIMEOUT); s_abort = 1; }
            if (last_stage) ++waits1; else ++waits0;
            if (__syncthreads_or(s_abort)) { failed = true; break; }
            tc_fence_after();
            {
                const int q = warp & 3;                 // TMEM lane quarter this warp may read
                const int col_half = warp >> 2;         // warps 0-3 take the first half of the token columns, warps 4-7 the second
                constexpr int HALF = NT / 2 < 16 ? 16 : NT / 2;
                const int feature = mt * 128 + q * 32 + lane;
                for (int cb = col_half * HALF; cb < col_half * HALF + HALF && cb < n_mma; cb += 16) {
                    float g[16], u[16];
                    const uint32_t taddr = tmem + ((uint32_t) (q * 32) << 16) + cb;
                    tmem_ld16(taddr, g);
                    if (DUAL) tmem_ld16(taddr + NT, u);
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
            }
            tc_fence_before();
            __syncthreads();   // every warp has drained its accumulators before the next tile overwrites them
        }
    }

    // drain: any commit not yet waited for (bounded), then give TMEM back
    if (tid == 0) {
        while (commits0 > waits0) { if (!mbar_wait_bounded(&bar[0], waits0 & 1u, 200000000ull)) break; ++waits0; }
        while (commits1 > waits1) { if (!mbar_wait_bounded(&bar[1], waits1 & 1u, 200000000ull)) break; ++waits1; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

template <int K, bool DUAL, int NT>
constexpr size_t mma_smem_bytes() { return 2 * ((DUAL ? 2 : 1) * 128 * 128 + 2 * NT * 128) + 1024; }

}  // namespace b200moe
