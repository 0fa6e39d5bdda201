// tcgen05 / TMEM building blocks of the tensor-core expert path: instruction wrappers, shared-memory and instruction
// descriptors, the NVFP4 -> fp16 decode, and the kernel that prepares expert-sorted fp16 activations.
// The grouped GEMM itself is in expert_gemm.cuh.
//
// Parity mode: activations stay on the reference's int8 grid (q * d, exactly what the CPU path multiplies with).  The
// product q * d has up to 18 significant bits, so it is carried as TWO fp16 numbers hi + lo (exact for the fp16 block
// scales of Q8_0) and each K step issues the MMA twice into the same accumulator; NVFP4 weights (E2M1 value x UE4M3 block
// scale) are exact in fp16.  The MMA is kind::f16 with fp32 accumulation, so the result differs from the integer path
// only in fp32 summation order and in the tensor core's internal alignment of products (~3e-5 of RMS).  (A single fp16
// activation, 2^-12 relative, was measured at 3e-3 of RMS on `hidden` and pushed `down` past the 1e-2 bar through
// requantisation flips.)
//
// Operand roles are swapped with respect to the usual GEMM: D[feature, token] = W[feature, k] * A[token, k], so the
// fixed M = 128 of the instruction covers output features and N (16..128) covers however many rows an expert received.
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
// One warp per (sorted row, 32-element activation block).  Rows are row_stride halfs apart in both planes: K with the lo
// plane stored after the hi plane, 2K with out_lo = out_hi + K when hi and lo rows alternate.
__global__ void __launch_bounds__(256) sorted_act_fp16_kernel(ActQuant act, const int * __restrict__ perm, const int * __restrict__ meta, int rows,
                                                             int K, int n_ids, int ne11, __half * __restrict__ out_hi,
                                                             __half * __restrict__ out_lo, int row_stride) {
    pdl_wait();
    pdl_launch_dependents();

    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int nb = K / 32;
    if (warp >= rows * nb) return;
    const int i = warp / nb, b = warp % nb;
    if (i >= meta[1]) return;   // rows that are in no group (empty exchange slots) have no sorted position
    const int r = perm[i];
    const int arow = (r / n_ids) * ne11 + (r % n_ids) % ne11;
    const float d = act.d[(size_t) arow * nb + b];
    const int q = act.q[(size_t) arow * K + b * 32 + lane];
    const int e = lane & 15;                                  // position inside the 16-group
    const int pos = (e < 8) ? 2 * e : 2 * (e - 8) + 1;        // 0->0, 8->1, 1->2, 9->3, ...
    const float v = __fmul_rn((float) q, d);
    const __half hi = __float2half_rn(v);
    const size_t o = (size_t) i * row_stride + b * 32 + (lane & 16) + pos;
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

}  // namespace b200moe
