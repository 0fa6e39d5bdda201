// Shared device helpers for the sm_100a MoE-FFN kernels: mbarrier + bulk-copy (TMA 1-D) wrappers with
// bounded waits, exact fp32 helpers that reproduce the reference CPU arithmetic, warp reductions.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

// ---- device error flag -----------------------------------------------------------------------
// Kernels never trap.  A bounded wait that runs out, or an index check that fails, records a code
// here and the kernel returns; the host reads the word after synchronising.
enum DeviceError : int {
    DEV_OK = 0,
    DEV_ERR_BARRIER_TIMEOUT = 1,
    DEV_ERR_BAD_EXPERT_ID = 2,
    DEV_ERR_BAD_SHAPE = 3,
};

__device__ __forceinline__ void report_error(int * flag, int code) {
    if (flag) atomicCAS(flag, 0, code);
}

// ---- shared-memory barriers and bulk async copies ---------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t * bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Wait with a time limit (default 2 s of wall clock).  Returns false when the limit ran out; the caller
// records the error and leaves the kernel, so a copy that never lands cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t * bar, uint32_t parity, uint64_t limit_ns = 2000000000ull) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t i = 0; i < (1u << 30); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63 && global_timer_ns() - t0 > limit_ns) return false;
    }
    return false;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void * dst_smem, const void * src_gmem, uint32_t bytes, uint64_t * bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its prologue / wait for the
// previous kernel's memory to be visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- exact fp32 helpers -------------------------------------------------------------------------
// The reference CPU path is built for AVX2+FMA.  These reproduce its operation sequence with explicit
// round-to-nearest intrinsics so the compiler can neither contract nor reassociate.

// ggml_v_expf, one lane (ggml-cpu/vec.h:1215-1252 in the reference's vendored ggml).
__device__ __forceinline__ float ggml_expf(float x) {
    const float r = 0x1.8p23f;
    const float z = __fmaf_rn(x, 0x1.715476p+0f, r);
    const float n = __fsub_rn(z, r);
    const float b = __fmaf_rn(-n, 0x1.7f7d1cp-20f,
                              __fmaf_rn(-n, 0x1.62e4p-1f, x));
    const uint32_t e = __float_as_uint(z) << 23;
    const float k = __uint_as_float(e + 0x3f800000u);
    const bool c = fabsf(n) > 126.0f;
    const float u = __fmul_rn(b, b);
    const float j = __fmaf_rn(
        __fmaf_rn(__fmaf_rn(0x1.0e4020p-7f, b, 0x1.573e2ep-5f), u,
                  __fmaf_rn(0x1.555e66p-3f, b, 0x1.fffdb6p-2f)),
        u, __fmul_rn(0x1.ffffecp-1f, b));
    if (!c) return __fmaf_rn(j, k, k);
    const uint32_t g = (n <= 0.0f) ? 0x82000000u : 0u;
    const float s1 = __uint_as_float(g + 0x7f000000u);
    const float s2 = __uint_as_float(e - g);
    if (fabsf(n) > 192.0f) return __fmul_rn(s1, s1);
    return __fmul_rn(__fmaf_rn(s2, j, s2), s1);
}

// ggml_v_silu (ggml-cpu/vec.h:1255-1262): x / (1 + exp(0 - x)), IEEE division.
__device__ __forceinline__ float ggml_silu(float x) {
    const float neg_x = __fsub_rn(0.0f, x);
    return __fdiv_rn(x, __fadd_rn(1.0f, ggml_expf(neg_x)));
}

// ---- warp helpers ------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum_xor(float v, int width = 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        if (o < width) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Reduce NV per-lane partials across the lanes of a group of LW lanes (LW a power of two, LW >= NV not
// required).  On return lane (lane % LW) == i*(LW/NVr) ... holds the sum of value i, where the layout is:
// value index v lives on lane_in_group == v * (LW / min(NV, LW)) when NV <= LW.  Implemented as a halving
// butterfly: each step exchanges half of the remaining values, so the shuffle count is about NV + log2(LW/NV)
// instead of NV*log2(LW).
template <int NV, int LW>
__device__ __forceinline__ void group_reduce(float (&v)[NV], int lane_in_group) {
    static_assert((NV & (NV - 1)) == 0 && (LW & (LW - 1)) == 0, "powers of two");
    int n = NV;
    int off = LW >> 1;
#pragma unroll
    for (; n > 1 && off > 0; n >>= 1, off >>= 1) {
        const bool upper = (lane_in_group & off) != 0;
        const int h = n >> 1;
#pragma unroll
        for (int i = 0; i < NV / 2; ++i) {
            if (i < h) {
                // lower half of the lane pair keeps values [0,h), upper half keeps [h,n)
                const float send = upper ? v[i] : v[i + h];
                const float keep = upper ? v[i + h] : v[i];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
        }
    }
    // n == 1 value left per lane (or off ran out): finish with plain butterflies over the remaining lanes
#pragma unroll
    for (; off > 0; off >>= 1) {
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (i < n) v[i] += __shfl_xor_sync(0xffffffffu, v[i], off);
    }
}

// After group_reduce<NV,LW>, which value index does lane_in_group hold in v[0]?  (NV <= LW case.)
template <int NV, int LW>
__device__ __forceinline__ int group_reduce_owner_value(int lane_in_group) {
    // steps consumed bits LW/2, LW/4, ... for log2(NV) steps; bit set => upper half of the value range
    int idx = 0;
    int off = LW >> 1;
#pragma unroll
    for (int n = NV; n > 1; n >>= 1, off >>= 1) idx = (idx << 1) | ((lane_in_group & off) ? 1 : 0);
    return idx;
}

// Exact int -> float for |i| < 2^22 without the conversion unit (which issues at a fraction of the ALU rate):
// 0x4B400000 is 1.5*2^23, whose ulp is 1, so adding i to the bit pattern adds i to the value.
__device__ __forceinline__ float small_int_to_float(int i) { return __int_as_float(0x4B400000 + i) - 12582912.0f; }

}  // namespace b200moe
