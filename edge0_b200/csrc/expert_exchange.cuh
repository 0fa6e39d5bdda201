// Expert-parallel exchange, device side: routed latent rows are packed into fixed-capacity slots per destination rank, the
// owner of an expert computes on the slots it received (empty slots carry expert id -1), and the token's rank combines the rows
// that come back in slot order.  Nothing here reads a count on the host: every rank sends `capacity` slots to every peer, so the
// split sizes of the collective are equal and known before the step starts (capacity = the rank's routed rows, its worst case).
//
// Slot layout (floats): [width values of the row][expert id local to the destination rank, as int][3 words of padding]:
// slot stride (width + 4) * 4 bytes keeps rows 16-byte aligned, and the slots of all source ranks form ONE array with a
// uniform stride, so the owner reads rows and ids in place.
//
// Semantics follow edge0-strata's latent layer with one label group (src/latent/latent_moe.cpp:38-92); the reference has no
// multi-GPU form of it (its peer experts are host-staged, src/core/peer_experts.cpp:186-192).
#pragma once
#include "common.cuh"

namespace b200moe {

constexpr int EP_SLOT_EXTRA = 4;   // words behind the row: expert id + padding to 16 bytes

// every slot empty, every fill counter zero
__global__ void __launch_bounds__(256) ep_clear_kernel(float * __restrict__ slots, int n_slots, int slot_words, int width, int * __restrict__ fill,
                                                      int n_ranks) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_slots) reinterpret_cast<int *>(slots + (size_t) i * slot_words)[width] = -1;
    if (i < n_ranks) fill[i] = 0;
}

// one block per routed row r = t * k + s
__global__ void __launch_bounds__(256) ep_pack_kernel(const float * __restrict__ rows, const int32_t * __restrict__ ids, int n_routed, int k,
                                                     int width, int n_ranks, int experts_per_rank, int capacity, float * __restrict__ slots,
                                                     int32_t * __restrict__ slot_of, int * __restrict__ fill, int * err) {
    __shared__ int s_slot;
    const int r = blockIdx.x;
    if (r >= n_routed) return;
    if (threadIdx.x == 0) {
        const int e = ids[r];
        const int dest = e >= 0 ? e / experts_per_rank : -1;
        int slot = -1;
        if (dest < 0 || dest >= n_ranks) {
            report_error(err, DEV_ERR_BAD_EXPERT_ID);
        } else {
            const int pos = atomicAdd(&fill[dest], 1);
            if (pos < capacity) {
                slot = dest * capacity + pos;
                reinterpret_cast<int *>(slots + (size_t) slot * (width + EP_SLOT_EXTRA))[width] = e - dest * experts_per_rank;
            } else {
                report_error(err, DEV_ERR_BAD_SHAPE);   // cannot happen with capacity = routed rows of the rank
            }
        }
        slot_of[r] = slot;
        s_slot = slot;
    }
    __syncthreads();
    const int slot = s_slot;
    if (slot < 0) return;
    const float4 * src = reinterpret_cast<const float4 *>(rows + (size_t) (r / k) * width);
    float4 * dst = reinterpret_cast<float4 *>(slots + (size_t) slot * (width + EP_SLOT_EXTRA));
    for (int i = threadIdx.x; i < width / 4; i += blockDim.x) dst[i] = src[i];
}

// out[t][i] = sum over slots s in order of back[slot_of[t*k+s]][i] * w[t][s]: the arithmetic of combine_kernel behind an index
__global__ void __launch_bounds__(256) ep_combine_kernel(const float * __restrict__ back, const int32_t * __restrict__ slot_of,
                                                        const float * __restrict__ w, float * __restrict__ out, int n, int k, int T, int n_slots) {
    const int i4 = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (i4 * 4 >= n || t >= T) return;
    const int32_t * so = slot_of + (size_t) t * k;
    const float * wr = w + (size_t) t * k;
    float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < k; ++s) {
        const int slot = so[s];
        float4 b = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (slot >= 0 && slot < n_slots) b = reinterpret_cast<const float4 *>(back + (size_t) slot * n)[i4];
        const float ws = wr[s];
        if (s == 0) {
            a.x = __fmul_rn(b.x, ws); a.y = __fmul_rn(b.y, ws); a.z = __fmul_rn(b.z, ws); a.w = __fmul_rn(b.w, ws);
        } else {
            a.x = __fadd_rn(a.x, __fmul_rn(b.x, ws));
            a.y = __fadd_rn(a.y, __fmul_rn(b.y, ws));
            a.z = __fadd_rn(a.z, __fmul_rn(b.z, ws));
            a.w = __fadd_rn(a.w, __fmul_rn(b.w, ws));
        }
    }
    reinterpret_cast<float4 *>(out + (size_t) t * n)[i4] = a;
}

}  // namespace b200moe
