// Probe of the block-scaled FP4 tensor-core instruction (tcgen05.mma kind::mxf4nvf4, one UE4M3 scale per 16 elements):
//   * one K = 256 tile product D[128, 256] = A[128, 256] * B[256, 256]^T from host-given codes and scale bytes, for checking the
//     operand formats against a host model (tests), and
//   * its sustained dense rate with operands resident in shared memory - the denominator of "% of FP4 peak".
// Operand formats (what expert_gemm_fp4.cuh relies on):
//   values   E2M1 codes, two per byte, K-major rows of 128 bytes (256 values) in the 128-byte-swizzled tile layout
//            (row r at (r / 8) * 1024 + (r % 8) * 128, 16-byte chunk c of the row at position c ^ (r % 8));
//            one instruction consumes 32 bytes (K = 64) of every row: descriptor start address + 2 per step
//   scales   UE4M3, one per 16 values = 4 bytes per row and instruction; in shared memory as 512-byte tiles of 128 rows
//            (row r at (r % 32) * 16 + (r / 32) * 4), copied by tcgen05.cp 32x128b.warpx4 into 4 tensor-memory columns per tile
#pragma once
#include "common.cuh"
#include "expert_gemm_fp4.cuh"
#include "expert_mma.cuh"

namespace b200moe {

constexpr int PROBE_NB = 256;
constexpr int PROBE_A_BYTES = 128 * 128, PROBE_B_BYTES = PROBE_NB * 128, PROBE_SFA_BYTES = 4 * 512, PROBE_SFB_BYTES = 4 * (PROBE_NB / 128) * 512;
constexpr int PROBE_TILE_BYTES = PROBE_A_BYTES + PROBE_B_BYTES + PROBE_SFA_BYTES + PROBE_SFB_BYTES;
constexpr int PROBE_SMEM = PROBE_TILE_BYTES + 1024;

// rounds == 0: one pass over K = 256 (4 instructions, N = 256), D -> out[128][256].
// rounds > 0: `rounds` passes of 4 * n_acc instructions of width n_mma that alternate between n_acc accumulators; nothing is read back.
__global__ void __launch_bounds__(128, 1) fp4_probe_kernel(const uint8_t * __restrict__ tiles, float * __restrict__ out, int rounds, int n_mma,
                                                          int n_acc, int * err) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t * sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t s_tmem;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    const uint4 * src = reinterpret_cast<const uint4 *>(tiles);
    for (int i = tid; i < PROBE_TILE_BYTES / 16; i += 128) reinterpret_cast<uint4 *>(sm)[i] = src[i];
    fence_async_smem();
    if (warp == 0) { tmem_alloc(&s_tmem, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t a_addr = smem_u32(sm), b_addr = a_addr + PROBE_A_BYTES, sfa_addr = b_addr + PROBE_B_BYTES, sfb_addr = sfa_addr + PROBE_SFA_BYTES;
    const int width = rounds == 0 ? PROBE_NB : n_mma, accs = rounds == 0 ? 1 : n_acc;
    const uint32_t idesc = umma_idesc_fp4(width);
    const uint32_t sf_col = (uint32_t) (accs * width);          // scale factors behind the accumulators: 4 + 8 columns per step, reused
    if (tid == 0) {
        const uint32_t a_lo = DESC_LO | (a_addr >> 4), b_lo = DESC_LO | (b_addr >> 4);
        for (int kb = 0; kb < 4; ++kb) {
            tmem_cp_sf(tmem + sf_col + 12 * kb, sfa_addr + kb * 512);
            tmem_cp_sf(tmem + sf_col + 12 * kb + 4, sfb_addr + kb * 1024);
            tmem_cp_sf(tmem + sf_col + 12 * kb + 8, sfb_addr + kb * 1024 + 512);
        }
        const int passes = rounds == 0 ? 1 : rounds;
        for (int r = 0; r < passes; ++r)
            for (int kb = 0; kb < 4; ++kb)
                for (int a = 0; a < accs; ++a)
                    umma_fp4(tmem + (uint32_t) (a * width), a_lo + 2 * kb, b_lo + 2 * kb, DESC_HI, idesc, tmem + sf_col + 12 * kb,
                             tmem + sf_col + 12 * kb + 4, r > 0 || kb > 0);
        umma_commit(&bar);
    }
    __syncwarp();
    if (!mbar_wait_bounded(&bar, 0, 8000000000ull) && lane == 0) report_error(err, DEV_ERR_BARRIER_TIMEOUT);
    __syncwarp();
    tc_fence_after();
    if (rounds == 0 && blockIdx.x == 0) {
        for (int cb = 0; cb < PROBE_NB; cb += 16) {
            float v[16];
            tmem_ld16(tmem + ((uint32_t) (warp * 32) << 16) + cb, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) out[(size_t) (warp * 32 + lane) * PROBE_NB + cb + j] = v[j];
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 512);
}

// host: codes [rows][256] (one E2M1 code per byte), scale bytes [rows][16] -> the device tile image
inline void fp4_probe_pack(const uint8_t * a, const uint8_t * b, const uint8_t * sfa, const uint8_t * sfb, uint8_t * tiles) {
    memset(tiles, 0, PROBE_TILE_BYTES);
    auto put = [&](uint8_t * base, const uint8_t * codes, int rows) {
        for (int r = 0; r < rows; ++r)
            for (int j = 0; j < 128; ++j)
                base[(size_t) (r >> 3) * 1024 + (r & 7) * 128 + (((j >> 4) ^ (r & 7)) << 4) + (j & 15)] =
                    (uint8_t) ((codes[r * 256 + 2 * j] & 15) | ((codes[r * 256 + 2 * j + 1] & 15) << 4));
    };
    put(tiles, a, 128);
    put(tiles + PROBE_A_BYTES, b, PROBE_NB);
    for (int kb = 0; kb < 4; ++kb) {
        for (int r = 0; r < 128; ++r)
            for (int s = 0; s < 4; ++s) tiles[PROBE_A_BYTES + PROBE_B_BYTES + kb * 512 + sf_tile_offset(r) + s] = sfa[r * 16 + 4 * kb + s];
        for (int r = 0; r < PROBE_NB; ++r)
            for (int s = 0; s < 4; ++s)
                tiles[PROBE_A_BYTES + PROBE_B_BYTES + PROBE_SFA_BYTES + kb * 1024 + (r / 128) * 512 + sf_tile_offset(r % 128) + s] = sfb[r * 16 + 4 * kb + s];
    }
}

}  // namespace b200moe
