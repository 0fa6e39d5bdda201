// Grouped expert GEMM on the block-scaled FP4 tensor-core instruction (tcgen05.mma kind::mxf4nvf4, one UE4M3 scale per 16
// elements, fp32 accumulators in tensor memory) for NVFP4 experts in batched decode.
//
// Why it fits: ggml's block_nvfp4 IS the operand format of that instruction - E2M1 codes, one UE4M3 scale per 16 elements
// (ggml-common.h:221-227; the doubled code table and the halved scale decode of ggml-impl.h:514-527 cancel).  A weight row
// needs no arithmetic at all before the MMA: the 4 scale bytes in front of every 32 code bytes are stripped while the row moves
// from the raw TMA stage into the 128B-swizzled K-major operand tile, and collected as the scale-factor tile that tcgen05.cp
// copies into tensor memory.  Element order inside a 16-block does not matter as long as both operands agree on it, so the
// activations are simply stored in ggml's nibble order (byte j = elements j and j+8 of the block).
//
// Activations stay on the reference's int8 grid (q * d with d an fp16 number per 32 elements, the Q8_0 rows the CPU path
// multiplies with).  With d = M * 2^e (M an 11-bit integer) the product q * M is an 18-bit integer; its seven balanced
// radix-8 digits (each in [-4, 4], all E2M1 values) are seven "planes" of one routed row, and 2^e - relative to the row's
// largest block exponent - is a power of two that UE4M3 holds exactly.  So
//     x_hat[k] = 2^(E_row - 8) * sum_p 8^p * digit_p[k] * sf[k / 16]
// is exact (blocks more than 17 binades below the row's largest flush to zero: a relative 2^-17 of the row's unit), every
// product inside the tensor core is exact, and the result differs from the integer path only by fp32 accumulation.
//
// Operand roles: D[feature, plane] = W[feature, k] * P[plane, k].  M = 128 weight rows, N = 7 planes x up to 14 routed rows
// (N = 8 .. 104), K = 64 per instruction.  The seven plane columns of a routed row sit next to each other in one lane of tensor
// memory, so the epilogue recombines them with a Horner chain in registers and stores 32 consecutive features per warp.
// Two weight tiles are in flight per stage with an accumulator each (gate and up rows of the same 128 features, or two
// consecutive 128-row tiles of `down`): dependent MMAs on one accumulator issue every ~190-230 cycles, MMAs that alternate
// between two accumulators every ~116 (measured with the probe kernel in fp4_probe.cuh).
//
// Roles (every wait bounded, as in expert_gemm.cuh):
//   warp 0      raw-weight producer: tiled TMA of [128 rows][144 bytes] boxes (K = 256 per row) of both tiles
//   warp 1      activation producer: one tiled TMA box [98 plane rows][128 bytes] + one bulk copy of the 2 KB scale tile, into a
//               ring of its own that runs three stages ahead (the planes come from L2 with about a microsecond of latency)
//   warp 2      MMA issuer: per K = 64 step three tcgen05.cp (scales of tile 0, tile 1, planes) and two tcgen05.mma
//   warp 3      owns tensor memory
//   warps 4-7   epilogue
//   warps 8-15  repack: thread = one weight row of one tile; 9 x 16-byte loads, 8 x 16-byte stores, 4 scale words
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "expert_gemm.cuh"
#include "expert_mma.cuh"
#include "formats.cuh"

namespace b200moe {

constexpr int FP4_PLANES = 7;
constexpr int FP4_RPT = TOKEN_TILE_ROWS;          // 14 routed rows per token tile
constexpr int FP4_NROW = FP4_PLANES * FP4_RPT;    // 98 plane rows per token tile
constexpr int FP4_NCOL = 104;                     // accumulator columns per weight tile: N of the instruction is a multiple of 8
constexpr int FP4_SF_TILE = 4 * 512;              // scale factors of 128 rows for the four K = 64 steps of a stage
constexpr int FP4_THREADS = 512;

__device__ __forceinline__ void umma_fp4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                         bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %7, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], da, db, %4, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"((uint32_t) accumulate)
        : "memory");
}
// shared memory -> tensor memory: 32 rows x 16 bytes, replicated to the four lane quarters (the layout the MMA reads scales from)
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint32_t smem_addr) {
    // matrix descriptor without swizzle: 8-row groups of 16-byte rows, 128 bytes apart
    const uint64_t desc = (uint64_t) ((smem_addr >> 4) & 0x3fff) | ((uint64_t) (128 >> 4) << 32) | ((uint64_t) 1 << 46);
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
// instruction descriptor: E2M1 x E2M1, UE4M3 scales, both operands K-major, M = 128, N = n (a multiple of 8)
__host__ __device__ constexpr uint32_t umma_idesc_fp4(int n) { return (1u << 7) | (1u << 10) | ((uint32_t) (n >> 3) << 17) | ((128u >> 4) << 24); }
// byte offset of the 4 scale bytes of row r (0..127) inside the 512-byte scale tile of one K = 64 step
__host__ __device__ constexpr uint32_t sf_tile_offset(int r) { return (uint32_t) ((r & 31) * 16 + (r >> 5) * 4); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
        "%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- activation planes ---------------------------------------------------------------------------------------------------
// Expert-sorted routed row i -> seven plane rows 7i .. 7i+6 of `planes` (K/2 bytes each, ggml nibble order inside every
// 16-block), its scale bytes in the scale tiles of its token tile, and the power of two the epilogue multiplies with.
//   tile_of_expert[e]: index of expert e's first token tile (prefix of ceil(rows_e / 14)); tile_expert[tile]: the inverse
//   sf tiles: [tile][K / 256][4 steps][512 bytes], byte for (plane row n of the tile, 16-block g of the step) at sf_tile_offset(n) + g
struct PlaneOut {
    uint8_t * planes;       // [rows * 7][K / 2]
    uint8_t * sf;           // [tiles][K / 256][2048]
    float *   row_scale;    // [rows] by sorted position
    int *     tile_expert;  // [tiles] expert of every token tile
};

// digits, codes and scale bytes of one quad: 16-block g, bytes j0 .. j0+3 (elements 16g + j and 16g + j + 8) with int8 values lo[], hi[]
// and the fp32 bits of the block scale d (an fp16 number: d = M * 2^(exp8 - 137) with M the top 11 bits of the significand).
// The four code bytes of every plane leave as one 32-bit store.
__device__ __forceinline__ void plane_quad(const int (&lo)[4], const int (&hi)[4], uint32_t dbits, int E_row, int g, int j0, int K, int in_tile,
                                           uint8_t * __restrict__ prow, uint8_t * __restrict__ sft) {
    const bool nz = (dbits & 0x7fffffffu) != 0;
    const int M = nz ? (int) (((dbits & 0x7fffffu) | 0x800000u) >> 13) : 0;
    const int s = nz ? (int) ((dbits >> 23) & 0xff) - 137 - E_row + 8 : -100;           // scale exponent, at most 8
    const int Ms = s >= -9 ? M : 0;                                                     // flushed blocks contribute nothing
    int p0[4], p1[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) { p0[m] = lo[m] * Ms; p1[m] = hi[m] * Ms; }
    uint32_t * pw = reinterpret_cast<uint32_t *>(prow + 8 * g + j0);
    // Balanced radix-8 digits, lowest first: digit = ((p + 4) & 7) - 4 and carry (p + 4) >> 3.  The digit's E2M1 code comes from
    // a table indexed by p & 7 (residues 0..3 are the digits 0..3, residues 4..7 the digits -4..-1): codes 0,2,4,5 and, with the
    // sign bit, E,D,C,A.  The top plane takes what is left (|p| <= 4) through the magnitude table 0,2,4,5,6.
#pragma unroll
    for (int p = 0; p < FP4_PLANES; ++p) {
        uint32_t word = 0;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            uint32_t c0, c1;
            if (p < FP4_PLANES - 1) {
                c0 = (0xACDE5420u >> (4 * (p0[m] & 7))) & 0xfu;
                c1 = (0xACDE5420u >> (4 * (p1[m] & 7))) & 0xfu;
                p0[m] = (p0[m] + 4) >> 3;
                p1[m] = (p1[m] + 4) >> 3;
            } else {
                c0 = ((0x65420u >> (4 * abs(p0[m]))) & 0xfu) | (p0[m] < 0 ? 8u : 0u);
                c1 = ((0x65420u >> (4 * abs(p1[m]))) & 0xfu) | (p1[m] < 0 ? 8u : 0u);
            }
            word |= (c0 | (c1 << 4)) << (8 * m);
        }
        pw[(size_t) p * (K / 8)] = word;
    }
    if (j0 == 0) {
        // UE4M3 byte of 2^s: normal for s >= -6, the three power-of-two subnormals below, zero when flushed
        const uint32_t sb = s >= -6 ? (uint32_t) (s + 7) << 3 : s == -7 ? 4u : s == -8 ? 2u : s == -9 ? 1u : 0u;
        uint8_t * dst = sft + (size_t) (g >> 4) * FP4_SF_TILE + ((g >> 2) & 3) * 512 + (g & 3);
#pragma unroll
        for (int p = 0; p < FP4_PLANES; ++p) dst[sf_tile_offset(in_tile * FP4_PLANES + p)] = (uint8_t) sb;
    }
}

// K / 8 threads per expert-sorted routed row (at most 256: a block holds 256 * 8 / K rows, and a thread two quads when K = 4096).
// SRC_F32 = false: the row's activations are already quantised (ActQuant planes, Q8_0).
// SRC_F32 = true: they are fp32 (`src`, rows `src_stride` floats apart) and are quantised here exactly as quantize_q8_0_block
// does it (d = half(amax / 127), q = rint(v * (127 / amax))), which saves the separate quantisation pass; `emit`, when it has
// planes, receives that quantised form as well (row index as in `src`).
template <bool SRC_F32>
__global__ void __launch_bounds__(256) act_planes_kernel(ActQuant act, const float * __restrict__ src, int64_t src_stride,
                                                        const int * __restrict__ perm, const int32_t * __restrict__ ids,
                                                        const int * __restrict__ offsets, const int * __restrict__ tile_of_expert,
                                                        const int * __restrict__ meta, int rows, int K, int n_ids, int ne11, int n_as,
                                                        PlaneOut out, ActQuant emit) {
    constexpr int MAX_QUADS = 2;
    __shared__ int s_E[8];
    const int tid = threadIdx.x, lane = tid & 31;
    const int tpr = min(256, K / 8), rpb = 256 / tpr, qpt = (K / 8) / tpr;
    const int lrow = tid / tpr, t_in = tid % tpr;
    const int i = blockIdx.x * rpb + lrow;          // sorted position
    if (tid < 8) s_E[tid] = -1000;
    __syncthreads();
    // meta[1]: rows that are in a group (fewer than `rows` when slots are empty); threads beyond the block's last whole row idle (K = 768)
    const bool live = lrow < rpb && i < rows && i < meta[1];
    int arow = 0, in_tile = 0, tile = 0;
    if (live) {
        const int r = perm[i];
        arow = (r / n_ids) * ne11 + (r % n_ids) % ne11;
        int e = ids[r];
        e = e < 0 ? 0 : (e >= n_as ? n_as - 1 : e);    // bad ids were reported by the grouping kernels; stay inside the tables
        const int row_beg = offsets[e];
        in_tile = (i - row_beg) % FP4_RPT;
        tile = tile_of_expert[e] + (i - row_beg) / FP4_RPT;
        if (in_tile == 0 && t_in == 0) out.tile_expert[tile] = e;
    }
    const int nb32 = K / 32;
    int lo[MAX_QUADS][4], hi[MAX_QUADS][4];
    uint32_t db[MAX_QUADS];
    int emax = -1000;
#pragma unroll
    for (int u = 0; u < MAX_QUADS; ++u) {
        db[u] = 0u;
        if (u < qpt && live) {
            const int qd = t_in + tpr * u, g = qd >> 1, j0 = (qd & 1) * 4;
            if (SRC_F32) {
                const float * xrow = src + (size_t) arow * src_stride + 16 * g + j0;
                const float4 a = *reinterpret_cast<const float4 *>(xrow), b = *reinterpret_cast<const float4 *>(xrow + 8);
                const float va[4] = { a.x, a.y, a.z, a.w }, vb[4] = { b.x, b.y, b.z, b.w };
                float amax = 0.0f;
#pragma unroll
                for (int m = 0; m < 4; ++m) amax = fmaxf(amax, fmaxf(fabsf(va[m]), fabsf(vb[m])));
                // the four quads of a 32-block sit in four consecutive lanes (all live or none: a row never splits a warp)
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                const float d = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
                const float id = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    lo[u][m] = __float2int_rn(__fmul_rn(va[m], id));
                    hi[u][m] = __float2int_rn(__fmul_rn(vb[m], id));
                }
                db[u] = __float_as_uint(d);
                if (emit.q) {
                    int8_t * qo = emit.q + (size_t) arow * K + 16 * g + j0;
                    *reinterpret_cast<uint32_t *>(qo) = (uint32_t) (lo[u][0] & 0xff) | ((uint32_t) (lo[u][1] & 0xff) << 8) |
                                                        ((uint32_t) (lo[u][2] & 0xff) << 16) | ((uint32_t) (lo[u][3] & 0xff) << 24);
                    *reinterpret_cast<uint32_t *>(qo + 8) = (uint32_t) (hi[u][0] & 0xff) | ((uint32_t) (hi[u][1] & 0xff) << 8) |
                                                            ((uint32_t) (hi[u][2] & 0xff) << 16) | ((uint32_t) (hi[u][3] & 0xff) << 24);
                    if ((qd & 3) == 0) emit.d[(size_t) arow * nb32 + (g >> 1)] = d;
                }
            } else {
                const int8_t * qrow = act.q + (size_t) arow * K + 16 * g + j0;
                const uint32_t wa = *reinterpret_cast<const uint32_t *>(qrow), wb = *reinterpret_cast<const uint32_t *>(qrow + 8);
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    lo[u][m] = (int) (int8_t) (wa >> (8 * m));
                    hi[u][m] = (int) (int8_t) (wb >> (8 * m));
                }
                db[u] = __float_as_uint(act.d[(size_t) arow * nb32 + (g >> 1)]);
            }
            if (db[u] & 0x7fffffffu) emax = max(emax, (int) ((db[u] >> 23) & 0xff) - 137);
        } else if (SRC_F32 && u < qpt) {   // keep the warp's shuffles uniform
            __shfl_xor_sync(0xffffffffu, 0.0f, 1);
            __shfl_xor_sync(0xffffffffu, 0.0f, 2);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) emax = max(emax, __shfl_xor_sync(0xffffffffu, emax, o));
    if (lane == 0 && live) atomicMax(&s_E[lrow], emax);
    __syncthreads();
    if (!live) return;
    const int E_row = s_E[lrow];
    if (t_in == 0) out.row_scale[i] = E_row > -1000 ? __uint_as_float((uint32_t) (E_row - 8 + 127) << 23) : 0.0f;   // 2^(E_row - 8): far from the fp32 limits
    uint8_t * prow = out.planes + (size_t) i * FP4_PLANES * (K / 2);
    uint8_t * sft = out.sf + (size_t) tile * (K / 256) * FP4_SF_TILE;
#pragma unroll
    for (int u = 0; u < MAX_QUADS; ++u)
        if (u < qpt) {
            const int qd = t_in + tpr * u;
            plane_quad(lo[u], hi[u], db[u], E_row, qd >> 1, (qd & 1) * 4, K, in_tile, prow, sft);
        }
}

// Development builds (-DB200MOE_FP4_PROF) record, per CTA, the cycles each role spends waiting on each of its barriers.
#ifdef B200MOE_FP4_PROF
#define FP4_PROF_T0() const long long prof_t0_ = clock64()
#define FP4_PROF_ADD(slot) prof_[slot] += clock64() - prof_t0_
#define FP4_PROF_DECL() long long prof_[4] = {0, 0, 0, 0}; const long long prof_beg_ = clock64()
#define FP4_PROF_STORE(base, n) do { if (p.prof) { for (int i_ = 0; i_ < n; ++i_) p.prof[blockIdx.x * 24 + base + i_] = prof_[i_]; p.prof[blockIdx.x * 24 + base + n] = clock64() - prof_beg_; } } while (0)
#else
#define FP4_PROF_T0()
#define FP4_PROF_ADD(slot)
#define FP4_PROF_DECL()
#define FP4_PROF_STORE(base, n)
#endif

struct Fp4Params {
    const float * scale0;   // per-expert fp32 scale of tile 0's tensor (or null)
    const float * scale1;
    const uint8_t * sf;     // activation scale tiles
    const float * row_scale;
    const int * offsets;    // [n_as + 1]
    const int * perm;       // [rows]
    const int * active;     // [n_as]
    const int * meta;
    const int * tile_of_expert;   // [n_as + 1]: first token tile of every expert, total number of tiles at the end
    const int * tile_expert;      // [tiles]
    float * out;            // [rows][n_out] indexed by routed row
    int n_out;
    int n_as;
    int * err;
    long long * prof;       // development builds only
};

template <int K>
struct Fp4Cfg {
    static constexpr int A_TILE = 128 * 128;                         // 128 weight rows x 256 K as fp4
    static constexpr int B_BYTES = FP4_NROW * 128;                   // 98 plane rows arrive per stage
    static constexpr int B_TILE = 13 * 1024;                         // their room (rows 98..103 of an N = 104 instruction read what lies there: columns nobody uses)
    static constexpr int STAGE = 2 * A_TILE + 2 * FP4_SF_TILE;      // repacked weights of both tiles, then their scale tiles
    static constexpr int ACT_STAGE = B_TILE + FP4_SF_TILE;           // digit planes, then their scale tile
    static constexpr int RAW_STAGE = 256 * GEMM_RAW_ROW;
    static constexpr int RS = 3;
    static constexpr int TS = 2;
    static constexpr int AS = 3;                                      // plane tiles come from L2 with ~1 us latency: fetched three stages ahead
    static constexpr uint32_t TMEM_COLS = 512;                        // 2 buffers x 2 accumulators x 104 columns, then two sets of scale factors
    static constexpr uint32_t SF_COL = 4 * FP4_NCOL;                  // 416; 48 columns per set
    static_assert(TS == 2 && B_TILE >= B_BYTES + 6 * 128, "one scale-factor set per operand stage");
    static_assert(STAGE % 1024 == 0 && ACT_STAGE % 1024 == 0, "stages keep the 1024-byte alignment of swizzled tiles");
    static_assert(K % GEMM_RAW_K == 0, "K must be a multiple of 256");
    static constexpr size_t SMEM = (size_t) TS * STAGE + (size_t) AS * ACT_STAGE + (size_t) RS * RAW_STAGE + 1024;
};

// DUAL: tile 0 = gate rows f .. f+127, tile 1 = up rows of the same features; epilogue = SwiGLU; 128 features per item.
// single: tiles 0 and 1 = 256 consecutive rows of the one tensor; 256 features per item.
template <int K, bool DUAL>
__global__ void __launch_bounds__(FP4_THREADS, 1)
expert_gemm_fp4_kernel(const Fp4Params p, const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                       const __grid_constant__ CUtensorMap map_planes) {
    using C = Fp4Cfg<K>;
    constexpr int TS = C::TS, RS = C::RS, AS = C::AS;
    constexpr int KC = K / GEMM_RAW_K;
    constexpr int FEAT = DUAL ? 128 : 256;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t * tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint8_t * acts = tiles + (size_t) TS * C::STAGE;
    uint8_t * raws = acts + (size_t) AS * C::ACT_STAGE;
    __shared__ uint64_t raw_full[RS], raw_empty[RS], tile_full[TS], tile_empty[TS], act_full[AS], act_empty[AS], acc_full[2], acc_empty[2], sf_full[TS];
    __shared__ uint32_t s_tmem;
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < RS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 8); }
        for (int i = 0; i < TS; ++i) { mbar_init(&tile_full[i], 256); mbar_init(&tile_empty[i], 1); mbar_init(&sf_full[i], 1); }
        for (int i = 0; i < AS; ++i) { mbar_init(&act_full[i], 1); mbar_init(&act_empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        mbar_fence_init();
        s_abort = 0;
    }
    if (warp == 3) {
        tmem_alloc(&s_tmem, C::TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 32) {   // the first use of a tensor map otherwise pays for its fetch
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w0) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_planes) : "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;

    // Work unit = (token tile of an expert, feature tile): every role walks the same units, blockIdx.x, blockIdx.x + gridDim.x, ...
    // Feature tiles of one token tile are neighbours in that order, so they find the tile's planes in L2; token tiles of one
    // expert follow each other, so a second pass over an expert's weights comes from L2 as well.
    const int f_tiles = p.n_out / FEAT;
    const int n_units = p.tile_of_expert[p.n_as] * f_tiles;
    struct Unit { int e, ft, row0, nt, tile; };
    auto unit_at = [&](int u) {
        Unit w;
        w.tile = u / f_tiles;
        w.ft = u - w.tile * f_tiles;
        w.e = p.tile_expert[w.tile];
        const int row_beg = p.offsets[w.e], t0 = (w.tile - p.tile_of_expert[w.e]) * FP4_RPT;
        w.row0 = row_beg + t0;                                   // first expert-sorted row of the token tile
        w.nt = min(FP4_RPT, p.offsets[w.e + 1] - w.row0);
        return w;
    };
    // weight stage: [A0][A1][SFA0][SFA1]; activation stage: [B][SFB]
    constexpr uint32_t OFF_A1 = C::A_TILE, OFF_SFA = 2 * C::A_TILE, OFF_SFB = C::B_TILE;

    if (warp == 0) {
        // ---------------------------------------------------------------- raw weight producer
        if (lane == 0) {
            Ring raw;
            FP4_PROF_DECL();
            for (int u = blockIdx.x; u < n_units && !s_abort; u += gridDim.x) {
                const Unit w = unit_at(u);
                const int row0 = w.e * p.n_out + w.ft * FEAT;
                for (int kc = 0; kc < KC; ++kc) {
                    FP4_PROF_T0();
                    if (!wait_or_abort<200>(&raw_empty[raw.stage], raw.phase ^ 1u, &s_abort, p.err)) break;
                    FP4_PROF_ADD(0);
                    uint8_t * dst = raws + (size_t) raw.stage * C::RAW_STAGE;
                    mbar_arrive_expect_tx(&raw_full[raw.stage], C::RAW_STAGE);
                    tma_load_2d(dst, &map_w0, kc * GEMM_RAW_ROW, row0, &raw_full[raw.stage]);
                    if (DUAL) tma_load_2d(dst + 128 * GEMM_RAW_ROW, &map_w1, kc * GEMM_RAW_ROW, row0, &raw_full[raw.stage]);
                    else tma_load_2d(dst + 128 * GEMM_RAW_ROW, &map_w0, kc * GEMM_RAW_ROW, row0 + 128, &raw_full[raw.stage]);
                    raw.template advance<RS>();
                }
            }
            FP4_PROF_STORE(0, 1);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- activation producer
        if (lane == 0) {
            Ring act;
            FP4_PROF_DECL();
            for (int u = blockIdx.x; u < n_units && !s_abort; u += gridDim.x) {
                const Unit w = unit_at(u);
                const uint8_t * sft = p.sf + (size_t) w.tile * KC * FP4_SF_TILE;
                for (int kc = 0; kc < KC; ++kc) {
                    FP4_PROF_T0();
                    if (!wait_or_abort<100>(&act_empty[act.stage], act.phase ^ 1u, &s_abort, p.err)) break;
                    FP4_PROF_ADD(0);
                    uint8_t * st = acts + (size_t) act.stage * C::ACT_STAGE;
                    mbar_arrive_expect_tx(&act_full[act.stage], C::B_BYTES + FP4_SF_TILE);
                    tma_load_2d(st, &map_planes, kc * 128, FP4_PLANES * w.row0, &act_full[act.stage]);
                    bulk_g2s(st + OFF_SFB, sft + (size_t) kc * FP4_SF_TILE, FP4_SF_TILE, &act_full[act.stage]);
                    act.template advance<AS>();
                }
            }
            FP4_PROF_STORE(2, 1);
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            Ring tile, act, acc;
            FP4_PROF_DECL();
            for (int u = blockIdx.x; u < n_units && !s_abort; u += gridDim.x) {
                {
                    const int nt = unit_at(u).nt;
                    const uint32_t idesc = umma_idesc_fp4((FP4_PLANES * nt + 7) & ~7);
                    {
                        FP4_PROF_T0();
                        if (!wait_or_abort<40>(&acc_empty[acc.stage], acc.phase ^ 1u, &s_abort, p.err)) break;
                        FP4_PROF_ADD(0);
                    }
                    tc_fence_after();
                    const uint32_t d0 = tmem + (uint32_t) acc.stage * (2 * FP4_NCOL), d1 = d0 + FP4_NCOL;
                    for (int kc = 0; kc < KC; ++kc) {
                        {
                            FP4_PROF_T0();
                            if (!wait_or_abort<20>(&act_full[act.stage], act.phase, &s_abort, p.err)) break;
                            FP4_PROF_ADD(1);
                        }
                        {
                            FP4_PROF_T0();
                            if (!wait_or_abort<20>(&tile_full[tile.stage], tile.phase, &s_abort, p.err)) break;
                            FP4_PROF_ADD(2);
                        }
                        tc_fence_after();
                        const uint32_t sbase = smem_u32(tiles + (size_t) tile.stage * C::STAGE);
                        const uint32_t abase = smem_u32(acts + (size_t) act.stage * C::ACT_STAGE);
                        const uint32_t da = DESC_LO | (sbase >> 4), db = DESC_LO | (abase >> 4);
                        // The scale factors of this stage were copied into their set of tensor-memory columns by the scale-copy thread
                        // (warp 3); its commit on sf_full says the copies are complete.
                        {
                            FP4_PROF_T0();
                            if (!wait_or_abort<20>(&sf_full[tile.stage], tile.phase, &s_abort, p.err)) break;
                            FP4_PROF_ADD(2);
                        }
                        tc_fence_after();
                        const uint32_t sf_set = tmem + C::SF_COL + 48 * (uint32_t) tile.stage;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {   // 4 x K64 = 256; 32 bytes (2 units) further along the 128-byte row each
                            const uint32_t t_sfa0 = sf_set + 12 * kk, t_sfa1 = t_sfa0 + 4, t_sfb = t_sfa0 + 8;
                            const bool accum = kc != 0 || kk != 0;
                            umma_fp4(d0, da + 2 * kk, db + 2 * kk, DESC_HI, idesc, t_sfa0, t_sfb, accum);
                            umma_fp4(d1, da + (OFF_A1 >> 4) + 2 * kk, db + 2 * kk, DESC_HI, idesc, t_sfa1, t_sfb, accum);
                        }
                        umma_commit(&tile_empty[tile.stage]);   // frees both operand stages when these MMAs have read them
                        umma_commit(&act_empty[act.stage]);
                        tile.template advance<TS>();
                        act.template advance<AS>();
                    }
                    umma_commit(&acc_full[acc.stage]);
                    acc.template advance<2>();
                }
            }
            FP4_PROF_STORE(4, 3);
        }
    } else if (warp == 3) {
        // ---------------------------------------------------------------- scale-factor copies (shared memory -> tensor memory)
        // A thread of its own (splitting the copies over two threads was tried: no faster, and one parity case failed): a tcgen05.cp holds its issuing thread for ~80 cycles, and twelve of them per stage in front of the
        // MMAs were more than half of the MMA thread's time.  The set of columns that belongs to an operand stage was last read by
        // the MMAs of the stage two back, and those have completed: their commit released the operand stage, the repack threads
        // waited for that before refilling it, and only then can tile_full be seen here.  (A scale copy is not ordered behind an
        // earlier MMA on another accumulator: with one set of columns a copy was measured to overtake MMAs of the previous stage.)
        if (lane == 0) {
            Ring tile, act;
            FP4_PROF_DECL();
            for (int u = blockIdx.x; u < n_units && !s_abort; u += gridDim.x) {
                bool ok = true;
                for (int kc = 0; kc < KC; ++kc) {
                    {
                        FP4_PROF_T0();
                        if (!wait_or_abort<20>(&act_full[act.stage], act.phase, &s_abort, p.err)) { ok = false; break; }
                        FP4_PROF_ADD(0);
                    }
                    {
                        FP4_PROF_T0();
                        if (!wait_or_abort<20>(&tile_full[tile.stage], tile.phase, &s_abort, p.err)) { ok = false; break; }
                        FP4_PROF_ADD(1);
                    }
                    tc_fence_after();
                    const uint32_t sbase = smem_u32(tiles + (size_t) tile.stage * C::STAGE);
                    const uint32_t abase = smem_u32(acts + (size_t) act.stage * C::ACT_STAGE);
                    const uint32_t sf_set = tmem + C::SF_COL + 48 * (uint32_t) tile.stage;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint32_t t_sfa0 = sf_set + 12 * kk;
                        tmem_cp_sf(t_sfa0, sbase + OFF_SFA + kk * 512);
                        tmem_cp_sf(t_sfa0 + 4, sbase + OFF_SFA + FP4_SF_TILE + kk * 512);
                        tmem_cp_sf(t_sfa0 + 8, abase + OFF_SFB + kk * 512);
                    }
                    umma_commit(&sf_full[tile.stage]);
                    tile.template advance<TS>();
                    act.template advance<AS>();
                }
                if (!ok) break;
            }
            FP4_PROF_STORE(13, 2);
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------------------------------------------------------- epilogue
        Ring acc;
        FP4_PROF_DECL();
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        for (int u = blockIdx.x; u < n_units && !s_abort; u += gridDim.x) {
            const Unit w = unit_at(u);
            const float sc0 = p.scale0 ? p.scale0[w.e] : 1.0f;
            const float sc1 = DUAL ? (p.scale1 ? p.scale1[w.e] : 1.0f) : sc0;
            const int feature = w.ft * FEAT + q * 32 + lane;
            {
                const int nt = w.nt;
                // lanes leave the polling loop one by one: the vote reconverges the warp (tcgen05.ld below needs all of it)
                {
                    FP4_PROF_T0();
                    if (!__all_sync(0xffffffffu, wait_or_abort<200>(&acc_full[acc.stage], acc.phase, &s_abort, p.err))) break;
                    FP4_PROF_ADD(0);
                }
                tc_fence_after();
                const uint32_t d0 = tmem + (uint32_t) acc.stage * (2 * FP4_NCOL) + ((uint32_t) (q * 32) << 16);
                for (int g = 0; g < nt; g += 4) {          // four routed rows = 28 plane columns per load (the last load of a full tile reads past its 98)
                    float v0[32], v1[32];
                    tmem_ld32(d0 + FP4_PLANES * g, v0);
                    tmem_ld32(d0 + FP4_NCOL + FP4_PLANES * g, v1);
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) {
                        if (g + rr < nt) {
                            const int i = w.row0 + g + rr;
                            const float rs = p.row_scale[i];
                            // sum_p 8^p * plane_p, highest plane first
                            float x0 = v0[7 * rr + 6], x1 = v1[7 * rr + 6];
#pragma unroll
                            for (int pl = 5; pl >= 0; --pl) {
                                x0 = __fmaf_rn(x0, 8.0f, v0[7 * rr + pl]);
                                x1 = __fmaf_rn(x1, 8.0f, v1[7 * rr + pl]);
                            }
                            x0 = __fmul_rn(__fmul_rn(x0, rs), sc0);
                            x1 = __fmul_rn(__fmul_rn(x1, rs), sc1);
                            float * orow = p.out + (size_t) p.perm[i] * p.n_out;
                            if (DUAL) orow[feature] = __fmul_rn(ggml_silu(x0), x1);
                            else { orow[feature] = x0; orow[feature + 128] = x1; }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc.stage]);
                acc.template advance<2>();
            }
        }
        if (warp == 4 && lane == 0) FP4_PROF_STORE(8, 1);
    } else if (warp >= 8) {
        // ---------------------------------------------------------------- repack: strip the scale bytes, keep everything else
        const int dq = tid - 256;
        const int trow = dq & 127, tsel = dq >> 7;
        uint32_t a_off[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) a_off[c] = tsel * C::A_TILE + sw128_offset(trow, c);
        const uint32_t sf_off = OFF_SFA + tsel * FP4_SF_TILE + sf_tile_offset(trow);
        const uint32_t raw_off = (uint32_t) dq * GEMM_RAW_ROW;
        Ring raw, tile;
        FP4_PROF_DECL();
        for (int u = blockIdx.x; u < n_units && !s_abort; u += gridDim.x) {
            {
                for (int kc = 0; kc < KC && !s_abort; ++kc) {
                    {
                        FP4_PROF_T0();
                        if (!__all_sync(0xffffffffu, wait_or_abort(&raw_full[raw.stage], raw.phase, &s_abort, p.err))) break;
                        FP4_PROF_ADD(0);
                    }
                    uint32_t R[36];                // 4 blocks of [scale word][8 code words]
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
                    {
                        FP4_PROF_T0();
                        if (!__all_sync(0xffffffffu, wait_or_abort(&tile_empty[tile.stage], tile.phase ^ 1u, &s_abort, p.err))) break;
                        FP4_PROF_ADD(1);
                    }
                    uint8_t * st = tiles + (size_t) tile.stage * C::STAGE;
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        *reinterpret_cast<uint4 *>(st + a_off[2 * kb]) = make_uint4(R[9 * kb + 1], R[9 * kb + 2], R[9 * kb + 3], R[9 * kb + 4]);
                        *reinterpret_cast<uint4 *>(st + a_off[2 * kb + 1]) = make_uint4(R[9 * kb + 5], R[9 * kb + 6], R[9 * kb + 7], R[9 * kb + 8]);
                        // The reference reads scale bytes through ggml_ue4m3_to_fp32: bit 7 ignored, 0x7f decodes to zero; to the tensor
                        // core 0x7f is NaN.  Clear bit 7 and turn 0x7f into 0 (t <= 0x7f per byte, so t + 1 carries into bit 7 only
                        // for 0x7f and never into the next byte).
                        const uint32_t t = R[9 * kb] & 0x7f7f7f7fu;
                        const uint32_t nan1 = ((t + 0x01010101u) >> 7) & 0x01010101u;
                        *reinterpret_cast<uint32_t *>(st + sf_off + kb * 512) = t & ~((nan1 << 7) - nan1);
                    }
                    // every writer orders its own stores against the tensor core's (async proxy) reads and then arrives itself
                    fence_async_smem();
                    mbar_arrive(&tile_full[tile.stage]);
                    tile.template advance<TS>();
                }
            }
        }
        if (tid == 256) FP4_PROF_STORE(10, 2);
    }

    // ---- teardown: everyone meets here (all waits above are bounded), then tensor memory goes back
    if (s_abort) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 3) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace b200moe
