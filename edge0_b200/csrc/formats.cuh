// Decoding of ggml's quantised weight blocks and the per-lane dot-product pieces built on them.
// Everything here is __host__ __device__ so the bit manipulation can be unit-tested on the CPU
// (tests/host_math_check.cpp) against the checker before it ever runs on a GPU.
//
// Work unit: 32 consecutive K positions of one weight row ("unit").
//   NVFP4: unit u = half (u&1) of 64-element block u>>1: two 16-element sub-blocks, each with one UE4M3
//          scale; it pairs with exactly one Q8_0 activation block (32 int8 + one scale).
//   Q3_K : unit u = (super-block sb = u>>3, position group p = u&7): the 4 byte columns l = 4p..4p+3 of
//          the super-block, i.e. elements 128*j + 32*shift + 4p + {0..3} for j in {0,1}, shift in {0..3}.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200moe {

constexpr int TYPE_F32 = 0, TYPE_Q3_K = 11, TYPE_BF16 = 30, TYPE_NVFP4 = 40;
constexpr int NVFP4_BLOCK_BYTES = 36, NVFP4_BLOCK_ELEMS = 64;
constexpr int Q3K_BLOCK_BYTES = 110, Q3K_BLOCK_ELEMS = 256;

B200_HD int64_t weight_row_bytes(int type, int64_t k) {
    return type == TYPE_NVFP4 ? k / NVFP4_BLOCK_ELEMS * NVFP4_BLOCK_BYTES
         : type == TYPE_Q3_K  ? k / Q3K_BLOCK_ELEMS * Q3K_BLOCK_BYTES
         : type == TYPE_F32   ? k * 4
                              : -1;
}

// ---- portable stand-ins for the integer intrinsics -------------------------------------------------
B200_HD uint32_t byte_perm(uint32_t x, uint32_t y, uint32_t s) {
#if defined(__CUDA_ARCH__)
    // PTX prmt directly: the __byte_perm intrinsic drops bit 3 of each selector nibble, and the NVFP4 decode
    // relies on that bit's "replicate the sign of the selected byte" meaning.
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(y), "r"(s));
    return r;
#else
    const uint64_t v = ((uint64_t) y << 32) | x;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        const uint32_t sel = (s >> (4 * i)) & 0xf;
        uint32_t b = (uint32_t) (v >> (8 * (sel & 7))) & 0xff;
        if (sel & 8) b = (b & 0x80) ? 0xff : 0x00;
        r |= b << (8 * i);
    }
    return r;
#endif
}

B200_HD int dot4(int a, int b, int c) {
#if defined(__CUDA_ARCH__)
    return __dp4a(a, b, c);
#else
    for (int i = 0; i < 4; ++i) c += (int) (int8_t) (a >> (8 * i)) * (int) (int8_t) (b >> (8 * i));
    return c;
#endif
}

// UE4M3 byte -> float, already halved (pairs with the doubled E2M1 table), as ggml_ue4m3_to_fp32
// (ggml-impl.h:514-527): 0 and 0x7F decode to 0.
B200_HD float ue4m3_half_to_f32(uint32_t x) {
    x &= 0xff;
    if (x == 0 || x == 0x7f) return 0.0f;
    const uint32_t exp = (x >> 3) & 0xf, man = x & 7;
    union { uint32_t u; float f; } v;
    if (exp == 0) {
        v.f = (float) man * 0.0009765625f;  // man * 2^-9 * 0.5
        return v.f;
    }
    v.u = ((exp + 119u) << 23) | (man << 20);  // 2^(exp-7) * (1+man/8) * 0.5
    return v.f;
}

// ---- NVFP4 --------------------------------------------------------------------------------------------
// Doubled E2M1 magnitudes 0,1,2,3 | 4,6,8,12 as the two PRMT source words.
constexpr uint32_t FP4_MAG_LO = 0x03020100u, FP4_MAG_HI = 0x0c080604u;

// One 32-bit word of qs holds 4 bytes = 8 nibbles; byte b carries element (j0+b) in its low nibble and
// element (j0+b+8) in its high nibble (ggml-quants.c:409-414).  PRMT takes 4 selector nibbles from the
// low 16 bits, so prmt(tab, w) yields elements [j0, j0+8, j0+1, j0+9] and prmt(tab, w>>16) yields
// [j0+2, j0+10, j0+3, j0+11].  A selector nibble with bit 3 set returns the replicated sign bit of the
// table byte, which is 0 for these magnitudes: so prmt(tab, w) gives the magnitudes of the POSITIVE
// codes (0 elsewhere) and prmt(tab, w ^ 0x8888...) those of the NEGATIVE codes.
struct Fp4Word {
    uint32_t pos_a, pos_b, neg_a, neg_b;  // a: from low 16 bits, b: from high 16 bits
};
B200_HD Fp4Word fp4_decode_word(uint32_t w) {
    const uint32_t wn = w ^ 0x88888888u;
    Fp4Word r;
    r.pos_a = byte_perm(FP4_MAG_LO, FP4_MAG_HI, w);
    r.pos_b = byte_perm(FP4_MAG_LO, FP4_MAG_HI, w >> 16);
    r.neg_a = byte_perm(FP4_MAG_LO, FP4_MAG_HI, wn);
    r.neg_b = byte_perm(FP4_MAG_LO, FP4_MAG_HI, wn >> 16);
    return r;
}

// Activation words of one 16-element sub-block (a0..a3 = elements 0-3, 4-7, 8-11, 12-15) rearranged to the
// element order fp4_decode_word produces for the sub-block's two qs words:
//   word0 -> [0,8,1,9] [2,10,3,11]    word1 -> [4,12,5,13] [6,14,7,15]
B200_HD void fp4_permute_act16(const uint32_t a[4], uint32_t p[4]) {
    p[0] = byte_perm(a[0], a[2], 0x5140);
    p[1] = byte_perm(a[0], a[2], 0x7362);
    p[2] = byte_perm(a[1], a[3], 0x5140);
    p[3] = byte_perm(a[1], a[3], 0x7362);
}

// Integer dot of one 16-element sub-block: qs words w0,w1 against permuted activation words p[0..3].
B200_HD int fp4_sub_dot(uint32_t w0, uint32_t w1, const uint32_t p[4]) {
    const Fp4Word d0 = fp4_decode_word(w0), d1 = fp4_decode_word(w1);
    int pos = dot4((int) d0.pos_a, (int) p[0], 0);
    pos = dot4((int) d0.pos_b, (int) p[1], pos);
    pos = dot4((int) d1.pos_a, (int) p[2], pos);
    pos = dot4((int) d1.pos_b, (int) p[3], pos);
    int neg = dot4((int) d0.neg_a, (int) p[0], 0);
    neg = dot4((int) d0.neg_b, (int) p[1], neg);
    neg = dot4((int) d1.neg_a, (int) p[2], neg);
    neg = dot4((int) d1.neg_b, (int) p[3], neg);
    return pos - neg;
}

// ---- Q3_K ---------------------------------------------------------------------------------------------
// The 16 six-bit sub-block scales of a super-block, minus 32, as 4 words of int8
// (unpacking of ggml-quants.c:1322-1327).  s0,s1,s2 = the 12 scale bytes as little-endian words.
B200_HD void q3k_unpack_scales(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t out[4]) {
    const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu;
    uint32_t a0 = (s0 & kmask2) | (((s2 >> 0) & kmask1) << 4);
    uint32_t a1 = (s1 & kmask2) | (((s2 >> 2) & kmask1) << 4);
    uint32_t a2 = ((s0 >> 4) & kmask2) | (((s2 >> 4) & kmask1) << 4);
    uint32_t a3 = ((s1 >> 4) & kmask2) | (((s2 >> 6) & kmask1) << 4);
    // subtract 32 from every byte: values are 0..63, so (v | 0x80) - 32 never borrows, then clear the guard
    out[0] = ((a0 | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
    out[1] = ((a1 | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
    out[2] = ((a2 | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
    out[3] = ((a3 | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
}

B200_HD int q3k_scale_at(const uint32_t sc[4], int i) { return (int) (int8_t) (sc[i >> 2] >> (8 * (i & 3))); }

// Unit (sb, p): integer part of the dot, with codes taken as UNSIGNED q' = code + 4 in [0,7]:
//   sum over (j, shift) of scale[8j + 2*shift + (p>=4)] * dot4(q', act word)
// qs0/qs1: the words at qs[4p] and qs[32+4p]; hm: the word at hmask[4p]; act[8]: activation words for
// elements 128*j + 32*shift + 4p .. +3 in order (j, shift) -> act[4*j + shift].
// The caller subtracts 4 * sum_sub(scale_sub * bsum_sub) once per super-block for the -4 offset.
B200_HD int q3k_unit_dot(uint32_t qs0, uint32_t qs1, uint32_t hm, const uint32_t sc[4], int p, const uint32_t act[8]) {
    int total = 0;
    const int hi = p >= 4 ? 1 : 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int j = 0; j < 2; ++j) {
        const uint32_t w = j ? qs1 : qs0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (int s = 0; s < 4; ++s) {
            const int bit = 4 * j + s;
            const uint32_t lo2 = (w >> (2 * s)) & 0x03030303u;
            const uint32_t hb4 = bit >= 2 ? ((hm >> (bit - 2)) & 0x04040404u) : ((hm << (2 - bit)) & 0x04040404u);
            const int d = dot4((int) (lo2 | hb4), (int) act[4 * j + s], 0);
            total += q3k_scale_at(sc, 8 * j + 2 * s + hi) * d;
        }
    }
    return total;
}

}  // namespace b200moe
