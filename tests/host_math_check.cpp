// CPU check of the bit manipulation the CUDA kernels use (edge0_b200/csrc/formats.cuh compiles for the
// host too): per-unit integer dots of NVFP4 and Q3_K rows against the checker's dot products.
// Built and run by tests/test_host_math.py with g++; exits non-zero on the first mismatch.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "../edge0_b200/csrc/formats.cuh"
#include "../oracle/moe_oracle.h"

using namespace b200moe;

static int fails = 0;
#define CHECK(c, ...) do { if (!(c)) { printf("FAIL %s:%d: ", __FILE__, __LINE__); printf(__VA_ARGS__); printf("\n"); if (++fails > 10) exit(1); } } while (0)

static uint32_t rd32(const uint8_t * p) { uint32_t v; memcpy(&v, p, 4); return v; }

int main() {
    std::mt19937 rng(1234);
    std::normal_distribution<float> nd(0.f, 1.f);

    // UE4M3 decode for every byte
    for (int i = 0; i < 256; ++i) CHECK(ue4m3_half_to_f32(i) == orc_ue4m3_to_fp32((uint8_t) i), "ue4m3 %d", i);

    for (int K : {256, 768, 2048}) {
        for (int trial = 0; trial < 20; ++trial) {
            std::vector<float> w(K), x(K);
            for (auto & v : w) v = nd(rng) * (trial % 3 == 0 ? 30.f : 0.02f);
            for (auto & v : x) v = nd(rng);
            // ---------------- NVFP4 x Q8_0
            {
                std::vector<uint8_t> wq(orc_row_size(ORC_TYPE_NVFP4, K)), aq(K / 32 * 34);
                orc_quantize_row_nvfp4(w.data(), wq.data(), K);
                if (trial == 1) for (auto & b : wq) b = (uint8_t) rng();   // arbitrary bytes, incl. "-0" codes
                orc_quantize_row_q8_0(x.data(), aq.data(), K);
                float ref = orc_vec_dot_nvfp4_q8_0(K, wq.data(), aq.data());
                double acc = 0;
                for (int u = 0; u < K / 32; ++u) {
                    const uint8_t * blk = wq.data() + (u >> 1) * 36;
                    const int hf = u & 1;
                    const uint8_t * ab = aq.data() + u * 34;
                    uint16_t dh; memcpy(&dh, ab, 2);
                    const float dy = orc_fp16_to_fp32(dh);
                    uint32_t a[8], p[8];
                    for (int j = 0; j < 8; ++j) a[j] = rd32(ab + 2 + 4 * j);
                    fp4_permute_act16(a, p);
                    fp4_permute_act16(a + 4, p + 4);
                    for (int s = 0; s < 2; ++s) {
                        const uint32_t w0 = rd32(blk + 4 + 16 * hf + 8 * s), w1 = rd32(blk + 4 + 16 * hf + 8 * s + 4);
                        const int isum = fp4_sub_dot(w0, w1, p + 4 * s);
                        // straight integer reference for this sub-block
                        static const int kv[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
                        int want = 0;
                        for (int j = 0; j < 8; ++j) {
                            const uint8_t qv = blk[4 + (2 * hf + s) * 8 + j];
                            want += kv[qv & 15] * (int) (int8_t) ab[2 + 16 * s + j] + kv[qv >> 4] * (int) (int8_t) ab[2 + 16 * s + j + 8];
                        }
                        CHECK(isum == want, "nvfp4 sub dot K=%d u=%d s=%d got %d want %d", K, u, s, isum, want);
                        acc += (double) (ue4m3_half_to_f32(blk[2 * hf + s]) * dy) * isum;
                    }
                }
                CHECK(std::fabs(acc - ref) <= 1e-5 * (std::fabs(ref) + 1e-3) + 1e-6 * std::fabs(acc), "nvfp4 row K=%d: %g vs %g", K, acc, (double) ref);
            }
            // ---------------- Q3_K x Q8_K  (weights: arbitrary bytes with a sane fp16 scale)
            {
                const int nb = K / 256;
                std::vector<uint8_t> wq(nb * 110), aq(nb * 292);
                for (auto & b : wq) b = (uint8_t) rng();
                for (int b = 0; b < nb; ++b) { uint16_t h = orc_fp32_to_fp16(0.001f * (1 + (rng() % 7))); memcpy(&wq[b * 110 + 108], &h, 2); }
                orc_quantize_row_q8_K(x.data(), aq.data(), K);
                float ref = orc_vec_dot_q3_K_q8_K(K, wq.data(), aq.data());
                double acc = 0;
                for (int sb = 0; sb < nb; ++sb) {
                    const uint8_t * blk = wq.data() + sb * 110;
                    const uint8_t * ab = aq.data() + sb * 292;
                    float dx; memcpy(&dx, ab, 4);
                    const int8_t * q8 = (const int8_t *) ab + 4;
                    const int16_t * bs = (const int16_t *) (ab + 4 + 256);
                    uint32_t sc[4];
                    q3k_unpack_scales(rd32(blk + 96), rd32(blk + 100), rd32(blk + 104), sc);
                    uint16_t dh; memcpy(&dh, blk + 108, 2);
                    long long isum = 0;
                    for (int p = 0; p < 8; ++p) {
                        uint32_t act[8];
                        for (int j = 0; j < 8; ++j) act[j] = rd32((const uint8_t *) q8 + 32 * j + 4 * p);
                        int v = q3k_unit_dot(rd32(blk + 32 + 4 * p), rd32(blk + 64 + 4 * p), rd32(blk + 4 * p), sc, p, act);
                        v -= 4 * (q3k_scale_at(sc, 2 * p) * bs[2 * p] + q3k_scale_at(sc, 2 * p + 1) * bs[2 * p + 1]);
                        isum += v;
                    }
                    // straight reference
                    std::vector<float> deq(256);
                    long long want = 0;
                    for (int idx = 0; idx < 256; ++idx) {
                        const int half = idx >> 7, shift = (idx >> 5) & 3, l = idx & 31;
                        const int lo = (blk[32 + 32 * half + l] >> (2 * shift)) & 3;
                        const int hb = (blk[l] >> (4 * half + shift)) & 1;
                        want += (long long) q3k_scale_at(sc, idx >> 4) * (lo - (hb ? 0 : 4)) * q8[idx];
                    }
                    CHECK(isum == want, "q3k block K=%d sb=%d got %lld want %lld", K, sb, isum, want);
                    acc += (double) (orc_fp16_to_fp32(dh) * dx) * (double) isum;
                }
                CHECK(std::fabs(acc - ref) <= 1e-5 * (std::fabs(ref) + 1e-3) + 1e-6 * std::fabs(acc), "q3k row K=%d: %g vs %g", K, acc, (double) ref);
            }
        }
    }
    // dequantiser of the scales against the checker's dequantised row
    {
        std::vector<uint8_t> blk(110);
        for (auto & b : blk) b = (uint8_t) rng();
        uint16_t h = orc_fp32_to_fp16(0.5f); memcpy(&blk[108], &h, 2);
        std::vector<float> deq(256);
        orc_dequantize_row_q3_K(blk.data(), deq.data(), 256);
        uint32_t sc[4];
        q3k_unpack_scales(rd32(&blk[96]), rd32(&blk[100]), rd32(&blk[104]), sc);
        for (int idx = 0; idx < 256; ++idx) {
            const int half = idx >> 7, shift = (idx >> 5) & 3, l = idx & 31;
            const int lo = (blk[32 + 32 * half + l] >> (2 * shift)) & 3, hb = (blk[l] >> (4 * half + shift)) & 1;
            CHECK(deq[idx] == 0.5f * q3k_scale_at(sc, idx >> 4) * (lo - (hb ? 0 : 4)), "q3k dequant idx %d", idx);
        }
    }
    if (fails) { printf("%d failures\n", fails); return 1; }
    printf("host math ok\n");
    return 0;
}
