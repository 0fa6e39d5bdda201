"""The plain-C restatement against (a) golden vectors produced by the compiled reference and (b) the compiled
reference itself when its binary is present.  Bit-exact: the restatement emulates the reference's AVX2 lanes."""
import os

import numpy as np
import pytest

from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_NVFP4, TYPE_Q3_K
from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
FIELDS = ("logits", "probs", "ids", "weights", "hidden", "down_out", "moe_out", "out")


def load_case(name):
    from tests.golden.make_golden import CASES
    cfg, T, bf16 = CASES[name]
    z = np.load(os.path.join(GOLD, name + ".npz"))
    if cfg.wtype == TYPE_Q3_K:
        layer = W.make_layer(cfg, quantize_q3k=lambda w: np.zeros(w.shape[:-1] + (w.shape[-1] // 256 * 110,), np.uint8))
        layer.gate, layer.up, layer.down = z["gate"], z["up"], z["down"]
    else:
        layer = W.make_layer(cfg)
        sums = [int(a.astype(np.uint64).sum()) for a in (layer.gate, layer.up, layer.down)]
        assert sums == [int(v) for v in z["weight_sum"]], "seeded NVFP4 weights drifted from the fixture"
    x = W.make_tokens(cfg, T, bf16=bf16)
    assert np.array_equal(x, z["x"])
    return cfg, layer, x, z


@pytest.mark.parametrize("name", ["q3k_small", "nvfp4_small", "nvfp4_small_bias", "nvfp4_small_latent", "nvfp4_small_shexp"])
def test_restatement_matches_golden_bitwise(name, restatement):
    cfg, layer, x, z = load_case(name)
    r = restatement.moe_layer(x=x, **layer.checker_kwargs())
    for f in FIELDS + (("shexp_gated",) if cfg.n_ff_shexp else ()):
        assert np.array_equal(getattr(r, f), z[f]), f"{name}: {f} differs from the reference's golden output"


def test_kat_codecs_and_dots(restatement):
    z = np.load(os.path.join(GOLD, "kat.npz"))
    for wname, wt, K in (("q3k", TYPE_Q3_K, 512), ("nvfp4", TYPE_NVFP4, 512)):
        wq, aq = z[f"{wname}_wq"], z[f"{wname}_aq"]
        assert np.array_equal(restatement.quantize_activation(wt, z[f"{wname}_x"]), aq)
        assert np.array_equal(restatement.dequantize(wt, wq, K), z[f"{wname}_deq"])
        dots = np.array([[restatement.vec_dot(wt, K, wq[i], aq[j]) for j in range(3)] for i in range(8)], dtype=np.float32)
        assert np.array_equal(dots, z[f"{wname}_dots"])
    assert np.array_equal(restatement.quantize(TYPE_NVFP4, z["nvfp4_w"]), z["nvfp4_wq"])


def test_ue4m3_and_fp16_codecs(restatement):
    lib = restatement.lib
    # UE4M3: 0 and 0x7F decode to zero; 0x38 is 1.0 -> 0.5 after the halving; encode/decode round trip on the grid
    assert lib.orc_ue4m3_to_fp32(0) == 0.0 and lib.orc_ue4m3_to_fp32(0x7F) == 0.0
    assert lib.orc_ue4m3_to_fp32(0x38) == 0.5
    for b in range(1, 0x78):
        v = lib.orc_ue4m3_to_fp32(b) * 2.0
        assert lib.orc_fp32_to_ue4m3(v) == b
    # the reference encoder sends every value with exponent 2^8 (256..448) to 0x7E (ggml-impl.h:548-550)
    assert lib.orc_fp32_to_ue4m3(256.0) == 0x7E and lib.orc_fp32_to_ue4m3(300.0) == 0x7E
    assert lib.orc_fp32_to_ue4m3(1e9) == 0x7E and lib.orc_fp32_to_ue4m3(-1.0) == 0
    # fp16 against numpy for every half bit pattern and for a sweep of floats
    allh = np.arange(65536, dtype=np.uint16)
    f = allh.view(np.float16).astype(np.float32)
    for h in list(range(0, 65536, 257)) + [0x7BFF, 0x0001, 0x03FF, 0x0400, 0x8001]:
        got = lib.orc_fp16_to_fp32(h)
        assert (np.isnan(got) and np.isnan(f[h])) or got == f[h]
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.normal(0, 1, 500), rng.normal(0, 1e-5, 200), [65504.0, 65519.9, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8, 0.0]]).astype(np.float32)
    want = xs.astype(np.float16).view(np.uint16)
    for x, w in zip(xs, want):
        assert lib.orc_fp32_to_fp16(float(x)) == int(w), x


def test_top_k_ties_use_lower_index(restatement):
    import ctypes as C
    p = np.array([0.1, 0.3, 0.3, 0.2, 0.3, 0.0, 0.0, 0.1], dtype=np.float32)
    ids = np.zeros(3, dtype=np.int32)
    f = restatement.lib.orc_top_k_row
    f.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    f.restype = C.c_int
    tie = f(8, 3, p.ctypes.data, ids.ctypes.data)
    assert list(ids) == [1, 2, 4] and tie == 1


@pytest.mark.skipif(not O.have_reference(), reason="compiled reference not present")
@pytest.mark.parametrize("wname,latent,bias", [("q3_k", 0, False), ("nvfp4", 0, True), ("nvfp4", 256, False)])
def test_restatement_matches_compiled_reference(wname, latent, bias, restatement):
    ref = O.reference()
    wt = O.TYPE_BY_NAME[wname]
    if latent and wt == TYPE_Q3_K:
        pytest.skip("latent uses NVFP4")
    cfg = W.small_config(wt, n_embd=512, n_latent=latent, n_expert=16, top_k=4, n_ff=256, router_bias=bias, seed=77)
    layer = W.make_layer(cfg, quantize_q3k=lambda w: ref.quantize(TYPE_Q3_K, w))
    x = W.make_tokens(cfg, 7)
    a = ref.moe_layer(x=x, n_threads=3, **layer.checker_kwargs())
    b = restatement.moe_layer(x=x, **layer.checker_kwargs())
    for f in FIELDS:
        assert np.array_equal(getattr(a, f), getattr(b, f)), f


def test_restated_q3k_quantiser_matches_reference_bytes(restatement):
    """The restated weight quantiser (quantize_row_q3_K_ref) against the reference's bytes stored in the fixture and, when the
    compiled reference is present, against it on fresh draws with zero blocks and large values."""
    z = np.load(os.path.join(GOLD, "kat.npz"))
    assert np.array_equal(restatement.quantize(TYPE_Q3_K, z["q3k_w"]), z["q3k_wq"])
    if O.have_reference():
        rng = np.random.default_rng(12)
        w = rng.normal(0, 0.02, (4, 24, 768)).astype(np.float32)
        w[0, 0, :32] = 0
        w[1] *= 3000
        assert np.array_equal(restatement.quantize(TYPE_Q3_K, w), O.reference().quantize(TYPE_Q3_K, w))


def test_synthetic_q3k_blocks_are_valid_and_gaussian_like(restatement):
    """workloads.synth_q3_K draws block_q3_K bytes in the quantised domain (bench inputs): they must decode, with the spread the
    configurations ask for."""
    q = W.synth_q3_K(np.random.default_rng(5), (64, 1024))
    assert q.shape == (64, 440) and q.dtype == np.uint8
    w = restatement.dequantize(TYPE_Q3_K, q, 1024)
    assert np.isfinite(w).all() and 0.012 < float(w.std()) < 0.03 and abs(float(w.mean())) < 2e-3
