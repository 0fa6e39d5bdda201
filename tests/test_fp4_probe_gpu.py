"""The block-scaled FP4 tensor-core instruction against a host model of its operand formats: E2M1 codes, UE4M3 scale per 16
values, ggml's block_nvfp4 conventions (a scale byte 0x7f never reaches the tensor core: the FP4 engine clears it first)."""
import ctypes as C

import numpy as np
import pytest

from edge0_b200 import capi

pytestmark = pytest.mark.gpu

E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], np.float64)


def ue4m3(b):
    b = b.astype(np.int64)
    e, m = (b >> 3) & 15, b & 7
    return np.where(e == 0, m * 2.0 ** -9, (1 + m / 8.0) * 2.0 ** (e - 7.0))


def model(a, b, sfa, sfb):
    av = (E2M1[a].reshape(128, 16, 16) * ue4m3(sfa)[:, :, None]).reshape(128, 256)
    bv = (E2M1[b].reshape(256, 16, 16) * ue4m3(sfb)[:, :, None]).reshape(256, 256)
    return av @ bv.T


@pytest.mark.parametrize("scales", ["unit", "normal", "all_codes"])
def test_fp4_tile_product_matches_host_model(scales, gpu_ctx):
    rng = np.random.default_rng({"unit": 1, "normal": 2, "all_codes": 3}[scales])
    a = rng.integers(0, 16, (128, 256)).astype(np.uint8)
    b = rng.integers(0, 16, (256, 256)).astype(np.uint8)
    if scales == "unit":
        sfa, sfb = np.full((128, 16), 0x38, np.uint8), np.full((256, 16), 0x38, np.uint8)
    elif scales == "normal":
        sfa, sfb = rng.integers(0x20, 0x50, (128, 16)).astype(np.uint8), rng.integers(0x20, 0x50, (256, 16)).astype(np.uint8)
    else:   # zero, subnormal and the largest codes; 0x7f (NaN to the hardware) is excluded
        sfa, sfb = rng.integers(0, 0x7f, (128, 16)).astype(np.uint8), rng.integers(0, 0x7f, (256, 16)).astype(np.uint8)
    d = np.zeros((128, 256), np.float32)
    rc = capi.load().b200moe_probe_fp4_tile(0, a.ctypes.data, b.ctypes.data, sfa.ctypes.data, sfb.ctypes.data, d.ctypes.data)
    assert rc == 0
    want = model(a, b, sfa, sfb)
    scale = np.abs(E2M1[a].reshape(128, 16, 16) * ue4m3(sfa)[:, :, None]).reshape(128, 256) @ \
        np.abs(E2M1[b].reshape(256, 16, 16) * ue4m3(sfb)[:, :, None]).reshape(256, 256).T
    # fp32 accumulation of exact products: error relative to the sum of magnitudes
    assert np.max(np.abs(d - want) / (scale + 1e-30)) <= 2e-6
    if scales == "unit":
        assert np.array_equal(d, want.astype(np.float32))       # small integers and halves: exact


def test_fp4_rate_probe_reports_a_plausible_peak(gpu_ctx):
    lib = capi.load()
    tf = C.c_double(0.0)
    assert lib.b200moe_probe_fp4_rate(0, 256, 1, 2000, C.byref(tf)) == 0
    assert 1000.0 < tf.value < 20000.0
    assert lib.b200moe_probe_fp4_rate(0, 255, 1, 10, C.byref(tf)) != 0      # N must be a multiple of 8
    assert lib.b200moe_probe_fp4_rate(0, 256, 2, 10, C.byref(tf)) != 0      # two accumulators of 256 columns leave no room for scales
