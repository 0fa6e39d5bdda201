"""C-ABI library on a machine without a GPU: it loads, exports every declared symbol, validates arguments,
and refuses to compute (there is no CPU fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

from edge0_b200 import capi, moe
from edge0_b200.capi import TYPE_NVFP4, TYPE_Q3_K

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "edge0_b200_moe.h")).read()
    declared = set(re.findall(r"B200MOE_API[^;]*?\b(b200moe_\w+)\s*\(", hdr))
    assert declared and declared == set(capi.SIGNATURES), declared ^ set(capi.SIGNATURES)
    lib = capi.load()
    for name in declared:
        assert getattr(lib, name) is not None


def test_row_sizes_and_status_strings():
    lib = capi.load()
    assert lib.b200moe_row_size(TYPE_Q3_K, 2048) == 880 and lib.b200moe_row_size(TYPE_NVFP4, 2048) == 1152
    assert lib.b200moe_row_size(TYPE_Q3_K, 100) == -1 and lib.b200moe_row_size(TYPE_NVFP4, 96) == -1
    assert lib.b200moe_status_string(0) == b"ok" and b"unsupported" in lib.b200moe_status_string(2)


def test_nvfp4_quantiser_and_dequantisers_match_checker(restatement):
    rng = np.random.default_rng(3)
    w = rng.normal(0, 0.02, (5, 3, 256)).astype(np.float32)
    w[0] *= 5000
    w[1, 0, :16] = 0
    q = moe.quantize_nvfp4(w)
    assert np.array_equal(q, restatement.quantize(TYPE_NVFP4, w))
    assert np.array_equal(moe.dequantize(TYPE_NVFP4, q, 256), restatement.dequantize(TYPE_NVFP4, q, 256))
    z = np.load(os.path.join(ROOT, "tests", "golden", "kat.npz"))
    assert np.array_equal(moe.dequantize(TYPE_Q3_K, z["q3k_wq"], 512), z["q3k_deq"])
    assert np.array_equal(moe.quantize_nvfp4(z["nvfp4_w"]), z["nvfp4_wq"])


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_device_means_no_compute():
    lib = capi.load()
    h = C.c_void_p()
    rc = lib.b200moe_create(0, C.byref(h))
    assert rc == 6 and not h.value          # B200MOE_ERR_NO_DEVICE, and nothing silently falls back
    with pytest.raises(capi.B200MoeError):
        moe.Context(0)
    assert lib.b200moe_reserve(None, None, 1) == 1   # null context is an argument error, not a crash


def test_ggml_adapter_loads_without_gpu():
    """libggml-b200.so (built where the host application's ggml headers are present) loads next to that ggml, exports
    the entry points include/ggml-b200.h declares, and reports no device on a machine without a B200."""
    import ctypes as C
    import os
    from oracle import oracle as O
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    adapter = os.path.join(root, "edge0_b200", "lib", "libggml-b200.so")
    if not os.path.exists(adapter) or not O.have_reference():
        pytest.skip("adapter or compiled reference ggml not built here")
    O.reference()   # ggml symbols, RTLD_GLOBAL
    lib = C.CDLL(adapter)
    for name in ("ggml_backend_b200_reg", "ggml_backend_b200_init", "ggml_backend_is_b200", "ggml_backend_b200_buffer_type",
                 "ggml_backend_b200_set_expert_path", "ggml_backend_b200_graph_stats", "ggml_backend_b200_last_error"):
        assert hasattr(lib, name), name
    import torch
    if not torch.cuda.is_available():
        lib.ggml_backend_b200_init.restype = C.c_void_p
        assert lib.ggml_backend_b200_init(0) is None
