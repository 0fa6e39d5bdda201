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


def test_strata_expert_blobs_unpack_into_the_layer_layout():
    """edge0-strata's experts.bin blobs ([gate | up | down] + {s_gate, s_up, s_down, 0}, docs/NVFP4.md:44-47) unpack into the tensors and
    scale arrays of b200moe_layer byte for byte (host destinations here; the device path is the same copies with cudaMemcpyAsync)."""
    from edge0_b200 import workloads as W
    cfg = W.small_config(TYPE_NVFP4, n_embd=256, n_expert=8, top_k=2, n_ff=128, seed=31)
    layer = W.make_layer(cfg)
    blobs = W.pack_expert_blobs_nvfp4(layer)
    lib = capi.load()
    assert blobs.shape[1] == lib.b200moe_expert_blob_bytes_nvfp4(256, 128) == 2 * 128 * 144 + 256 * 72 + 16
    padded = np.concatenate([blobs, np.full((8, 48), 0xEE, np.uint8)], axis=1)          # a pack may align its blobs
    for b in (blobs, padded):
        g, u, d, sg, su, sd = moe.unpack_expert_blobs_nvfp4(b, 256, 128)
        assert np.array_equal(g, layer.gate) and np.array_equal(u, layer.up) and np.array_equal(d, layer.down)
        assert np.array_equal(sg, layer.gate_scale) and np.array_equal(su, layer.up_scale) and np.array_equal(sd, layer.down_scale)
    assert lib.b200moe_expert_blob_bytes_nvfp4(250, 128) == -1
    with pytest.raises(ValueError):
        moe.unpack_expert_blobs_nvfp4(blobs[:, :-1], 256, 128)


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
