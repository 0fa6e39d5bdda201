"""The ggml backend adapter (libggml-b200.so) driven by the reference's own graph.

oracle/_ref's driver builds the route + ffn graph of edge0-infer (forward.cpp:262-271, 300-311) with the reference's
ggml and computes it once on the reference's CPU backend and once on the B200 backend; with the integer expert
kernels every observed tensor has to come back identical, with every tensor in its own memory and under ggml's
graph allocator (memory reused between tensors)."""
import ctypes as C
import os

import numpy as np
import pytest

from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_NVFP4, TYPE_Q3_K
from oracle import oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ADAPTER = os.path.join(ROOT, "edge0_b200", "lib", "libggml-b200.so")


class Stats(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_route", "n_ffn", "n_dense", "n_single", "n_nodes", "n_deferred")]


@pytest.fixture(scope="module")
def host():
    if not O.have_reference() or not os.path.exists(ADAPTER):
        pytest.skip("needs the compiled reference ggml and libggml-b200.so (built where the reference tree is present)")
    ref = O.reference()
    lib = C.CDLL(ADAPTER, mode=C.RTLD_GLOBAL)
    lib.ggml_backend_b200_init.restype = C.c_void_p
    lib.ggml_backend_b200_init.argtypes = [C.c_int]
    lib.ggml_backend_b200_set_expert_path.argtypes = [C.c_void_p, C.c_int]
    lib.ggml_backend_b200_graph_stats.argtypes = [C.c_void_p, C.POINTER(Stats)]
    lib.ggml_backend_b200_last_error.restype = C.c_char_p
    lib.ggml_backend_b200_last_error.argtypes = [C.c_void_p]
    be = lib.ggml_backend_b200_init(0)
    assert be, "ggml_backend_b200_init(0) returned NULL"
    yield ref, lib, C.c_void_p(be)
    ref.lib.ref_backend_free(C.c_void_p(be))


def compare(host, cfg, T, use_gallocr, path=1, expect=None):
    ref, lib, be = host
    assert lib.ggml_backend_b200_set_expert_path(be, path) == 0
    layer = W.make_layer(cfg)
    x = W.make_tokens(cfg, T)
    want = ref.moe_layer(x=x, **layer.checker_kwargs())
    got = ref.moe_layer(x=x, backend=be, use_gallocr=use_gallocr, **layer.checker_kwargs())
    st = Stats()
    assert lib.ggml_backend_b200_graph_stats(be, C.byref(st)) == 0
    print(f"nodes {st.n_nodes} route {st.n_route} ffn {st.n_ffn} dense {st.n_dense} single {st.n_single} deferred {st.n_deferred}")
    if expect is not None:
        assert (st.n_route, st.n_ffn, st.n_dense) == expect, (st.n_route, st.n_ffn, st.n_dense, st.n_single)
    assert np.array_equal(got.ids, want.ids)
    for name in ("logits", "probs", "weights", "hidden", "down_out", "moe_out", "out"):
        a, b = getattr(got, name), getattr(want, name)
        if path == 1:
            assert np.array_equal(a, b), f"{name} differs: max abs {np.max(np.abs(a - b))}"
        else:
            rms = float(np.sqrt(np.mean(b.astype(np.float64) ** 2)))
            assert float(np.max(np.abs(a - b))) <= 1e-2 * rms, name


@pytest.mark.parametrize("use_gallocr", [False, True])
@pytest.mark.parametrize("wtype", [TYPE_NVFP4, TYPE_Q3_K])
@pytest.mark.parametrize("T", [1, 9])
def test_route_ffn_graph_identical(host, wtype, T, use_gallocr):
    cfg = W.small_config(wtype, n_embd=512, n_expert=16, top_k=4, n_ff=256, seed=21)
    compare(host, cfg, T, use_gallocr, expect=(1, 1, 0))


@pytest.mark.parametrize("use_gallocr", [False, True])
def test_bias_and_unscaled(host, use_gallocr):
    cfg = W.small_config(TYPE_NVFP4, n_embd=512, n_expert=16, top_k=4, n_ff=256, seed=22, router_bias=True, tensor_scales=False)
    compare(host, cfg, 5, use_gallocr, expect=(1, 1, 0))


@pytest.mark.parametrize("use_gallocr", [False, True])
def test_latent_graph_identical(host, use_gallocr):
    cfg = W.small_config(TYPE_NVFP4, n_embd=1024, n_latent=512, n_expert=16, top_k=4, n_ff=256, seed=23)
    compare(host, cfg, 7, use_gallocr, expect=(1, 1, 2))


@pytest.mark.parametrize("use_gallocr", [False, True])
def test_shared_expert_graph(host, use_gallocr):
    """The layer with its shared expert and sigmoid gate (forward.cpp:312-314): the routed part runs as the two fused sub-graphs, the
    shared expert as dense quantised products and per-operator kernels; everything on the backend, results the CPU backend's
    (the sigmoid's expf is the one step that is not the reference's own arithmetic: 1e-6 of RMS on what follows it)."""
    ref, lib, be = host
    assert lib.ggml_backend_b200_set_expert_path(be, 1) == 0
    cfg = W.small_config(TYPE_NVFP4, n_embd=512, n_expert=16, top_k=4, n_ff=256, n_ff_shexp=512, seed=25)
    layer = W.make_layer(cfg)
    x = W.make_tokens(cfg, 6)
    want = ref.moe_layer(x=x, **layer.checker_kwargs())
    got = ref.moe_layer(x=x, backend=be, use_gallocr=use_gallocr, **layer.checker_kwargs())
    st = Stats()
    assert lib.ggml_backend_b200_graph_stats(be, C.byref(st)) == 0
    assert (st.n_route, st.n_ffn, st.n_dense) == (1, 1, 3), (st.n_route, st.n_ffn, st.n_dense, st.n_single)
    for name in ("logits", "probs", "weights", "hidden", "down_out", "moe_out"):
        assert np.array_equal(getattr(got, name), getattr(want, name)), name
    assert np.array_equal(got.ids, want.ids)
    for name in ("shexp_gated", "out"):
        a, b = getattr(got, name), getattr(want, name)
        assert float(np.max(np.abs(a - b))) <= 1e-6 * float(np.sqrt(np.mean(b.astype(np.float64) ** 2))), name


def test_device_failure_is_latched_and_reported_once(host):
    """A graph whose device-side check fails (an expert id outside the table: the kernels record it and skip the row) is reported
    the way the application asks for it: synchronize finds it, the next graph_compute - the empty graph edge0-infer uses to
    confirm completion - returns FAILED once, and the backend works again afterwards."""
    ref, lib, be = host
    lib.ggml_backend_b200_set_expert_path(be, 1)
    cfg = W.small_config(TYPE_NVFP4, n_embd=512, n_expert=16, top_k=4, n_ff=256, seed=26)
    layer = W.make_layer(cfg)
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, (3, 4, 512)).astype(np.float32)
    good = np.array([[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11]], dtype=np.int32)
    bad = good.copy()
    bad[1, 2] = 99                                  # >= n_expert
    assert ref.backend_confirm(be) == 0
    ref.mul_mat_id_backend(be, TYPE_NVFP4, layer.gate, x, bad)      # the check runs on the device: the status comes later
    assert ref.backend_confirm(be) == 4, "the failure must reach the graph that confirms completion"
    assert b"device" in lib.ggml_backend_b200_last_error(be).lower() or lib.ggml_backend_b200_last_error(be)
    assert ref.backend_confirm(be) == 0, "reported once"
    rc, got = ref.mul_mat_id_backend(be, TYPE_NVFP4, layer.gate, x, good)
    assert rc == 0 and ref.backend_confirm(be) == 0
    rc, want = ref.mul_mat_id_backend(None, TYPE_NVFP4, layer.gate, x, good)
    assert rc == 0 and np.array_equal(got, want)


def test_single_expert_per_token(host):
    cfg = W.small_config(TYPE_NVFP4, n_embd=512, n_expert=16, top_k=1, n_ff=256, seed=24)
    compare(host, cfg, 3, False, expect=(1, 1, 0))


def test_config2_default_path(host):
    """BASELINE configs[1] shape through the backend with the default kernel policy: within the stated tolerance."""
    compare(host, W.CONFIGS["c2_nvfp4"], 64, True, path=0, expect=(1, 1, 0))
