"""The GGUF reader of the C ABI (b200moe_gguf_*): files written by the reference's own gguf writer are read back tensor for tensor,
in ggml's block layout, and mapped onto a b200moe_layer by edge0-infer's tensor names.  No GPU needed."""
import ctypes as C
import os

import numpy as np
import pytest

from edge0_b200 import capi, moe
from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_NVFP4, TYPE_Q3_K, B200MoeError
from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ("router_w", "gate", "up", "down", "gate_shexp", "up_shexp", "down_shexp", "gate_inp_shexp")


def test_committed_gguf_fixture_reads_back():
    """tests/golden/moe_block_nvfp4.gguf was written by the compiled reference (tests/golden/make_golden.py gguf)."""
    from tests.golden.make_golden import GGUF_CASE
    cfg, layer_no = GGUF_CASE["config"], GGUF_CASE["layer"]
    want = W.make_layer(cfg)
    g = moe.GgufFile(os.path.join(GOLD, GGUF_CASE["file"]))
    assert g.n_tensors() == 8
    assert g.metadata_u64("qwen3next.expert_count") == cfg.n_expert and g.metadata_u64("qwen3next.block_count") == layer_no + 1
    t = g.moe_layer_tensors(layer_no)                 # top-k from <architecture>.expert_used_count
    assert t["top_k"] == cfg.top_k and t["wtype"] == TYPE_NVFP4 and t["router_bias"] is None
    for name in NAMES:
        assert np.array_equal(t[name], getattr(want, name)), name
    typ, ne, raw = g.tensor(f"blk.{layer_no}.ffn_down_exps.weight")
    assert typ == TYPE_NVFP4 and ne == (cfg.n_ff, cfg.n_embd, cfg.n_expert, 1) and raw.size == want.down.size
    with pytest.raises(B200MoeError):
        g.moe_layer_tensors(layer_no + 1)             # no such block
    with pytest.raises(B200MoeError):
        g.tensor("blk.0.attn_q.weight")
    g.close()


@pytest.mark.parametrize("wtype,shexp", [(TYPE_NVFP4, 256), (TYPE_Q3_K, 0)])
def test_reference_writes_we_read(tmp_path, wtype, shexp):
    if not O.have_reference():
        pytest.skip("needs the compiled reference (its gguf writer)")
    ref = O.reference()
    cfg = W.small_config(wtype, n_embd=256, n_expert=8, top_k=2, n_ff=256, n_ff_shexp=shexp, seed=36, tensor_scales=False)
    layer = W.make_layer(cfg, quantize_q3k=(lambda w: ref.quantize(TYPE_Q3_K, w)) if wtype == TYPE_Q3_K else None)
    path = tmp_path / "block.gguf"
    ref.write_moe_gguf(path, layer=0, wtype=wtype, router_w=layer.router_w, gate=layer.gate, up=layer.up, down=layer.down, top_k=2,
                       sh_gate=layer.gate_shexp, sh_up=layer.up_shexp, sh_down=layer.down_shexp, sh_gate_inp=layer.gate_inp_shexp)
    g = moe.GgufFile(path)
    t = g.moe_layer_tensors(0, top_k=2)
    for name in NAMES:
        a, b = t.get(name), getattr(layer, name)
        assert (a is None and b is None) or np.array_equal(a, b), name


def test_malformed_files_are_refused(tmp_path):
    lib = capi.load()
    h, err = C.c_void_p(), C.create_string_buffer(256)
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUX" + bytes(60))
    assert lib.b200moe_gguf_open(str(bad).encode(), C.byref(h), err, 256) != 0 and b"magic" in err.value and not h.value
    from tests.golden.make_golden import GGUF_CASE
    whole = open(os.path.join(GOLD, GGUF_CASE["file"]), "rb").read()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(whole[: len(whole) // 2])           # tensor data missing
    assert lib.b200moe_gguf_open(str(cut).encode(), C.byref(h), err, 256) != 0 and not h.value
    cut.write_bytes(whole[:100])                        # metadata cut short
    assert lib.b200moe_gguf_open(str(cut).encode(), C.byref(h), err, 256) != 0 and not h.value
    assert lib.b200moe_gguf_open(str(tmp_path / "missing.gguf").encode(), C.byref(h), err, 256) != 0
