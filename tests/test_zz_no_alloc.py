"""b200moe_route_noalloc: routing for callers that may not allocate device memory (a serving loop that must
not hit cudaMalloc, a process whose memory pool owns the whole GPU).  It keeps its intermediate logits in an array
built into the library instead of context scratch, so its answers must be the very same bits as b200moe_route's.
Collected last on purpose: a failure here cannot hide any other test's result."""
import ctypes as C

import numpy as np
import pytest
import torch

from edge0_b200 import capi, moe
from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_BF16, TYPE_NVFP4

pytestmark = pytest.mark.gpu


def call_noalloc(layer: moe.MoeLayer, x: torch.Tensor):
    lib = capi.load()
    T = x.shape[0]
    # outputs are the caller's: allocated here, before the call under test
    ids = torch.empty((T, layer.top_k), dtype=torch.int32, device=x.device)
    w = torch.empty((T, layer.top_k), dtype=torch.float32, device=x.device)
    err = C.create_string_buffer(256)
    xt = TYPE_BF16 if x.dtype == torch.bfloat16 else 0
    rc = lib.b200moe_route_noalloc(layer.ctx.device, C.byref(layer.desc), x.data_ptr(), xt, T, ids.data_ptr(), w.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, err.value.decode(), ids, w


def test_noalloc_route_equals_route_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import oracle as O
    ctx = moe.Context(0)
    cfg = W.CONFIGS["c2_nvfp4"]
    small = W.small_config(TYPE_NVFP4, n_embd=cfg.n_embd, n_expert=cfg.n_expert, top_k=cfg.top_k, n_ff=256, seed=41)
    host = W.make_layer(small)
    layer = host.to_device(ctx)
    for call, T in enumerate((64, 37)):            # two calls in a row share the built-in array
        x_np = W.make_tokens(small, T, bf16=True, seed_offset=call)
        x = torch.from_numpy(x_np).cuda().to(torch.bfloat16)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc, msg, ids, w = call_noalloc(layer, x)
        assert rc == 0, msg
        torch.cuda.synchronize()
        if call > 0:   # the first call on a device may load the module; after that the device's free memory must not move
            assert torch.cuda.mem_get_info()[0] == free_before
        ids_ref, w_ref = layer.route(x)
        ctx.synchronize()
        assert torch.equal(ids, ids_ref), f"call {call}: expert ids differ"
        assert torch.equal(w, w_ref), f"call {call}: route weights differ"
        # and directly against the checker (the reference's CPU path): ids and route weights bit for bit
        want = O.best_checker().moe_layer(x=x_np, **host.checker_kwargs())
        assert np.array_equal(ids.cpu().numpy(), want.ids) and np.array_equal(w.cpu().numpy(), want.weights), f"call {call}"
    # beyond the built-in scratch: refused with a message, nothing launched
    big = torch.zeros((capi.NOALLOC_MAX_LOGITS // small.n_expert + 1, small.n_embd), device="cuda")
    rc, msg, _, _ = call_noalloc(layer, big)
    assert rc == 2 and "exceeds" in msg
    ctx.close()
