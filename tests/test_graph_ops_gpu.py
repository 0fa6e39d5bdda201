"""The per-operator F32 kernels behind the C ABI (b200moe_op_*): what the ggml backend runs for graph nodes outside the fused
route / FFN sub-graphs.  Each is compared with the reference operator's arithmetic: exact numpy statements for the single-rounding
operators, and the CPU checker's router outputs (bit-exact with the reference's CPU backend) for the matmul, soft-max and argsort."""
import ctypes as C

import numpy as np
import pytest
import torch

from edge0_b200 import capi, moe
from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_NVFP4, Tensor

pytestmark = pytest.mark.gpu


def view(t: torch.Tensor, ne=None, nb=None) -> Tensor:
    """ggml's description of a torch tensor: ne[0] is the fastest dimension."""
    shape = list(reversed(t.shape)) + [1] * (4 - t.dim())
    strides = [s * t.element_size() for s in reversed(t.stride())]
    while len(strides) < 4:
        strides.append(strides[-1] * shape[len(strides) - 1])
    v = Tensor()
    v.data = t.data_ptr()
    v.ne[:] = ne or shape
    v.nb[:] = nb or strides
    return v


@pytest.fixture(scope="module")
def ops(gpu_ctx):
    lib = capi.load()
    st = torch.cuda.current_stream().cuda_stream

    def call(name, *args):
        rc = getattr(lib, "b200moe_op_" + name)(gpu_ctx.handle, *args, st)
        assert rc == 0, lib.b200moe_last_error(gpu_ctx.handle).decode()
        torch.cuda.synchronize()
    return call


def test_binary_operators_broadcast_like_ggml(ops):
    rng = np.random.default_rng(1)
    a = rng.normal(0, 1, (3, 5, 64)).astype(np.float32)          # ggml ne = [64, 5, 3]
    for b_shape in ((3, 5, 64), (1, 1, 64), (3, 1, 1), (1, 5, 64)):
        b = rng.normal(0, 1, b_shape).astype(np.float32) + 2.0
        ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
        for op, fn in ((0, np.add), (1, np.multiply), (2, np.divide)):
            td = torch.empty_like(ta)
            ops("binary", op, C.byref(view(ta)), C.byref(view(tb)), C.byref(view(td)))
            assert np.array_equal(td.cpu().numpy(), fn(a, np.broadcast_to(b, a.shape))), (op, b_shape)


def test_binary_on_strided_view(ops):
    """The weighted slots of the FFN sub-graph are views with a row stride: operands are addressed through nb[]."""
    rng = np.random.default_rng(2)
    full = torch.from_numpy(rng.normal(0, 1, (6, 4, 32)).astype(np.float32)).cuda()
    a, b = full[:, 1, :], full[:, 2, :]                              # [6][32] with stride 4*32
    d = torch.empty((6, 32), device="cuda")
    ops("binary", 0, C.byref(view(a)), C.byref(view(b)), C.byref(view(d)))
    assert torch.equal(d, a + b)


def test_clamp_repeat_get_rows_sum_rows(ops, gpu_ctx):
    rng = np.random.default_rng(3)
    a = rng.normal(0, 2, (7, 96)).astype(np.float32)
    ta = torch.from_numpy(a).cuda()
    td = torch.empty_like(ta)
    ops("unary", 2, C.byref(view(ta)), C.byref(view(td)), C.c_float(-1.5), C.c_float(0.75))
    assert np.array_equal(td.cpu().numpy(), np.clip(a, -1.5, 0.75))
    # repeat [1][96] over 7 rows
    row = torch.from_numpy(a[:1].copy()).cuda()
    ops("repeat", C.byref(view(row)), C.byref(view(td)))
    assert np.array_equal(td.cpu().numpy(), np.repeat(a[:1], 7, axis=0))
    # get_rows: a [7][96], ids [5] -> [5][96]
    ids = np.array([6, 0, 3, 3, 1], dtype=np.int32)
    tid = torch.from_numpy(ids).cuda()
    tg = torch.empty((5, 96), device="cuda")
    ops("get_rows", C.byref(view(ta)), C.byref(view(tid)), C.byref(view(tg)))
    assert np.array_equal(tg.cpu().numpy(), a[ids])
    # sum_rows: sequential accumulation in double, rounded once
    ts = torch.empty((7, 1), device="cuda")
    ops("sum_rows", C.byref(view(ta)), C.byref(view(ts)))
    want = np.cumsum(a.astype(np.float64), axis=1)[:, -1].astype(np.float32)
    assert np.array_equal(ts.cpu().numpy()[:, 0], want)


def test_get_rows_reports_bad_index(ops, gpu_ctx):
    a = torch.zeros((4, 32), device="cuda")
    tid = torch.tensor([1, 9], dtype=torch.int32, device="cuda")        # 9 >= 4 rows: recorded and skipped, not read
    d = torch.full((2, 32), 7.0, device="cuda")
    ops("get_rows", C.byref(view(a)), C.byref(view(tid)), C.byref(view(d)))
    with pytest.raises(capi.B200MoeError, match="device check"):
        gpu_ctx.synchronize()
    gpu_ctx.synchronize()                                                 # reported once
    assert torch.equal(d[1], torch.full((32,), 7.0, device="cuda"))


def test_router_chain_operator_by_operator(ops, checker):
    """mul_mat (F32) -> soft_max -> argsort: the router as separate operators gives the fused router's (and the reference's) bits."""
    cfg = W.small_config(TYPE_NVFP4, n_embd=512, n_expert=128, top_k=8, n_ff=256, seed=9)
    layer = W.make_layer(cfg)
    x = W.make_tokens(cfg, 11)
    r = checker.moe_layer(x=x, **layer.checker_kwargs())
    tx, tw = torch.from_numpy(x).cuda(), torch.from_numpy(layer.router_w).cuda()
    logits = torch.empty((11, 128), device="cuda")
    ops("mul_mat_f32", tw.data_ptr(), 512, 128, tx.data_ptr(), 11, logits.data_ptr())
    assert np.array_equal(logits.cpu().numpy(), r.logits)
    probs = torch.empty_like(logits)
    ops("soft_max", C.byref(view(logits)), C.byref(view(probs)), C.c_float(1.0))
    assert np.array_equal(probs.cpu().numpy(), r.probs)
    order = torch.empty((11, 128), dtype=torch.int32, device="cuda")
    ops("argsort_desc", C.byref(view(probs)), C.byref(view(order)))
    got = order.cpu().numpy()
    assert np.array_equal(got[:, :8], r.ids)
    assert np.array_equal(got, np.argsort(-r.probs, axis=1, kind="stable"))


def test_silu_and_sigmoid(ops):
    from oracle import oracle as O
    silu = O.restatement().lib.orc_silu
    rng = np.random.default_rng(4)
    a = rng.normal(0, 3, (5, 64)).astype(np.float32)
    ta = torch.from_numpy(a).cuda()
    td = torch.empty_like(ta)
    ops("unary", 1, C.byref(view(ta)), C.byref(view(td)), C.c_float(0), C.c_float(0))
    one = np.float32(1.0)
    want = one / (one + np.exp(-a.astype(np.float64)).astype(np.float32))
    assert np.array_equal(td.cpu().numpy(), want)
    ops("unary", 0, C.byref(view(ta)), C.byref(view(td)), C.c_float(0), C.c_float(0))
    assert np.array_equal(td.cpu().numpy(), np.array([silu(float(v)) for v in a.ravel()], dtype=np.float32).reshape(a.shape))
