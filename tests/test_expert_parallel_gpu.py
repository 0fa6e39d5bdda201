"""Expert-parallel latent layer on GPUs: the C-ABI arithmetic under the dispatch/combine bookkeeping.
World size 1 runs in-process; world size 2 spawns two ranks over NCCL when two GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

from edge0_b200 import moe
from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_NVFP4
from edge0_b200.expert_parallel import CudaBackend, ExpertParallelLayer, combine_slots, pack_slots, slot_capacity, token_range

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rel_err(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - want)) / (np.sqrt(np.mean(want ** 2)) + 1e-30))


def case(T=24):
    cfg = W.small_config(TYPE_NVFP4, n_embd=512, n_latent=256, n_expert=16, top_k=4, n_ff=256, seed=71)
    return cfg, W.make_layer(cfg), W.make_tokens(cfg, T)


def test_dense_ops_match_checker(gpu_ctx, checker):
    rng = np.random.default_rng(4)
    w = rng.normal(0, 0.02, (64, 512)).astype(np.float32)
    wq = moe.quantize_nvfp4(w)
    x = rng.normal(0, 1, (9, 512)).astype(np.float32)
    s = np.array([0.37], np.float32)
    y = gpu_ctx.mul_mat(TYPE_NVFP4, torch.from_numpy(wq).cuda(), torch.from_numpy(x).cuda(), 512, torch.from_numpy(s).cuda())
    gpu_ctx.synchronize()
    want = np.zeros((9, 64), np.float32)
    for t in range(9):
        aq = checker.quantize_activation(TYPE_NVFP4, x[t])
        for r in range(64):
            want[t, r] = np.float32(checker.vec_dot(TYPE_NVFP4, 512, wq[r], aq)) * s[0]
    assert np.array_equal(y.cpu().numpy(), want)           # reference summation order: bit-identical
    src = torch.from_numpy(rng.normal(0, 1, (7, 64)).astype(np.float32)).cuda()
    idx = torch.tensor([6, 0, 0, 3], dtype=torch.int32, device="cuda")
    assert torch.equal(gpu_ctx.gather_rows(src, idx), src[idx.long()])
    yk = torch.from_numpy(rng.normal(0, 1, (5, 3, 64)).astype(np.float32)).cuda()
    wk = torch.from_numpy(rng.uniform(0, 1, (5, 3)).astype(np.float32)).cuda()
    acc = yk[:, 0] * wk[:, 0:1]
    for sl in range(1, 3):
        acc = acc + yk[:, sl] * wk[:, sl:sl + 1]
    assert torch.equal(gpu_ctx.combine(yk, wk), acc)           # same fp32 operations in the same order
    gpu_ctx.synchronize()


def test_exchange_kernels_match_their_host_statement(gpu_ctx):
    """b200moe_ep_pack / b200moe_ep_combine against pack_slots / combine_slots (any placement order inside a destination is valid:
    compare through slot_of), and the owner's entry point against b200moe_ffn with one slot of weight 1 per row."""
    rng = np.random.default_rng(12)
    cfg = W.small_config(TYPE_NVFP4, n_embd=256, n_expert=8, top_k=2, n_ff=256, seed=72)
    layer = W.make_layer(cfg)
    T, k, w, world, per = 11, 3, 256, 4, 2
    rows = rng.normal(0, 1, (T, w)).astype(np.float32)
    ids = rng.integers(0, 8, (T, k)).astype(np.int32)
    cap = slot_capacity(T * world, world, k)
    slots, slot_of = gpu_ctx.ep_pack(torch.from_numpy(rows).cuda(), torch.from_numpy(ids).cuda(), world, per, cap)
    gpu_ctx.synchronize()
    sl = slots.cpu().numpy().view(np.float32).reshape(world, cap, w + 4)
    so = slot_of.cpu().numpy()
    eid = sl.view(np.int32)[:, :, w]
    assert (eid >= 0).sum() == T * k and len(set(so.reshape(-1).tolist())) == T * k
    for t in range(T):
        for s_ in range(k):
            d, p_ = divmod(int(so[t, s_]), cap)
            assert d == ids[t, s_] // per and eid[d, p_] == ids[t, s_] % per and np.array_equal(sl[d, p_, :w], rows[t])
    # owner: slots of "rank 0" hold local ids 0..1 of an 8-expert layer cut to its first two experts
    local = moe.MoeLayer(gpu_ctx, wtype=cfg.wtype, top_k=1, router_w=np.zeros((per, w), np.float32), gate=layer.gate[:per], up=layer.up[:per],
                         down=layer.down[:per], gate_scale=layer.gate_scale[:per], up_scale=layer.up_scale[:per], down_scale=layer.down_scale[:per])
    mine = slots[0].contiguous()
    for path in (1, 8):
        gpu_ctx.set_expert_path(path)
        try:
            y = local.ep_expert_rows(mine)
            valid = np.nonzero(eid[0] >= 0)[0]
            xs = torch.from_numpy(np.ascontiguousarray(sl[0, valid, :w])).cuda()
            want = local.ffn(xs, torch.from_numpy(np.ascontiguousarray(eid[0, valid]).reshape(-1, 1)).cuda(), torch.ones((len(valid), 1), device="cuda"))
            gpu_ctx.synchronize()
        finally:
            gpu_ctx.set_expert_path(0)
        assert torch.equal(y[torch.from_numpy(valid).cuda()], want), path
        assert torch.count_nonzero(y[torch.from_numpy(np.nonzero(eid[0] < 0)[0]).cuda()]) == 0      # empty slots stay untouched
    back = torch.from_numpy(rng.normal(0, 1, (world * cap, w)).astype(np.float32)).cuda()
    wts = torch.from_numpy(rng.uniform(0, 1, (T, k)).astype(np.float32)).cuda()
    got = gpu_ctx.ep_combine(back, slot_of, wts)
    gpu_ctx.synchronize()
    assert np.array_equal(got.cpu().numpy(), combine_slots(back.cpu().numpy(), so, wts.cpu().numpy()))


def test_expert_parallel_world1_matches_checker_and_fused_layer(gpu_ctx, checker):
    cfg, layer, x_np = case()
    want = checker.moe_layer(x=x_np, **layer.checker_kwargs())
    ep = ExpertParallelLayer(CudaBackend(gpu_ctx, layer), cfg.n_expert, cfg.top_k)
    out, ids, w = ep.forward(torch.from_numpy(x_np).cuda(), return_routing=True)
    gpu_ctx.synchronize()
    assert np.array_equal(ids.cpu().numpy(), want.ids) and np.array_equal(w.cpu().numpy(), want.weights)
    assert rel_err(out.cpu().numpy(), want.out) <= TOL
    fused = layer.to_device(gpu_ctx).forward(torch.from_numpy(x_np).cuda())
    gpu_ctx.synchronize()
    assert rel_err(fused.cpu().numpy(), want.out) <= TOL


def _rank_main(rank, world, port, T, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = moe.Context(rank)
    cfg, layer, x_np = case(T)
    lo, hi = token_range(T, world, rank)
    ep = ExpertParallelLayer(CudaBackend(ctx, layer, rank, world), cfg.n_expert, cfg.top_k, rank, world, capacity=slot_capacity(T, world, cfg.top_k))
    out, ids, _ = ep.forward(torch.from_numpy(x_np[lo:hi]).cuda(), return_routing=True)
    ctx.synchronize()
    ret[rank] = (lo, hi, out.cpu().numpy(), ids.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()
    ctx.close()


def test_expert_parallel_two_gpus(checker):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    T = 24
    cfg, layer, x_np = case(T)
    want = checker.moe_layer(x=x_np, **layer.checker_kwargs())
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(2, port, T, ret), nprocs=2, join=True)
    got = np.zeros_like(want.out)
    for r in range(2):
        lo, hi, out, ids = ret[r]
        got[lo:hi] = out
        assert np.array_equal(ids, want.ids[lo:hi])
    assert rel_err(got, want.out) <= TOL
