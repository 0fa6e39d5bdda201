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
from edge0_b200.expert_parallel import CudaBackend, ExpertParallelLayer, token_range

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
    ep = ExpertParallelLayer(CudaBackend(ctx, layer, rank, world), cfg.n_expert, cfg.top_k, rank, world)
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
