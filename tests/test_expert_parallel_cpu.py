"""Bookkeeping of the expert-parallel layer (token split, dispatch order, all-to-all split sizes, inverse permutation,
slot-order combine) exercised with 2 gloo ranks on CPU.  The arithmetic is plugged in from the CPU checker, so the
result must equal the single-process checker's latent layer bit for bit, for any world size."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_NVFP4
from edge0_b200.expert_parallel import ExpertParallelLayer, expert_owner, token_range


class CheckerBackend:
    """Same interface as CudaBackend, arithmetic from the plain-C restatement, tensors on CPU."""

    def __init__(self, layer, rank, world):
        from oracle import oracle as O
        self.o, self.layer, self.cfg = O.restatement(), layer, layer.cfg
        per = self.cfg.n_expert // world
        self.lo = rank * per

    def route(self, x):
        r = self.o.moe_layer(x=x.numpy(), **self.layer.checker_kwargs())
        return torch.from_numpy(r.ids), torch.from_numpy(r.weights)

    def _matvec(self, w, x, k, scale):
        wt = self.cfg.wtype
        out = np.zeros((x.shape[0], w.shape[0]), np.float32)
        for t in range(x.shape[0]):
            aq = self.o.quantize_activation(wt, x[t])
            for r in range(w.shape[0]):
                out[t, r] = self.o.vec_dot(wt, k, w[r], aq)
        if scale is not None:
            out = out * np.float32(scale[0])
        return out

    def project_down(self, x):
        return torch.from_numpy(self._matvec(self.layer.lat_down, x.numpy(), self.cfg.n_embd, self.layer.lat_down_scale))

    def project_up(self, m):
        return torch.from_numpy(self._matvec(self.layer.lat_up, m.numpy(), self.cfg.n_latent, self.layer.lat_up_scale))

    def expert_rows(self, rows, local_eid):
        L, wt, lib = self.layer, self.cfg.wtype, self.o.lib
        out = np.zeros((rows.shape[0], self.cfg.n_in), np.float32)
        for i in range(rows.shape[0]):
            e = int(local_eid[i]) + self.lo
            aq = self.o.quantize_activation(wt, rows[i].numpy())
            h = np.zeros(self.cfg.n_ff, np.float32)
            for r in range(self.cfg.n_ff):
                g = np.float32(self.o.vec_dot(wt, self.cfg.n_in, L.gate[e, r], aq))
                u = np.float32(self.o.vec_dot(wt, self.cfg.n_in, L.up[e, r], aq))
                if L.gate_scale is not None:
                    g, u = g * L.gate_scale[e], u * L.up_scale[e]
                h[r] = np.float32(lib.orc_silu(float(g))) * np.float32(u)
            hq = self.o.quantize_activation(wt, h)
            for r in range(self.cfg.n_in):
                d = np.float32(self.o.vec_dot(wt, self.cfg.n_ff, L.down[e, r], hq))
                out[i, r] = d * L.down_scale[e] if L.down_scale is not None else d
        return torch.from_numpy(out)

    def gather_rows(self, src, idx):
        return src[idx.long()].contiguous()

    def combine(self, y, w):
        acc = y[:, 0, :] * w[:, 0:1]
        for s in range(1, y.shape[1]):
            acc = acc + y[:, s, :] * w[:, s:s + 1]
        return acc


def make_case():
    cfg = W.small_config(TYPE_NVFP4, n_embd=256, n_latent=256, n_expert=8, top_k=2, n_ff=256, seed=61)
    return cfg, W.make_layer(cfg), W.make_tokens(cfg, 5)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, layer, x = make_case()
    lo, hi = token_range(x.shape[0], world, rank)
    ep = ExpertParallelLayer(CheckerBackend(layer, rank, world), cfg.n_expert, cfg.top_k, rank, world)
    out, ids, w = ep.forward(torch.from_numpy(x[lo:hi]), return_routing=True)
    ret[rank] = (lo, hi, out.numpy(), ids.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_partition_helpers():
    assert [token_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [token_range(2, 4, r) for r in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]      # ranks with no tokens
    assert [int(expert_owner(512, 8, e)) for e in (0, 63, 64, 511)] == [0, 0, 1, 7]


@pytest.mark.parametrize("world", [1, 2])
def test_expert_parallel_equals_single_process(world, restatement):
    cfg, layer, x = make_case()
    want = restatement.moe_layer(x=x, **layer.checker_kwargs())
    if world == 1:
        ep = ExpertParallelLayer(CheckerBackend(layer, 0, 1), cfg.n_expert, cfg.top_k)
        out = ep.forward(torch.from_numpy(x))
        assert np.array_equal(out.numpy(), want.out)
        return
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    got = np.zeros_like(want.out)
    for rank in range(world):
        lo, hi, out, ids = ret[rank]
        got[lo:hi] = out
        assert np.array_equal(ids, want.ids[lo:hi])
    assert np.array_equal(got, want.out), "expert-parallel result must not depend on the number of ranks"
