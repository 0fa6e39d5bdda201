"""The expert-parallel layer's exchange (token split, fixed-capacity slots per destination, equal-split all-to-alls, slot-order
combine behind the slot index) exercised with 2 gloo ranks on CPU.  The arithmetic is plugged in from the CPU checker and the
slot format from its host statement in edge0_b200.expert_parallel, so the result must equal the single-process checker's
latent layer bit for bit, for any world size."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from edge0_b200 import workloads as W
from edge0_b200.capi import TYPE_NVFP4
from edge0_b200.expert_parallel import (SLOT_EXTRA_WORDS, ExpertParallelLayer, combine_slots, expert_owner, pack_slots, slot_capacity,
                                        token_range)


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

    def pack(self, xl, ids, world, per, capacity):
        slots, slot_of = pack_slots(xl.numpy(), ids.numpy(), world, per, capacity)
        return torch.from_numpy(slots), torch.from_numpy(slot_of)

    def exchange_buffer(self, t):
        return torch.empty_like(t)

    def expert_rows(self, slots):
        """slots float32 [n_slots, w + 4]: word w is the local expert id (as int), -1 = empty."""
        L, wt, lib = self.layer, self.cfg.wtype, self.o.lib
        w = self.cfg.n_in
        slots = slots.numpy()
        assert slots.shape[1] == w + SLOT_EXTRA_WORDS
        eids = np.ascontiguousarray(slots[:, w]).view(np.int32)
        out = np.zeros((slots.shape[0], w), np.float32)
        for i in range(slots.shape[0]):
            if eids[i] < 0:
                continue
            e = int(eids[i]) + self.lo
            aq = self.o.quantize_activation(wt, np.ascontiguousarray(slots[i, :w]))
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

    def combine(self, back, slot_of, w):
        return torch.from_numpy(combine_slots(back.numpy(), slot_of.numpy(), w.numpy()))


def make_case():
    cfg = W.small_config(TYPE_NVFP4, n_embd=256, n_latent=256, n_expert=8, top_k=2, n_ff=256, seed=61)
    return cfg, W.make_layer(cfg), W.make_tokens(cfg, 5)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, layer, x = make_case()
    lo, hi = token_range(x.shape[0], world, rank)
    ep = ExpertParallelLayer(CheckerBackend(layer, rank, world), cfg.n_expert, cfg.top_k, rank, world,
                             capacity=slot_capacity(x.shape[0], world, cfg.top_k))
    out, ids, w = ep.forward(torch.from_numpy(x[lo:hi]), return_routing=True)
    ret[rank] = (lo, hi, out.numpy(), ids.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_slot_format_round_trip():
    rng = np.random.default_rng(3)
    rows = rng.normal(0, 1, (5, 8)).astype(np.float32)
    ids = np.array([[0, 5], [7, 2], [3, 3], [6, 1], [4, 0]], np.int32)
    cap = slot_capacity(10, 2, 2)
    assert cap == 12 and slot_capacity(1, 8, 1) == 4
    slots, slot_of = pack_slots(rows, ids, 2, 4, cap)
    eid = slots.view(np.int32)[:, :, 8]
    assert (eid >= 0).sum() == 10 and sorted(slot_of.reshape(-1).tolist()) == sorted(set(slot_of.reshape(-1).tolist()))
    for t in range(5):
        for s_ in range(2):
            d, p_ = divmod(int(slot_of[t, s_]), cap)
            assert d == ids[t, s_] // 4 and eid[d, p_] == ids[t, s_] % 4 and np.array_equal(slots[d, p_, :8], rows[t])
    back = slots.reshape(-1, 12)[:, :8].copy()
    w = rng.uniform(0, 1, (5, 2)).astype(np.float32)
    want = rows * w[:, 0:1] + rows * w[:, 1:2]
    assert np.array_equal(combine_slots(back, slot_of, w), want.astype(np.float32))


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


def test_backend_may_fuse_route_and_projection(restatement):
    """A backend that offers route_and_project (the CUDA backend runs the two side by side on two streams) is used through it, with
    the same result."""
    cfg, layer, x = make_case()
    want = restatement.moe_layer(x=x, **layer.checker_kwargs())

    class Fused(CheckerBackend):
        calls = 0

        def route_and_project(self, x):
            Fused.calls += 1
            ids, w = self.route(x)
            return ids, w, self.project_down(x)

    out = ExpertParallelLayer(Fused(layer, 0, 1), cfg.n_expert, cfg.top_k).forward(torch.from_numpy(x))
    assert Fused.calls == 1 and np.array_equal(out.numpy(), want.out)
