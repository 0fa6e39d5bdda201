"""Expert-parallel latent MoE layer over the GPUs of one box (one process per GPU, torch.distributed for the exchange).

Semantics follow edge0-strata's latent layer with one label group (src/latent/latent_moe.cpp:38-92):
    x [T, H] --D--> xl [T, L] --experts (L -> I -> L), top-k--> combine in slot order --U--> out [T, H]
The reference has no multi-GPU form of it; the partition here is:
  * tokens are split evenly over ranks for routing, D, the combine and U;
  * expert e lives on rank e // (E / N) (contiguous blocks), so expert weights are never moved;
  * one exchange each way (all-to-all): routed latent rows travel to their expert's owner, result rows travel back.
Every routed row is computed by exactly the arithmetic of the single-GPU layer (an ffn call with one slot and weight 1.0),
and the slot-order sum happens on the token's own rank, so results do not depend on N.

`backend` supplies the arithmetic.  CudaBackend calls the C ABI; tests on CPU plug in a backend made of the checker's
functions to exercise this file's bookkeeping over gloo.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist


def expert_owner(n_expert: int, world: int, e):
    return e // (n_expert // world)


def token_range(n_tokens: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, as even as possible; earlier ranks take the remainder."""
    base, rem = divmod(n_tokens, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


@dataclass
class DispatchPlan:
    """Bookkeeping of one exchange, all index tensors on the compute device.
    order        [R]  routed rows (t*k + s) of this rank sorted by destination rank (stable)
    send_counts  [N]  rows going to each rank            (python ints: they size the collective)
    recv_counts  [N]  rows arriving from each rank
    """
    order: torch.Tensor
    send_counts: list
    recv_counts: list


def plan_dispatch(ids: torch.Tensor, n_expert: int, world: int, group=None) -> DispatchPlan:
    """ids int32 [T_local, k].  One small all-to-all of counts; the counts come to the host because they size the
    payload collectives."""
    flat = ids.reshape(-1).to(torch.int64)
    dest = torch.div(flat, n_expert // world, rounding_mode="floor")
    order = torch.sort(dest, stable=True).indices.to(torch.int32)
    send = torch.bincount(dest, minlength=world).to(torch.int64)
    recv = torch.empty_like(send)
    if world > 1:
        dist.all_to_all_single(recv, send, group=group)
    else:
        recv.copy_(send)
    both = torch.stack([send, recv]).cpu()      # one device-to-host read for both count vectors
    return DispatchPlan(order=order, send_counts=[int(v) for v in both[0]], recv_counts=[int(v) for v in both[1]])


def exchange_rows(rows: torch.Tensor, send_counts, recv_counts, world: int, group=None) -> torch.Tensor:
    """rows [sum(send_counts), w], already ordered by destination -> [sum(recv_counts), w] ordered by source."""
    out = torch.empty((sum(recv_counts),) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    if world > 1:
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts), input_split_sizes=list(send_counts), group=group)
    else:
        out.copy_(rows)
    return out


class ExpertParallelLayer:
    """One rank's share of the layer.

    backend.route(x)                    -> ids int32 [T,k], weights float32 [T,k]      (full router, replicated)
    backend.project_down(x) / project_up(m)                                            (shared D / U, replicated)
    backend.expert_rows(xl_rows, local_expert_ids) -> float32 [R, L]                   (this rank's experts only)
    backend.gather_rows(src, idx), backend.combine(y [T,k,L], w [T,k])
    """

    def __init__(self, backend, n_expert: int, top_k: int, rank: int = 0, world: int = 1, group=None):
        if n_expert % world:
            raise ValueError("n_expert must divide evenly over the ranks")
        self.b, self.E, self.k, self.rank, self.world, self.group = backend, n_expert, top_k, rank, world, group

    def forward(self, x_local: torch.Tensor, return_routing: bool = False):
        """x_local: this rank's tokens [T_local, H] -> out [T_local, H]."""
        b, k = self.b, self.k
        T = x_local.shape[0]
        mark = self._mark
        mark("start")
        ids, w = b.route(x_local)                                    # [T,k]
        xl = b.project_down(x_local)                                 # [T,L] float32
        mark("route+D")
        plan = plan_dispatch(ids, self.E, self.world, self.group)
        # pack: routed row r = t*k+s carries token t's latent row and its expert id
        tok = torch.div(plan.order, k, rounding_mode="floor").to(torch.int32)
        send_rows = b.gather_rows(xl, tok)                           # [R, L] ordered by destination
        send_eid = ids.reshape(-1)[plan.order.long()].to(torch.int32).reshape(-1, 1)
        recv_rows = exchange_rows(send_rows, plan.send_counts, plan.recv_counts, self.world, self.group)
        recv_eid = exchange_rows(send_eid, plan.send_counts, plan.recv_counts, self.world, self.group)
        local_eid = (recv_eid.reshape(-1) - self.rank * (self.E // self.world)).to(torch.int32)
        mark("dispatch")
        y_rows = b.expert_rows(recv_rows, local_eid)                 # [R', L]
        mark("experts")
        back = exchange_rows(y_rows, plan.recv_counts, plan.send_counts, self.world, self.group)   # ordered like send_rows
        # unpack: back[i] is routed row plan.order[i]; bring rows into (t, s) order
        inv = torch.empty_like(plan.order)
        inv[plan.order.long()] = torch.arange(plan.order.numel(), dtype=torch.int32, device=plan.order.device)
        y = b.gather_rows(back, inv).reshape(T, k, -1)
        mark("return")
        moe = b.combine(y, w)                                        # slot-order weighted sum on the token's rank
        out = b.project_up(moe)
        mark("combine+U")
        return (out, ids, w) if return_routing else out

    # ---- per-phase device timing (off by default): CUDA events on the current stream at the phase boundaries
    def enable_phase_timing(self, on: bool = True):
        self._events = [] if on else None

    def _mark(self, name: str):
        ev = getattr(self, "_events", None)
        if ev is None or not torch.cuda.is_available():
            return
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        ev.append((name, e))

    def phase_times_ms(self):
        """{phase: milliseconds} of the last forward() since enable_phase_timing(); waits for the device."""
        ev = getattr(self, "_events", None) or []
        torch.cuda.synchronize()
        out = {}
        for (_, a), (name, bb) in zip(ev[:-1], ev[1:]):
            if name != "start":
                out[name] = out.get(name, 0.0) + a.elapsed_time(bb)
        self._events = []
        return out


class CudaBackend:
    """The product arithmetic: every call goes through the C ABI (edge0_b200.moe)."""

    def __init__(self, ctx, host_layer, rank: int = 0, world: int = 1):
        from . import moe
        cfg = host_layer.cfg
        self.ctx, self.cfg = ctx, cfg
        if cfg.n_latent:
            # The owner of an expert sees a plain layer of the latent width and cannot know that its rows are re-quantised
            # again by the up-projection on the token's rank: pin what the library does by default for a latent layer it sees
            # whole (tensor-core gate/up with the exact re-quantisation fix-up, integer down: bit-identical results).
            ctx.set_expert_path(5)
        E, per = cfg.n_expert, cfg.n_expert // world
        lo, hi = rank * per, (rank + 1) * per
        if host_layer.gate.shape[0] == per and world > 1:      # generated for this shard only (make_layer(expert_range=...))
            assert host_layer.expert_lo == lo
            sl = lambda a: a
        else:
            sl = lambda a: None if a is None else a[lo:hi]
        dev = torch.device("cuda", ctx.device)
        put = lambda a, dt: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev, dt)
        # full layer descriptor for routing (router only needs router_w; expert pointers point at the local shard)
        self.route_layer = moe.MoeLayer(ctx, wtype=cfg.wtype, top_k=cfg.top_k, router_w=host_layer.router_w, router_bias=host_layer.router_bias,
                                        gate=host_layer.gate[:1], up=host_layer.up[:1], down=host_layer.down[:1],
                                        lat_down=host_layer.lat_down, lat_up=host_layer.lat_up, check_shapes=False)  # used for routing only
        # local experts as a plain (non-latent) layer of width L with one slot per row
        self.local = moe.MoeLayer(ctx, wtype=cfg.wtype, top_k=1, router_w=np.zeros((per, cfg.n_in), np.float32), gate=sl(host_layer.gate),
                                  up=sl(host_layer.up), down=sl(host_layer.down), gate_scale=sl(host_layer.gate_scale),
                                  up_scale=sl(host_layer.up_scale), down_scale=sl(host_layer.down_scale))
        self.lat_down, self.lat_up = put(host_layer.lat_down, torch.uint8), put(host_layer.lat_up, torch.uint8)
        self.s_d, self.s_u = put(host_layer.lat_down_scale, torch.float32), put(host_layer.lat_up_scale, torch.float32)
        self.ones = None

    def route(self, x):
        return self.route_layer.route(x)

    def project_down(self, x):
        return self.ctx.mul_mat(self.cfg.wtype, self.lat_down, x.float() if x.dtype != torch.float32 else x, self.cfg.n_embd, self.s_d)

    def project_up(self, m):
        return self.ctx.mul_mat(self.cfg.wtype, self.lat_up, m, self.cfg.n_latent, self.s_u)

    def expert_rows(self, rows, local_eid):
        R = rows.shape[0]
        if R == 0:
            return torch.empty((0, self.cfg.n_in), dtype=torch.float32, device=rows.device)
        if self.ones is None or self.ones.shape[0] < R:
            self.ones = torch.ones((max(R, 1024), 1), dtype=torch.float32, device=rows.device)
        return self.local.ffn(rows, local_eid.reshape(R, 1), self.ones[:R])

    def gather_rows(self, src, idx):
        return self.ctx.gather_rows(src, idx)

    def combine(self, y, w):
        return self.ctx.combine(y.contiguous(), w)
