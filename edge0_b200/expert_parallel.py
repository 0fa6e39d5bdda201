"""Expert-parallel latent MoE layer over the GPUs of one box (one process per GPU, torch.distributed for the exchange).

Semantics follow edge0-strata's latent layer with one label group (src/latent/latent_moe.cpp:38-92):
    x [T, H] --D--> xl [T, L] --experts (L -> I -> L), top-k--> combine in slot order --U--> out [T, H]
The reference has no multi-GPU form of it; the partition here is:
  * tokens are split evenly over ranks for routing, D, the combine and U;
  * expert e lives on rank e // (E / N) (contiguous blocks), so expert weights are never moved;
  * one exchange each way: routed latent rows travel to their expert's owner, result rows travel back.

The exchange is planned on the DEVICE.  Every rank sends every peer the same number of SLOTS (`capacity` = the routed rows a rank
can have, T_local_max * k), so both all-to-alls have equal split sizes that are known before the step starts: no count is read
on the host between routing and the collective, nothing is allocated, and the whole step (route, D, pack, all-to-all, experts,
all-to-all, combine, U) is plain stream work that a CUDA graph can capture.  A slot is the fp32 row followed by the expert id
local to the destination rank; id -1 marks an empty slot, which the owner's kernels skip.

Every routed row is computed by exactly the arithmetic of the single-GPU layer (one slot of weight 1.0 on the owner's pinned
kernel path), and the slot-order sum happens on the token's own rank, so results do not depend on N.

`backend` supplies the arithmetic.  CudaBackend calls the C ABI; tests on CPU plug in a backend made of the checker's functions
(with pack_slots / combine_slots below as the host statement of the slot format) to exercise this file over gloo.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

SLOT_EXTRA_WORDS = 4   # behind the row: expert id + padding to 16 bytes (b200moe_ep_slot_bytes)


def expert_owner(n_expert: int, world: int, e):
    return e // (n_expert // world)


def token_range(n_tokens: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, as even as possible; earlier ranks take the remainder."""
    base, rem = divmod(n_tokens, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def slot_capacity(n_tokens_total: int, world: int, top_k: int) -> int:
    """Slots every rank sends to every peer: the routed rows of the rank with the most tokens, rounded up to a multiple of 4."""
    t_max = -(-n_tokens_total // world)
    return max(4, (t_max * top_k + 3) // 4 * 4)


def pack_slots(rows: np.ndarray, ids: np.ndarray, world: int, experts_per_rank: int, capacity: int):
    """Host statement of b200moe_ep_pack: rows float32 [T, w], ids int32 [T, k] -> (slots float32 [world, capacity, w + 4] with the
    expert id stored bitwise in word w, slot_of int32 [T, k]).  Rows are placed per destination in routed-row order (the device
    kernel places them in arrival order: any order is valid, slot_of records it)."""
    T, w = rows.shape
    k = ids.shape[1]
    slots = np.zeros((world, capacity, w + SLOT_EXTRA_WORDS), np.float32)
    slots.view(np.int32)[:, :, w] = -1
    fill = [0] * world
    slot_of = np.empty((T, k), np.int32)
    for t in range(T):
        for s in range(k):
            dest = int(ids[t, s]) // experts_per_rank
            pos = fill[dest]
            fill[dest] += 1
            slots[dest, pos, :w] = rows[t]
            slots.view(np.int32)[dest, pos, w] = int(ids[t, s]) - dest * experts_per_rank
            slot_of[t, s] = dest * capacity + pos
    return slots, slot_of


def combine_slots(back: np.ndarray, slot_of: np.ndarray, weights: np.ndarray) -> np.ndarray:
    """Host statement of b200moe_ep_combine: slots added in order, each product rounded to fp32 first."""
    if slot_of.shape[0] == 0:
        return np.zeros((0, back.shape[1]), np.float32)
    acc = back[slot_of[:, 0]] * weights[:, 0:1]
    for s in range(1, slot_of.shape[1]):
        acc = acc + back[slot_of[:, s]] * weights[:, s:s + 1]
    return acc.astype(np.float32)


class ExpertParallelLayer:
    """One rank's share of the layer.

    backend.route(x)                            -> ids int32 [T,k], weights float32 [T,k]      (full router, replicated)
    backend.project_down(x) / project_up(m)                                                    (shared D / U, replicated)
    backend.pack(xl, ids, world, per, capacity) -> slots [world, capacity, slot], slot_of int32 [T,k]
    backend.expert_rows(slots [n_slots, slot])  -> float32 [n_slots, L]                        (this rank's experts only)
    backend.combine(back [n_slots, L], slot_of, w) -> float32 [T, L]
    backend.exchange_buffer(t)                  -> tensor like t that receives the all-to-all
    """

    def __init__(self, backend, n_expert: int, top_k: int, rank: int = 0, world: int = 1, group=None, capacity: Optional[int] = None):
        if n_expert % world:
            raise ValueError("n_expert must divide evenly over the ranks")
        self.b, self.E, self.k, self.rank, self.world, self.group = backend, n_expert, top_k, rank, world, group
        if world > 1 and capacity is None:
            raise ValueError("capacity (slot_capacity(total tokens, world, top_k)) must be the same on every rank")
        self.capacity = capacity       # None (single rank): derived from the first batch
        self._events = None

    def forward(self, x_local: torch.Tensor, return_routing: bool = False):
        """x_local: this rank's tokens [T_local, H] -> out [T_local, H]."""
        b, k, N = self.b, self.k, self.world
        T = x_local.shape[0]
        if self.capacity is None:
            self.capacity = max(4, (T * k + 3) // 4 * 4)
        cap = self.capacity
        if T * k > cap:
            raise ValueError(f"{T} tokens x top-{k} exceed the slot capacity {cap} this layer was built for")
        mark = self._mark
        mark("start")
        if hasattr(b, "route_and_project"):                          # independent of each other: the backend may run them side by side
            ids, w, xl = b.route_and_project(x_local)
        else:
            ids, w = b.route(x_local)                                # [T,k]
            xl = b.project_down(x_local)                             # [T,L] float32
        mark("route+D")
        slots, slot_of = b.pack(xl, ids, N, self.E // N, cap)         # [N, cap, slot]
        recv = self._exchange(slots)
        mark("dispatch")
        y = b.expert_rows(recv.reshape(N * cap, -1))                  # [N*cap, L]; row (p, s) answers slot s of peer p
        mark("experts")
        back = self._exchange(y.reshape(N, cap, -1)).reshape(N * cap, -1)
        mark("return")
        moe = b.combine(back, slot_of, w)                             # slot-order weighted sum on the token's rank
        out = b.project_up(moe)
        mark("combine+U")
        return (out, ids, w) if return_routing else out

    def _exchange(self, t: torch.Tensor) -> torch.Tensor:
        """[N, ...] -> [N, ...]: chunk p goes to rank p, chunk p of the result came from rank p.  Equal splits."""
        if self.world == 1:
            return t
        out = self.b.exchange_buffer(t)
        dist.all_to_all_single(out, t, group=self.group)
        return out

    # ---- per-phase device timing (off by default): CUDA events on the current stream at the phase boundaries
    def enable_phase_timing(self, on: bool = True):
        self._events = [] if on else None

    def _mark(self, name: str):
        ev = self._events
        if ev is None or not torch.cuda.is_available():
            return
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        ev.append((name, e))

    def phase_times_ms(self):
        """{phase: milliseconds} of the last forward() since enable_phase_timing(); waits for the device."""
        ev = self._events or []
        torch.cuda.synchronize()
        out = {}
        for (_, a), (name, bb) in zip(ev[:-1], ev[1:]):
            if name != "start":
                out[name] = out.get(name, 0.0) + a.elapsed_time(bb)
        self._events = []
        return out


class CudaBackend:
    """The product arithmetic: every call goes through the C ABI (edge0_b200.moe).  Buffers of a step are allocated once and
    reused, so a captured step replays on fixed addresses."""

    def __init__(self, ctx, host_layer, rank: int = 0, world: int = 1):
        from . import moe
        cfg = host_layer.cfg
        self.ctx, self.cfg = ctx, cfg
        if cfg.n_latent:
            # The owner of an expert sees a plain layer of the latent width and cannot know that its rows are re-quantised
            # again by the up-projection on the token's rank: pin what the library does by default for a latent layer it sees
            # whole (FP4 tensor-core gate/up with the exact re-quantisation fix-up, FP4 down).  A pinned path also keeps the
            # choice of kernels - and with it every routed row's arithmetic - independent of how many rows a rank receives.
            ctx.set_expert_path(8)
        per = cfg.n_expert // world
        lo, hi = rank * per, (rank + 1) * per
        if host_layer.gate.shape[0] == per and world > 1:      # generated for this shard only (make_layer(expert_range=...))
            assert host_layer.expert_lo == lo
            sl = lambda a: a
        else:
            sl = lambda a: None if a is None else a[lo:hi]
        dev = torch.device("cuda", ctx.device)
        # full layer descriptor for routing (router only needs router_w; expert pointers point at the local shard)
        self.route_layer = moe.MoeLayer(ctx, wtype=cfg.wtype, top_k=cfg.top_k, router_w=host_layer.router_w, router_bias=host_layer.router_bias,
                                        gate=host_layer.gate[:1], up=host_layer.up[:1], down=host_layer.down[:1],
                                        lat_down=host_layer.lat_down, lat_up=host_layer.lat_up, lat_down_scale=host_layer.lat_down_scale,
                                        lat_up_scale=host_layer.lat_up_scale, check_shapes=False)   # router and latent projections only
        # local experts as a plain (non-latent) layer of width L with one slot per row
        self.local = moe.MoeLayer(ctx, wtype=cfg.wtype, top_k=1, router_w=np.zeros((per, cfg.n_in), np.float32), gate=sl(host_layer.gate),
                                  up=sl(host_layer.up), down=sl(host_layer.down), gate_scale=sl(host_layer.gate_scale),
                                  up_scale=sl(host_layer.up_scale), down_scale=sl(host_layer.down_scale))
        self.dev = dev
        self._buf = {}
        # The router and the latent down-projection read the same tokens and nothing of each other: the router gets a context
        # (scratch memory) and a stream of its own, so the two run side by side (both are small grids that leave SMs idle).
        self.ctx_router = moe.Context(ctx.device)
        self.router = moe.MoeLayer(self.ctx_router, wtype=cfg.wtype, top_k=cfg.top_k, router_w=host_layer.router_w, router_bias=host_layer.router_bias,
                                   gate=host_layer.gate[:1], up=host_layer.up[:1], down=host_layer.down[:1], check_shapes=False)
        self._side = torch.cuda.Stream(device=dev)

    def _get(self, name, shape, dtype, zero=False):
        t = self._buf.get(name)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
            t = (torch.zeros if zero else torch.empty)(tuple(shape), dtype=dtype, device=self.dev)
            self._buf[name] = t
        return t

    def route(self, x):
        return self.route_layer.route(x)

    def project_down(self, x):
        return self.route_layer.latent_down(x)

    def route_and_project(self, x):
        """(ids, weights, latent rows): routing on the side stream while the down-projection runs on the caller's."""
        T = x.shape[0]
        ids = self._get("ids", (T, self.cfg.top_k), torch.int32)
        w = self._get("w", (T, self.cfg.top_k), torch.float32)
        xl = self._get("xl", (T, self.cfg.n_latent), torch.float32)
        cur = torch.cuda.current_stream(self.dev)
        self._side.wait_stream(cur)
        with torch.cuda.stream(self._side):
            self.router.route(x, out=(ids, w))
        self.route_layer.latent_down(x, out=xl)
        cur.wait_stream(self._side)
        return ids, w, xl

    def project_up(self, m):
        return self.route_layer.latent_up(m)

    def pack(self, xl, ids, world, per, capacity):
        sb = int(self.ctx.lib.b200moe_ep_slot_bytes(xl.shape[1]))
        slots = self._get("slots", (world, capacity, sb), torch.uint8)
        slot_of = self._get("slot_of", tuple(ids.shape), torch.int32)
        fill = self._get("fill", (world,), torch.int32)
        return self.ctx.ep_pack(xl, ids, world, per, capacity, slots, slot_of, fill)

    def exchange_buffer(self, t):
        return self._get("xchg_%s" % t.dtype, tuple(t.shape), t.dtype)

    def expert_rows(self, slots):
        y = self._get("y", (slots.shape[0], self.cfg.n_in), torch.float32, zero=True)
        return self.local.ep_expert_rows(slots, y)

    def combine(self, back, slot_of, w):
        return self.ctx.ep_combine(back, slot_of, w)
