"""Host-side mirror of the reference's operator interface for the quantised MoE FFN.

Names follow edge0-infer: `route` and `ffn` are Builder::route / Builder::ffn
(edge0-infer/src/models/edge0_35b/forward.cpp:262-271, 300-311), `mul_mat_id` is ggml_mul_mat_id
(third_party/ggml/src/ggml.c:3392-3416).  Tensors are torch CUDA tensors used purely as device memory;
all arithmetic happens in libedge0_b200.so through the C ABI.  Shapes are written row-major, i.e. the
reverse of ggml's ne[] order: x [T, n_embd], ids [T, k], expert tensors [n_expert, n_out, row_bytes].
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import capi
from .capi import TYPE_BF16, TYPE_F32, TYPE_NVFP4, TYPE_Q3_K, B200MoeError, Layer, Observe

TYPE_BY_NAME = {"q3_k": TYPE_Q3_K, "nvfp4": TYPE_NVFP4}


def row_size(wtype: int, n: int) -> int:
    r = capi.load().b200moe_row_size(wtype, n)
    if r < 0:
        raise ValueError(f"width {n} is not a whole number of blocks of type {wtype}")
    return int(r)


def quantize_nvfp4(w: np.ndarray) -> np.ndarray:
    """float32 [..., n] -> ggml block_nvfp4 bytes [..., n/64*36] (quantize_row_nvfp4_ref, ggml-quants.c:384-417)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n = w.shape[-1]
    out = np.empty(w.shape[:-1] + (row_size(TYPE_NVFP4, n),), dtype=np.uint8)
    rc = capi.load().b200moe_quantize_nvfp4_host(w.ctypes.data, out.ctypes.data, w.size // n, n)
    if rc:
        raise B200MoeError(rc, "quantize_nvfp4_host")
    return out


def dequantize(wtype: int, q: np.ndarray, n: int) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    rows = q.size // row_size(wtype, n)
    out = np.empty(q.shape[:-1] + (n,), dtype=np.float32)
    rc = capi.load().b200moe_dequantize_host(wtype, q.ctypes.data, out.ctypes.data, rows, n)
    if rc:
        raise B200MoeError(rc, "dequantize_host")
    return out


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _x_type(x: torch.Tensor) -> int:
    if x.dtype == torch.float32:
        return TYPE_F32
    if x.dtype == torch.bfloat16:
        return TYPE_BF16
    raise TypeError("activations must be float32 or bfloat16")


def unpack_expert_blobs_nvfp4(blobs: np.ndarray, n_embd: int, n_ff: int, device=None):
    """edge0-strata expert blobs (uint8 [n_expert][>= blob bytes]) -> (gate, up, down, gate_scale, up_scale, down_scale) in the layout of
    b200moe_layer: numpy arrays, or torch tensors on `device` when one is given (copied straight from the blobs, no repacking)."""
    lib = capi.load()
    blobs = np.ascontiguousarray(blobs, dtype=np.uint8)
    E, stride = blobs.shape
    need = lib.b200moe_expert_blob_bytes_nvfp4(n_embd, n_ff)
    if need < 0 or stride < need:
        raise ValueError(f"blobs of {stride} bytes cannot hold experts of {n_embd} x {n_ff} ({need} bytes)")
    gu_row, d_row = n_embd // 64 * 36, n_ff // 64 * 36
    if device is None:
        g, u = np.empty((E, n_ff, gu_row), np.uint8), np.empty((E, n_ff, gu_row), np.uint8)
        d = np.empty((E, n_embd, d_row), np.uint8)
        sc = [np.empty(E, np.float32) for _ in range(3)]
        ptr = lambda a: a.ctypes.data
        stream = None
    else:
        g, u = (torch.empty((E, n_ff, gu_row), dtype=torch.uint8, device=device) for _ in range(2))
        d = torch.empty((E, n_embd, d_row), dtype=torch.uint8, device=device)
        sc = [torch.empty(E, dtype=torch.float32, device=device) for _ in range(3)]
        ptr = lambda a: a.data_ptr()
        stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    rc = lib.b200moe_unpack_expert_blobs_nvfp4(blobs.ctypes.data, stride, E, n_embd, n_ff, ptr(g), ptr(u), ptr(d), ptr(sc[0]), ptr(sc[1]), ptr(sc[2]),
                                               0 if device is None else 1, stream)
    if rc:
        raise B200MoeError(rc, "b200moe_unpack_expert_blobs_nvfp4")
    return g, u, d, sc[0], sc[1], sc[2]


class GgufFile:
    """A GGUF model file mapped read-only (b200moe_gguf_*): tensors come out as numpy views of the mapping in ggml's block layout.
    Keep the object alive while such views (or layers built from them before their copy to the device) are in use."""

    def __init__(self, path: str):
        self.lib = capi.load()
        h, err = C.c_void_p(), C.create_string_buffer(256)
        rc = self.lib.b200moe_gguf_open(str(path).encode(), C.byref(h), err, 256)
        if rc:
            raise B200MoeError(rc, err.value.decode())
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.b200moe_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def n_tensors(self) -> int:
        return int(self.lib.b200moe_gguf_n_tensors(self.handle))

    def tensor(self, name: str):
        """(ggml type, ne[4], uint8 view of the tensor's bytes)."""
        t, ne, data, nb = C.c_int32(), (C.c_int64 * 4)(), C.c_void_p(), C.c_uint64()
        rc = self.lib.b200moe_gguf_tensor(self.handle, name.encode(), C.byref(t), C.byref(ne), C.byref(data), C.byref(nb))
        if rc:
            raise B200MoeError(rc, f"tensor {name}")
        buf = (C.c_uint8 * nb.value).from_address(data.value)
        return t.value, tuple(ne), np.frombuffer(buf, dtype=np.uint8)

    def metadata_u64(self, key: str) -> int:
        v = C.c_uint64()
        rc = self.lib.b200moe_gguf_metadata_u64(self.handle, key.encode(), C.byref(v))
        if rc:
            raise KeyError(key)
        return int(v.value)

    def moe_layer_tensors(self, layer: int, top_k: int = 0) -> dict:
        """The MoE FFN tensors of block `layer` as keyword arguments of MoeLayer (numpy views of the mapping; MoeLayer copies them to
        the device as they are)."""
        d, err = Layer(), C.create_string_buffer(256)
        rc = self.lib.b200moe_gguf_moe_layer(self.handle, layer, top_k, C.byref(d), err, 256)
        if rc:
            raise B200MoeError(rc, err.value.decode())
        H, E, I, Is = d.n_embd, d.n_expert, d.n_ff, d.n_ff_shexp
        row = lambda n: int(self.lib.b200moe_row_size(d.wtype, n))

        def view(ptr, shape, dtype):
            if not ptr:
                return None
            n = int(np.prod(shape)) * np.dtype(dtype).itemsize
            return np.frombuffer((C.c_uint8 * n).from_address(ptr), dtype=dtype).reshape(shape)

        out = dict(wtype=d.wtype, top_k=d.n_expert_used, router_w=view(d.router_w, (E, H), np.float32), router_bias=view(d.router_bias, (E,), np.float32),
                   gate=view(d.gate, (E, I, row(H)), np.uint8), up=view(d.up, (E, I, row(H)), np.uint8), down=view(d.down, (E, H, row(I)), np.uint8))
        if Is:
            out.update(gate_shexp=view(d.gate_shexp, (Is, row(H)), np.uint8), up_shexp=view(d.up_shexp, (Is, row(H)), np.uint8),
                       down_shexp=view(d.down_shexp, (H, row(Is)), np.uint8), gate_inp_shexp=view(d.gate_inp_shexp, (H,), np.float32))
        return out


class Context:
    """One per GPU and stream of work (reference: one ggml backend instance, one graph in flight)."""

    def __init__(self, device: int = 0):
        self.lib = capi.load()
        h = C.c_void_p()
        rc = self.lib.b200moe_create(device, C.byref(h))
        if rc:
            raise B200MoeError(rc, "b200moe_create: " + self.lib.b200moe_status_string(rc).decode())
        self.handle = h
        self.device = device

    def close(self):
        if self.handle:
            self.lib.b200moe_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc: int):
        if rc:
            raise B200MoeError(rc, self.lib.b200moe_last_error(self.handle).decode())

    def synchronize(self):
        self.check(self.lib.b200moe_synchronize(self.handle, self._stream()))

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def launches(self) -> int:
        c = capi.Counters()
        self.check(self.lib.b200moe_get_counters(self.handle, C.byref(c)))
        return int(c.kernel_launches)

    def set_expert_path(self, path: int):
        """0 automatic, 1 integer GEMV always, 2 tensor-core grouped GEMM whenever the shape allows."""
        self.check(self.lib.b200moe_set_expert_path(self.handle, path))

    def set_launch_overlap(self, enable: bool) -> None:
        """Programmatic dependent launches between the kernels of a layer (default off); see b200moe_set_launch_overlap."""
        self.check(self.lib.b200moe_set_launch_overlap(self.handle, int(bool(enable))))

    def enable_kernel_timing(self, on: bool = True):
        self.check(self.lib.b200moe_enable_kernel_timing(self.handle, int(on)))

    def kernel_times(self):
        """[(launches, total_ms)] for the fused gate/up kernel, the single indexed matmul (down) and dense products; clears the record."""
        n = (C.c_int64 * 3)()
        ms = (C.c_double * 3)()
        self.check(self.lib.b200moe_kernel_times(self.handle, n, ms))
        return [(int(n[i]), float(ms[i])) for i in range(3)]

    def mul_mat(self, wtype: int, w: torch.Tensor, x: torch.Tensor, ne00: int, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """w uint8 [ne01, row_bytes]; x float32 [T, ne00] -> float32 [T, ne01] (ggml_mul_mat with a quantised matrix)."""
        T, ne01 = x.shape[0], w.shape[0]
        dst = torch.empty((T, ne01), dtype=torch.float32, device=x.device)
        self.check(self.lib.b200moe_mul_mat(self.handle, wtype, _ptr(w), ne00, ne01, _ptr(x), T, _ptr(scale), _ptr(dst), self._stream()))
        return dst

    def combine(self, y: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """y float32 [T, k, n], weights float32 [T, k] -> float32 [T, n], slots added in order."""
        T, k, n = y.shape
        out = torch.empty((T, n), dtype=torch.float32, device=y.device)
        self.check(self.lib.b200moe_combine(self.handle, _ptr(y), _ptr(weights), _ptr(out), n, k, T, self._stream()))
        return out

    def gather_rows(self, src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """src float32 [R, n], idx int32 [m] -> float32 [m, n]."""
        dst = torch.empty((idx.shape[0], src.shape[1]), dtype=torch.float32, device=src.device)
        self.check(self.lib.b200moe_gather_rows(self.handle, _ptr(src), src.shape[0], _ptr(idx), _ptr(dst), idx.shape[0], src.shape[1], self._stream()))
        return dst

    # ---- expert-parallel exchange (b200moe_ep_*): outputs may be passed in so a step allocates nothing
    def ep_pack(self, rows: torch.Tensor, ids: torch.Tensor, n_ranks: int, experts_per_rank: int, capacity: int,
                slots: Optional[torch.Tensor] = None, slot_of: Optional[torch.Tensor] = None, fill: Optional[torch.Tensor] = None):
        """rows float32 [T, w], ids int32 [T, k] -> (slots uint8 [n_ranks, capacity, slot_bytes], slot_of int32 [T, k])."""
        T, w = rows.shape
        k = ids.shape[1]
        sb = int(self.lib.b200moe_ep_slot_bytes(w))
        if slots is None:
            slots = torch.empty((n_ranks, capacity, sb), dtype=torch.uint8, device=rows.device)
        if slot_of is None:
            slot_of = torch.empty((T, k), dtype=torch.int32, device=rows.device)
        if fill is None:
            fill = torch.empty((n_ranks,), dtype=torch.int32, device=rows.device)
        self.check(self.lib.b200moe_ep_pack(self.handle, _ptr(rows), _ptr(ids), T, k, w, n_ranks, experts_per_rank, capacity, _ptr(slots),
                                            _ptr(slot_of), _ptr(fill), self._stream()))
        return slots, slot_of

    def ep_combine(self, back: torch.Tensor, slot_of: torch.Tensor, weights: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """back float32 [n_slots, w], slot_of int32 [T, k], weights float32 [T, k] -> float32 [T, w]."""
        n_slots, w = back.shape
        T, k = slot_of.shape
        if out is None:
            out = torch.empty((T, w), dtype=torch.float32, device=back.device)
        self.check(self.lib.b200moe_ep_combine(self.handle, _ptr(back), n_slots, _ptr(slot_of), _ptr(weights), T, k, w, _ptr(out), self._stream()))
        return out

    def mul_mat_id(self, wtype: int, experts: torch.Tensor, b: torch.Tensor, ids: torch.Tensor, ne00: int) -> torch.Tensor:
        """experts uint8 [n_as, ne01, row_bytes]; b float32 [T, ne11, ne00]; ids int32 [T, n_ids] (may be a
        column slice of a wider tensor) -> float32 [T, n_ids, ne01]."""
        n_as, ne01, _ = experts.shape
        T, ne11, _ = b.shape
        n_ids = ids.shape[1]
        dst = torch.empty((T, n_ids, ne01), dtype=torch.float32, device=b.device)
        self.check(self.lib.b200moe_mul_mat_id(self.handle, wtype, _ptr(experts), ne00, ne01, n_as, _ptr(b), ne11, _ptr(ids), n_ids,
                                               ids.stride(0) * 4 if T > 0 else n_ids * 4, T, _ptr(dst), self._stream()))
        return dst


@dataclass
class Observed:
    logits: torch.Tensor
    probs: torch.Tensor
    topk: torch.Tensor
    weights_norm: torch.Tensor
    hidden: torch.Tensor
    down: torch.Tensor
    shexp_gated: Optional[torch.Tensor] = None


class MoeLayer:
    """Weights of one MoE FFN layer on one GPU plus the calls the reference graph makes on them."""

    def __init__(self, ctx: Context, *, wtype: int, top_k: int, router_w, gate, up, down, router_bias=None, gate_scale=None,
                 up_scale=None, down_scale=None, lat_down=None, lat_up=None, lat_down_scale=None, lat_up_scale=None,
                 gate_shexp=None, up_shexp=None, down_shexp=None, gate_inp_shexp=None, check_shapes=True):
        dev = torch.device("cuda", ctx.device)

        def put(a, dtype):
            if a is None:
                return None
            if isinstance(a, torch.Tensor):
                return a.to(device=dev, dtype=dtype).contiguous()
            return torch.from_numpy(np.ascontiguousarray(a)).to(device=dev, dtype=dtype).contiguous()

        self.ctx, self.wtype, self.top_k = ctx, wtype, top_k
        self.router_w = put(router_w, torch.float32)
        self.router_bias = put(router_bias, torch.float32)
        self.gate, self.up, self.down = put(gate, torch.uint8), put(up, torch.uint8), put(down, torch.uint8)
        self.gate_scale, self.up_scale, self.down_scale = (put(s, torch.float32) for s in (gate_scale, up_scale, down_scale))
        self.lat_down, self.lat_up = put(lat_down, torch.uint8), put(lat_up, torch.uint8)
        self.lat_down_scale, self.lat_up_scale = put(lat_down_scale, torch.float32), put(lat_up_scale, torch.float32)
        self.gate_shexp, self.up_shexp, self.down_shexp = put(gate_shexp, torch.uint8), put(up_shexp, torch.uint8), put(down_shexp, torch.uint8)
        self.gate_inp_shexp = put(gate_inp_shexp, torch.float32)
        self.n_expert, self.n_embd = self.router_w.shape
        self.n_ff = self.gate.shape[1]
        self.n_latent = 0 if self.lat_down is None else self.lat_down.shape[0]
        self.n_in = self.n_latent or self.n_embd
        if check_shapes and self.gate.shape != (self.n_expert, self.n_ff, row_size(wtype, self.n_in)):
            raise ValueError(f"gate tensor has shape {tuple(self.gate.shape)}")
        if check_shapes and self.down.shape != (self.n_expert, self.n_in, row_size(wtype, self.n_ff)):
            raise ValueError(f"down tensor has shape {tuple(self.down.shape)}")
        self.desc = Layer(n_embd=self.n_embd, n_latent=self.n_latent, n_expert=self.n_expert, n_expert_used=top_k, n_ff=self.n_ff,
                          wtype=wtype)
        if self.gate_shexp is not None:
            self.desc.n_ff_shexp = self.gate_shexp.shape[0]
        for name in ("router_w", "router_bias", "gate", "up", "down", "gate_scale", "up_scale", "down_scale", "lat_down", "lat_up",
                     "lat_down_scale", "lat_up_scale", "gate_shexp", "up_shexp", "down_shexp", "gate_inp_shexp"):
            t = getattr(self, name)
            setattr(self.desc, name, None if t is None else t.data_ptr())

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.router_w, self.gate, self.up, self.down, self.lat_down, self.lat_up)
                   if t is not None)

    def _observe(self, T: int, dev) -> tuple[Observe, Observed]:
        k, E = self.top_k, self.n_expert
        o = Observed(logits=torch.empty((T, E), dtype=torch.float32, device=dev), probs=torch.empty((T, E), dtype=torch.float32, device=dev),
                     topk=torch.empty((T, k), dtype=torch.int32, device=dev), weights_norm=torch.empty((T, k), dtype=torch.float32, device=dev),
                     hidden=torch.empty((T, k, self.n_ff), dtype=torch.float32, device=dev),
                     down=torch.empty((T, k, self.n_in), dtype=torch.float32, device=dev))
        s = Observe(ffn_moe_logits=o.logits.data_ptr(), ffn_moe_probs=o.probs.data_ptr(), ffn_moe_topk=o.topk.data_ptr(),
                    ffn_moe_weights_norm=o.weights_norm.data_ptr(), ffn_moe_hidden=o.hidden.data_ptr(), ffn_moe_down=o.down.data_ptr())
        if self.gate_shexp is not None:
            o.shexp_gated = torch.empty((T, self.n_embd), dtype=torch.float32, device=dev)
            s.ffn_shexp_gated = o.shexp_gated.data_ptr()
        return s, o

    def route(self, x: torch.Tensor, out=None):
        """x [T, n_embd] -> (ids int32 [T, k], weights float32 [T, k]); out: that pair, allocated by the caller."""
        T = x.shape[0]
        if out is not None:
            ids, w = out
        else:
            ids = torch.empty((T, self.top_k), dtype=torch.int32, device=x.device)
            w = torch.empty((T, self.top_k), dtype=torch.float32, device=x.device)
        c = self.ctx
        c.check(c.lib.b200moe_route(c.handle, C.byref(self.desc), _ptr(x), _x_type(x), T, _ptr(ids), _ptr(w), None, c._stream()))
        return ids, w

    def ffn(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """x [T, n_in] with given routing -> float32 [T, n_in]."""
        T = x.shape[0]
        out = torch.empty((T, self.n_in), dtype=torch.float32, device=x.device)
        c = self.ctx
        c.check(c.lib.b200moe_ffn(c.handle, C.byref(self.desc), _ptr(x), _x_type(x), T, _ptr(ids.contiguous()), _ptr(weights.contiguous()),
                                  _ptr(out), None, c._stream()))
        return out

    def latent_down(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [T, n_embd] -> latent rows float32 [T, n_latent] (edge0-strata latent_moe.cpp: xl = D x)."""
        T = x.shape[0]
        xl = out if out is not None else torch.empty((T, self.n_latent), dtype=torch.float32, device=x.device)
        c = self.ctx
        c.check(c.lib.b200moe_latent_down(c.handle, C.byref(self.desc), _ptr(x), _x_type(x), T, _ptr(xl), c._stream()))
        return xl

    def latent_up(self, m: torch.Tensor) -> torch.Tensor:
        """m float32 [T, n_latent] -> float32 [T, n_embd] (y = U m)."""
        T = m.shape[0]
        out = torch.empty((T, self.n_embd), dtype=torch.float32, device=m.device)
        c = self.ctx
        c.check(c.lib.b200moe_latent_up(c.handle, C.byref(self.desc), _ptr(m), T, _ptr(out), c._stream()))
        return out

    def ep_expert_rows(self, slots: torch.Tensor, y: Optional[torch.Tensor] = None) -> torch.Tensor:
        """slots uint8 [n_slots, slot_bytes] as received from the exchange -> float32 [n_slots, n_in] (rows of empty slots untouched)."""
        n_slots = slots.numel() // slots.shape[-1]
        if y is None:
            y = torch.zeros((n_slots, self.n_in), dtype=torch.float32, device=slots.device)
        c = self.ctx
        c.check(c.lib.b200moe_ep_expert_rows(c.handle, C.byref(self.desc), _ptr(slots), n_slots, _ptr(y), c._stream()))
        return y

    def forward(self, x: torch.Tensor, observe: bool = False, out: Optional[torch.Tensor] = None):
        """The whole layer on device tensors: x [T, n_embd] -> float32 [T, n_embd] (and the observation tensors)."""
        T = x.shape[0]
        if out is None:
            out = torch.empty((T, self.n_embd), dtype=torch.float32, device=x.device)
        c = self.ctx
        if observe:
            s, o = self._observe(T, x.device)
            c.check(c.lib.b200moe_layer_forward(c.handle, C.byref(self.desc), _ptr(x), _x_type(x), T, _ptr(out), C.byref(s), c._stream()))
            return out, o
        c.check(c.lib.b200moe_layer_forward(c.handle, C.byref(self.desc), _ptr(x), _x_type(x), T, _ptr(out), None, c._stream()))
        return out

    def forward_host(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, ids: Optional[torch.Tensor] = None,
                     weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Same with HOST tensors (ideally pinned): copies in, computes, copies out, waits."""
        assert not x.is_cuda
        T = x.shape[0]
        if out is None:
            out = torch.empty((T, self.n_embd), dtype=torch.float32)
        c = self.ctx
        c.check(c.lib.b200moe_layer_forward_host(c.handle, C.byref(self.desc), _ptr(x), _x_type(x), T, _ptr(out), _ptr(ids), _ptr(weights),
                                                 c._stream()))
        return out
