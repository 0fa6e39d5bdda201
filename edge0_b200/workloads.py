"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark configurations.

No dataset is involved: every tensor is drawn from a seeded numpy Generator and quantised on the host.
  router   F32 [E, H]   ~ N(0, 0.02)
  experts  gate/up [E, I, n_in], down [E, n_in, I] ~ N(0, 0.02), then Q3_K or NVFP4
           (Q3_K: through the quantiser the caller passes - the tests pass the checker's, i.e. the reference's algorithm; without
           one the blocks are drawn directly in the quantised domain with the statistics such draws have, see synth_q3_K)
  x        [T, H] ~ N(0, 1) (F32, or rounded to bf16)
NVFP4 uses a two-level scheme: each expert matrix is divided by its fp32 tensor scale
s = amax / (6 * 448) before block quantisation (so the UE4M3 block scales sit in their normal range) and s
is handed to the layer as the per-expert scale that multiplies the matmul result.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np

from . import moe
from .capi import TYPE_NVFP4, TYPE_Q3_K


@dataclass
class LayerConfig:
    name: str
    wtype: int
    n_embd: int = 2048
    n_expert: int = 128
    top_k: int = 8
    n_ff: int = 768
    n_latent: int = 0
    n_ff_shexp: int = 0          # > 0: shared expert of this intermediate width with a sigmoid gate (edge0-infer forward.cpp:312-314)
    router_bias: bool = False
    tensor_scales: bool = True   # NVFP4 only
    seed: int = 0

    @property
    def n_in(self) -> int:
        return self.n_latent or self.n_embd


CONFIGS = {
    # BASELINE configs[0]: Q3_K decode
    "c1_q3k": LayerConfig("c1_q3k", TYPE_Q3_K, seed=101),
    # configs[1]: NVFP4 batched decode
    "c2_nvfp4": LayerConfig("c2_nvfp4", TYPE_NVFP4, seed=102),
    # configs[2]: NVFP4 prefill with per-expert logit bias
    "c3_nvfp4_prefill": LayerConfig("c3_nvfp4_prefill", TYPE_NVFP4, router_bias=True, seed=103),
    # configs[4]: latent expert-parallel layer
    "c5_latent": LayerConfig("c5_latent", TYPE_NVFP4, n_embd=4096, n_latent=1024, n_expert=512, top_k=10, n_ff=1024, seed=105),
}


@dataclass
class HostLayer:
    cfg: LayerConfig
    router_w: np.ndarray
    gate: np.ndarray
    up: np.ndarray
    down: np.ndarray
    router_bias: Optional[np.ndarray] = None
    gate_scale: Optional[np.ndarray] = None
    up_scale: Optional[np.ndarray] = None
    down_scale: Optional[np.ndarray] = None
    lat_down: Optional[np.ndarray] = None
    lat_up: Optional[np.ndarray] = None
    lat_down_scale: Optional[np.ndarray] = None
    lat_up_scale: Optional[np.ndarray] = None
    gate_shexp: Optional[np.ndarray] = None
    up_shexp: Optional[np.ndarray] = None
    down_shexp: Optional[np.ndarray] = None
    gate_inp_shexp: Optional[np.ndarray] = None
    expert_lo: int = 0   # first expert held in gate/up/down when the layer was generated for a shard

    def kwargs(self) -> dict:
        """Keyword arguments shared by edge0_b200.moe.MoeLayer and the checkers' moe_layer."""
        return dict(router_w=self.router_w, gate=self.gate, up=self.up, down=self.down, router_bias=self.router_bias)

    def to_device(self, ctx) -> "moe.MoeLayer":
        return moe.MoeLayer(ctx, wtype=self.cfg.wtype, top_k=self.cfg.top_k, router_w=self.router_w, gate=self.gate, up=self.up,
                            down=self.down, router_bias=self.router_bias, gate_scale=self.gate_scale, up_scale=self.up_scale,
                            down_scale=self.down_scale, lat_down=self.lat_down, lat_up=self.lat_up,
                            lat_down_scale=self.lat_down_scale, lat_up_scale=self.lat_up_scale, gate_shexp=self.gate_shexp,
                            up_shexp=self.up_shexp, down_shexp=self.down_shexp, gate_inp_shexp=self.gate_inp_shexp)

    def checker_kwargs(self) -> dict:
        return dict(wtype=self.cfg.wtype, router_w=self.router_w, gate=self.gate, up=self.up, down=self.down, top_k=self.cfg.top_k,
                    router_bias=self.router_bias, s_gate=self.gate_scale, s_up=self.up_scale, s_down=self.down_scale,
                    lat_d=self.lat_down, lat_u=self.lat_up, s_lat_d=self.lat_down_scale, s_lat_u=self.lat_up_scale,
                    sh_gate=self.gate_shexp, sh_up=self.up_shexp, sh_down=self.down_shexp, sh_gate_inp=self.gate_inp_shexp)


# code frequencies (-4 .. 3) of block_q3_K quantised from N(0, sigma) draws by the reference quantiser
_Q3K_CODE_P = np.array([0.0757, 0.0633, 0.1142, 0.1757, 0.2051, 0.1757, 0.1135, 0.0768])


def synth_q3_K(rng: np.random.Generator, shape) -> np.ndarray:
    """ggml block_q3_K bytes [..., n/256*110] drawn in the QUANTISED domain: 3-bit codes with the frequencies that quantised
    Gaussian weights show, 6-bit sub-block scales of magnitude 12..32 (one of them the extreme -32, as the quantiser's
    normalisation leaves it), an fp16 super-block scale near 4.9e-4 of either sign: dequantised values ~ N(0, 0.02).
    For timing and for kernel tests that need no particular weights; parity tests quantise real draws with the checker."""
    *lead, n = shape
    nb = int(np.prod(lead)) * (n // 256)
    codes = rng.choice(8, size=(nb, 256), p=_Q3K_CODE_P / _Q3K_CODE_P.sum()).astype(np.uint8)      # code + 4
    sc = (rng.integers(12, 33, (nb, 16)) * rng.choice([-1, 1], (nb, 16))).astype(np.int32)
    sc[np.arange(nb), rng.integers(0, 16, nb)] = -32
    sc = np.clip(sc, -32, 31) + 32
    out = np.zeros((nb, 110), np.uint8)
    lo2, hb = codes & 3, codes >> 2                      # element idx = 128*half + 32*shift + l
    for half in range(2):
        for shift in range(4):
            cols = slice(128 * half + 32 * shift, 128 * half + 32 * shift + 32)
            out[:, 32 + 32 * half:64 + 32 * half] |= (lo2[:, cols] << (2 * shift)).astype(np.uint8)
            out[:, 0:32] |= (hb[:, cols] << (4 * half + shift)).astype(np.uint8)
    for j in range(16):                                  # 6-bit scales: low 4 bits in nibbles of bytes 0-7, high 2 bits in bytes 8-11
        l = sc[:, j]
        if j < 8:
            out[:, 96 + j] |= (l & 0xF).astype(np.uint8)
        else:
            out[:, 96 + j - 8] |= ((l & 0xF) << 4).astype(np.uint8)
        out[:, 96 + 8 + j % 4] |= ((l >> 4) << (2 * (j // 4))).astype(np.uint8)
    d = (rng.uniform(3.5e-4, 6.5e-4, nb) * rng.choice([-1.0, 1.0], nb)).astype(np.float16)
    out[:, 108:110] = d.view(np.uint8).reshape(nb, 2)
    return out.reshape(*lead, n // 256 * 110)


def _quantize(wtype: int, w: np.ndarray, quantize_q3k: Optional[Callable]) -> np.ndarray:
    if wtype == TYPE_NVFP4:
        return moe.quantize_nvfp4(w)
    return quantize_q3k(w)


CHUNK_EXPERTS = 32


def _matrix(seed_key, shape, wtype, scaled, quantize_q3k, expert_range=None):
    """Draw and quantise [E, rows, n] in chunks of CHUNK_EXPERTS experts.  Every chunk has its own seeded generator, so
    a rank that owns only some experts draws only their chunks and still gets the same bytes as a full draw."""
    E = shape[0]
    lo, hi = expert_range if expert_range is not None else (0, E)
    outs, scales = [], []
    for e0 in range(0, E, CHUNK_EXPERTS):
        e1 = min(E, e0 + CHUNK_EXPERTS)
        if e1 <= lo or e0 >= hi:
            continue
        rng = np.random.default_rng(list(seed_key) + [e0 // CHUNK_EXPERTS])
        a, b = max(lo, e0) - e0, min(hi, e1) - e0
        if wtype == TYPE_Q3_K and quantize_q3k is None:
            outs.append(synth_q3_K(rng, (e1 - e0,) + tuple(shape[1:]))[a:b])
            continue
        w = rng.normal(0.0, 0.02, (e1 - e0,) + tuple(shape[1:])).astype(np.float32)
        w = w[a:b]
        if scaled:
            s = (np.abs(w).reshape(b - a, -1).max(axis=1) / np.float32(6 * 448)).astype(np.float32)
            w = w / s[:, None, None]
            scales.append(s)
        outs.append(_quantize(wtype, w, quantize_q3k))
    return np.concatenate(outs, axis=0), (np.concatenate(scales) if scaled else None)


def make_layer(cfg: LayerConfig, quantize_q3k: Optional[Callable] = None, seed_offset: int = 0, expert_range=None) -> HostLayer:
    """expert_range=(lo, hi): only those experts' gate/up/down (and scales) are generated; router and latent projections are
    always complete."""
    seed = cfg.seed + 7919 * seed_offset
    rng = np.random.default_rng([seed, 0])
    E, H, I, n_in = cfg.n_expert, cfg.n_embd, cfg.n_ff, cfg.n_in
    scaled = cfg.wtype == TYPE_NVFP4 and cfg.tensor_scales
    router_w = rng.normal(0.0, 0.02, (E, H)).astype(np.float32)
    gate, sg = _matrix([seed, 1], (E, I, n_in), cfg.wtype, scaled, quantize_q3k, expert_range)
    up, su = _matrix([seed, 2], (E, I, n_in), cfg.wtype, scaled, quantize_q3k, expert_range)
    down, sd = _matrix([seed, 3], (E, n_in, I), cfg.wtype, scaled, quantize_q3k, expert_range)
    layer = HostLayer(cfg, router_w, gate, up, down, gate_scale=sg, up_scale=su, down_scale=sd)
    layer.expert_lo = expert_range[0] if expert_range is not None else 0
    if cfg.router_bias:
        layer.router_bias = rng.normal(0.0, 1.0, E).astype(np.float32)
    if cfg.n_ff_shexp:
        # shared expert: dense tensors of the experts' type, quantised without a tensor scale; its gate vector stays F32
        Is = cfg.n_ff_shexp
        layer.gate_shexp = _matrix([seed, 6], (1, Is, H), cfg.wtype, False, quantize_q3k)[0][0]
        layer.up_shexp = _matrix([seed, 7], (1, Is, H), cfg.wtype, False, quantize_q3k)[0][0]
        layer.down_shexp = _matrix([seed, 8], (1, H, Is), cfg.wtype, False, quantize_q3k)[0][0]
        layer.gate_inp_shexp = np.random.default_rng([seed, 9]).normal(0.0, 0.02, H).astype(np.float32)
    if cfg.n_latent:
        d, s_d = _matrix([seed, 4], (1, cfg.n_latent, H), cfg.wtype, scaled, quantize_q3k)
        u, s_u = _matrix([seed, 5], (1, H, cfg.n_latent), cfg.wtype, scaled, quantize_q3k)
        layer.lat_down, layer.lat_up = d[0], u[0]
        layer.lat_down_scale, layer.lat_up_scale = s_d, s_u
    return layer


def make_tokens(cfg: LayerConfig, n_tokens: int, bf16: bool = False, seed_offset: int = 0) -> np.ndarray:
    """float32 [T, n_embd] ~ N(0,1); with bf16=True the values are rounded to bf16 (still stored as float32)."""
    rng = np.random.default_rng(cfg.seed * 1000 + 17 + seed_offset)
    x = rng.normal(0.0, 1.0, (n_tokens, cfg.n_embd)).astype(np.float32)
    if bf16:
        u = x.view(np.uint32)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)   # round to nearest even
        x = u.view(np.float32)
    return x


def small_config(wtype: int, *, n_embd=512, n_expert=16, top_k=4, n_ff=256, n_latent=0, router_bias=False, seed=1, tensor_scales=True,
                 n_ff_shexp=0):
    return LayerConfig(f"small_{wtype}", wtype, n_embd=n_embd, n_expert=n_expert, top_k=top_k, n_ff=n_ff, n_latent=n_latent,
                       router_bias=router_bias, seed=seed, tensor_scales=tensor_scales, n_ff_shexp=n_ff_shexp)


def algorithmic_bytes(cfg: LayerConfig, n_tokens: int, experts_touched: int, x_bytes_per_elt: int = 4) -> int:
    """Bytes one layer pass must move: routed experts' three matrices, the router, the latent projections, x in, out out."""
    per_matrix = cfg.n_ff * moe.row_size(cfg.wtype, cfg.n_in)
    down = cfg.n_in * moe.row_size(cfg.wtype, cfg.n_ff)
    b = experts_touched * (2 * per_matrix + down) + cfg.n_expert * cfg.n_embd * 4
    if cfg.n_latent:
        b += cfg.n_latent * moe.row_size(cfg.wtype, cfg.n_embd) + cfg.n_embd * moe.row_size(cfg.wtype, cfg.n_latent)
    b += n_tokens * cfg.n_embd * (x_bytes_per_elt + 4)
    return int(b)


def pack_expert_blobs_nvfp4(layer: "HostLayer") -> np.ndarray:
    """The layer's NVFP4 experts as edge0-strata writes them to experts.bin (tools/iq_pack.py; docs/NVFP4.md:44-47): one blob per
    expert, [gate rows | up rows | down rows] + the 16-byte tail {s_gate, s_up, s_down, 0}.  uint8 [n_expert][blob bytes]."""
    E = layer.gate.shape[0]
    one = np.ones(E, np.float32)
    sg = layer.gate_scale if layer.gate_scale is not None else one
    su = layer.up_scale if layer.up_scale is not None else one
    sd = layer.down_scale if layer.down_scale is not None else one
    tail = np.stack([sg, su, sd, np.zeros(E, np.float32)], axis=1).astype(np.float32).view(np.uint8).reshape(E, 16)
    return np.concatenate([layer.gate.reshape(E, -1), layer.up.reshape(E, -1), layer.down.reshape(E, -1), tail], axis=1)
