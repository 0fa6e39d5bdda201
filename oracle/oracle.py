"""TEST INFRASTRUCTURE: ctypes access to the two CPU checkers.

* ``restatement()`` -> oracle/libmoe_oracle.so, the plain-C restatement (moe_oracle.c).
* ``reference()``   -> oracle/_ref/libedge0_ref.so, the reference's own ggml CPU backend compiled by
  oracle/Makefile (present only where it was built; it travels as a binary).

Only tests, the smoke check and the benchmark's cpu_baseline / reference arm import this module.
The product package (edge0_b200) never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
RESTATEMENT_SO = os.path.join(HERE, "libmoe_oracle.so")
REFERENCE_SO = os.path.join(HERE, "_ref", "libedge0_ref.so")

TYPE_F32, TYPE_Q3_K, TYPE_NVFP4 = 0, 11, 40
TYPE_BY_NAME = {"f32": TYPE_F32, "q3_k": TYPE_Q3_K, "nvfp4": TYPE_NVFP4}


class MoeArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("H", "L", "E", "K", "I", "T", "wtype", "n_threads", "repeats", "latent")] + [
        (n, C.c_void_p)
        for n in (
            "x", "router_w", "router_bias", "gate", "up", "down", "s_gate", "s_up", "s_down",
            "lat_d", "lat_u", "s_lat_d", "s_lat_u",
            "logits", "probs", "ids", "weights", "hidden", "down_out", "moe_out", "out", "ms_best", "ms_median",
            "sh_gate", "sh_up", "sh_down", "sh_gate_inp", "shexp_gated",
        )
    ] + [("I_sh", C.c_int32), ("pad_", C.c_int32)]


def build(which: str = "restatement") -> None:
    """Compile a checker with oracle/Makefile (gcc only; `ref` needs the reference tree)."""
    subprocess.check_call(["make", "-s", "-C", HERE, which])


def row_size(wtype: int, n: int) -> int:
    return {TYPE_F32: 4 * n, TYPE_Q3_K: n // 256 * 110, TYPE_NVFP4: n // 64 * 36}[wtype]


def act_row_size(wtype: int, n: int) -> int:
    return {TYPE_Q3_K: n // 256 * 292, TYPE_NVFP4: n // 32 * 34}[wtype]


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


@dataclass
class LayerResult:
    logits: np.ndarray
    probs: np.ndarray
    ids: np.ndarray
    weights: np.ndarray
    hidden: np.ndarray
    down_out: np.ndarray
    moe_out: np.ndarray
    out: np.ndarray
    ms_best: float
    ms_median: float
    shexp_gated: np.ndarray = None


class _Checker:
    prefix = ""

    def __init__(self, path: str, mode: int = C.DEFAULT_MODE):
        self.path = path
        self.lib = C.CDLL(path, mode=mode)
        p = self.prefix
        getattr(self.lib, p + "moe_layer").argtypes = [C.POINTER(MoeArgs)]
        getattr(self.lib, p + "moe_layer").restype = C.c_int
        q = getattr(self.lib, p + "quantize")
        q.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
        q.restype = C.c_int
        d = getattr(self.lib, p + "dequantize")
        d.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        d.restype = C.c_int
        qa = getattr(self.lib, p + "quantize_activation")
        qa.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        qa.restype = C.c_int64
        vd = getattr(self.lib, p + "vec_dot")
        vd.argtypes = [C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
        vd.restype = C.c_int

    # -- formats
    def quantize(self, wtype: int, w: np.ndarray) -> np.ndarray:
        """w: float32 [..., n_per_row] -> uint8 [..., row_size]."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        n = w.shape[-1]
        rows = w.size // n
        out = np.empty(w.shape[:-1] + (row_size(wtype, n),), dtype=np.uint8)
        rc = getattr(self.lib, self.prefix + "quantize")(wtype, _ptr(w), _ptr(out), rows, n)
        if rc:
            raise RuntimeError(f"{self.prefix}quantize: type {wtype} not supported by this checker")
        return out

    def dequantize(self, wtype: int, q: np.ndarray, n_per_row: int) -> np.ndarray:
        q = np.ascontiguousarray(q, dtype=np.uint8)
        rows = q.size // row_size(wtype, n_per_row)
        out = np.empty(q.shape[:-1] + (n_per_row,), dtype=np.float32)
        rc = getattr(self.lib, self.prefix + "dequantize")(wtype, _ptr(q), _ptr(out), rows * n_per_row)
        if rc:
            raise RuntimeError("dequantize failed")
        return out

    def quantize_activation(self, wtype: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        n = x.shape[-1]
        out = np.empty(x.shape[:-1] + (act_row_size(wtype, n),), dtype=np.uint8)
        xs = x.reshape(-1, n)
        os_ = out.reshape(-1, out.shape[-1])
        f = getattr(self.lib, self.prefix + "quantize_activation")
        for i in range(xs.shape[0]):
            f(wtype, xs[i].ctypes.data_as(C.c_void_p), os_[i].ctypes.data_as(C.c_void_p), n)
        return out

    def vec_dot(self, wtype: int, n: int, wrow: np.ndarray, act: np.ndarray) -> float:
        out = np.zeros(1, dtype=np.float32)
        getattr(self.lib, self.prefix + "vec_dot")(wtype, n, _ptr(wrow), _ptr(act), _ptr(out))
        return float(out[0])

    # -- the layer
    def moe_layer(self, *, wtype, x, router_w, gate, up, down, top_k, router_bias=None,
                  s_gate=None, s_up=None, s_down=None, lat_d=None, lat_u=None, s_lat_d=None, s_lat_u=None,
                  sh_gate=None, sh_up=None, sh_down=None, sh_gate_inp=None,
                  n_threads=1, repeats=0, backend=None, use_gallocr=False) -> LayerResult:
        """backend: a ggml_backend_t (ctypes void pointer) to run the reference's graph on instead of its CPU backend
        (compiled reference only); use_gallocr: let ggml's graph allocator place the intermediate tensors."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        T, H = x.shape
        E = router_w.shape[0]
        I = gate.shape[1]
        latent = lat_d is not None
        L = lat_d.shape[0] if latent else H
        K = top_k
        f32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)
        u8 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.uint8)
        keep = dict(x=x, router_w=f32(router_w), router_bias=f32(router_bias), gate=u8(gate), up=u8(up), down=u8(down),
                    s_gate=f32(s_gate), s_up=f32(s_up), s_down=f32(s_down), lat_d=u8(lat_d), lat_u=u8(lat_u),
                    s_lat_d=f32(s_lat_d), s_lat_u=f32(s_lat_u), sh_gate=u8(sh_gate), sh_up=u8(sh_up), sh_down=u8(sh_down),
                    sh_gate_inp=f32(sh_gate_inp))
        assert keep["router_w"].shape == (E, H)
        assert keep["gate"].shape == (E, I, row_size(wtype, L)), (keep["gate"].shape, (E, I, row_size(wtype, L)))
        assert keep["down"].shape == (E, L, row_size(wtype, I))
        res = LayerResult(
            logits=np.zeros((T, E), np.float32), probs=np.zeros((T, E), np.float32),
            ids=np.zeros((T, K), np.int32), weights=np.zeros((T, K), np.float32),
            hidden=np.zeros((T, K, I), np.float32), down_out=np.zeros((T, K, L), np.float32),
            moe_out=np.zeros((T, L), np.float32), out=np.zeros((T, H if latent else L), np.float32),
            ms_best=0.0, ms_median=0.0)
        best, med = C.c_double(0), C.c_double(0)
        a = MoeArgs(H=H, L=L, E=E, K=K, I=I, T=T, wtype=wtype, n_threads=n_threads, repeats=repeats, latent=int(latent))
        if sh_gate is not None:
            assert not latent, "the shared expert is defined for plain layers"
            a.I_sh = keep["sh_gate"].shape[0]
            res.shexp_gated = np.zeros((T, H), np.float32)
            a.shexp_gated = _ptr(res.shexp_gated)
        for k, v in keep.items():
            setattr(a, k, _ptr(v))
        for k in ("logits", "probs", "ids", "weights", "hidden", "down_out", "moe_out", "out"):
            setattr(a, k, _ptr(getattr(res, k)))
        a.ms_best = C.cast(C.pointer(best), C.c_void_p)
        a.ms_median = C.cast(C.pointer(med), C.c_void_p)
        if backend is not None:
            rc = self.lib.ref_moe_layer_backend(C.byref(a), backend, int(use_gallocr))
        else:
            rc = getattr(self.lib, self.prefix + "moe_layer")(C.byref(a))
        if rc:
            raise RuntimeError(f"{self.prefix}moe_layer failed with {rc}")
        res.ms_best, res.ms_median = best.value, med.value
        return res


class Restatement(_Checker):
    prefix = "orc_"
    kind = "port"

    def __init__(self):
        if not os.path.exists(RESTATEMENT_SO):
            build("restatement")
        super().__init__(RESTATEMENT_SO)
        for name, res, args in (
            ("orc_expf", C.c_float, [C.c_float]), ("orc_silu", C.c_float, [C.c_float]),
            ("orc_fp16_to_fp32", C.c_float, [C.c_uint16]), ("orc_fp32_to_fp16", C.c_uint16, [C.c_float]),
            ("orc_ue4m3_to_fp32", C.c_float, [C.c_uint8]), ("orc_fp32_to_ue4m3", C.c_uint8, [C.c_float]),
        ):
            f = getattr(self.lib, name)
            f.restype, f.argtypes = res, args


class Reference(_Checker):
    prefix = "ref_"
    kind = "reference"

    def __init__(self):
        # RTLD_GLOBAL: a ggml backend library under test resolves its ggml symbols against this build of ggml
        super().__init__(REFERENCE_SO, mode=C.RTLD_GLOBAL)
        self.lib.ref_isa.restype = C.c_char_p
        self.lib.ref_moe_layer_backend.argtypes = [C.POINTER(MoeArgs), C.c_void_p, C.c_int]
        self.lib.ref_moe_layer_backend.restype = C.c_int
        self.lib.ref_mul_mat_id_backend.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                                    C.c_int64, C.c_int64, C.c_void_p, C.c_int]
        self.lib.ref_mul_mat_id_backend.restype = C.c_int
        self.lib.ref_write_moe_gguf.argtypes = [C.c_char_p, C.POINTER(MoeArgs), C.c_int]
        self.lib.ref_write_moe_gguf.restype = C.c_int
        self.lib.ref_backend_confirm.argtypes = [C.c_void_p]
        self.lib.ref_backend_confirm.restype = C.c_int
        self.lib.ref_backend_free.argtypes = [C.c_void_p]
        self.lib.ref_backend_free.restype = None

    def isa(self) -> str:
        return self.lib.ref_isa().decode()

    def mul_mat_id_backend(self, backend, wtype, experts, x, ids, n_threads=1):
        """One MUL_MAT_ID node on `backend` (None: the reference's CPU backend).  experts [n_as][ne01][row bytes] uint8,
        x [T][n_ids][ne00] F32 (every slot its own row), ids [T][n_ids] int32.  Returns (status 0/4, dst [T][n_ids][ne01])."""
        experts = np.ascontiguousarray(experts)
        x = np.ascontiguousarray(x, dtype=np.float32)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        T, n_ids, ne00 = x.shape
        n_as, ne01 = experts.shape[0], experts.shape[1]
        dst = np.zeros((T, n_ids, ne01), dtype=np.float32)
        rc = self.lib.ref_mul_mat_id_backend(backend, int(wtype), experts.ctypes.data, ne00, ne01, n_as, x.ctypes.data, ids.ctypes.data,
                                             n_ids, T, dst.ctypes.data, n_threads)
        return rc, dst

    def write_moe_gguf(self, path, *, layer, wtype, router_w, gate, up, down, top_k, sh_gate=None, sh_up=None, sh_down=None, sh_gate_inp=None):
        """One MoE block written as a GGUF file by the reference's own gguf writer (test input for the product's GGUF reader)."""
        f32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)
        u8 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.uint8)
        keep = dict(router_w=f32(router_w), gate=u8(gate), up=u8(up), down=u8(down), sh_gate=u8(sh_gate), sh_up=u8(sh_up), sh_down=u8(sh_down),
                    sh_gate_inp=f32(sh_gate_inp))
        E, H = keep["router_w"].shape
        a = MoeArgs(H=H, L=H, E=E, K=top_k, I=gate.shape[1], T=0, wtype=wtype, n_threads=1, repeats=0, latent=0)
        if sh_gate is not None:
            a.I_sh = keep["sh_gate"].shape[0]
        for k, v in keep.items():
            setattr(a, k, _ptr(v))
        rc = self.lib.ref_write_moe_gguf(str(path).encode(), C.byref(a), int(layer))
        if rc:
            raise RuntimeError(f"ref_write_moe_gguf failed with {rc}")

    def backend_confirm(self, backend) -> int:
        """Synchronize, then compute an empty graph on `backend`: 0 when everything before it completed, else 4."""
        return self.lib.ref_backend_confirm(backend)


_cache = {}


def restatement() -> Restatement:
    if "o" not in _cache:
        _cache["o"] = Restatement()
    return _cache["o"]


def have_reference() -> bool:
    return os.path.exists(REFERENCE_SO)


def reference() -> Reference:
    if "r" not in _cache:
        _cache["r"] = Reference()
    return _cache["r"]


def best_checker():
    """The compiled reference where it exists, else the restatement."""
    return reference() if have_reference() else restatement()
