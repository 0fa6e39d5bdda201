"""ctypes binding of libedge0_b200.so (the C ABI declared in include/edge0_b200_moe.h).

The library is the product; this module only loads it and declares the signatures.  It raises when the
library has not been built - there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

ROOT = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(ROOT, "lib", "libedge0_b200.so")

TYPE_F32, TYPE_Q3_K, TYPE_BF16, TYPE_NVFP4 = 0, 11, 30, 40
OK = 0
NOALLOC_MAX_LOGITS = 32768  # B200MOE_NOALLOC_MAX_LOGITS
STATUS = {0: "OK", 1: "INVALID_ARG", 2: "UNSUPPORTED", 3: "ALLOC", 4: "CUDA", 5: "DEVICE_CHECK", 6: "NO_DEVICE"}


class Layer(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_embd", "n_latent", "n_expert", "n_expert_used", "n_ff", "wtype")] + [
        (n, C.c_void_p) for n in ("router_w", "router_bias", "gate", "up", "down", "gate_scale", "up_scale", "down_scale",
                                  "lat_down", "lat_up", "lat_down_scale", "lat_up_scale", "gate_shexp", "up_shexp", "down_shexp",
                                  "gate_inp_shexp")] + [
        ("n_ff_shexp", C.c_int32), ("reserved_", C.c_int32)]


class Observe(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("ffn_moe_logits", "ffn_moe_probs", "ffn_moe_topk", "ffn_moe_weights_norm",
                                          "ffn_moe_hidden", "ffn_moe_down", "ffn_shexp_gated")]


class Tensor(C.Structure):
    """b200moe_tensor: data pointer, ne[4] elements, nb[4] byte strides (ggml's description of a tensor)."""
    _fields_ = [("data", C.c_void_p), ("ne", C.c_int64 * 4), ("nb", C.c_int64 * 4)]


class Counters(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("tokens", "experts_touched", "weight_bytes", "kernel_launches", "fixup_overflow")]


# name -> (restype, argtypes); every symbol include/edge0_b200_moe.h declares
SIGNATURES = {
    "b200moe_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "b200moe_destroy": (None, [C.c_void_p]),
    "b200moe_reserve": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_int32]),
    "b200moe_last_error": (C.c_char_p, [C.c_void_p]),
    "b200moe_status_string": (C.c_char_p, [C.c_int]),
    "b200moe_device_memory": (C.c_int, [C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "b200moe_get_counters": (C.c_int, [C.c_void_p, C.POINTER(Counters)]),
    "b200moe_synchronize": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b200moe_set_expert_path": (C.c_int, [C.c_void_p, C.c_int]),
    "b200moe_set_launch_overlap": (C.c_int, [C.c_void_p, C.c_int]),
    "b200moe_enable_kernel_timing": (C.c_int, [C.c_void_p, C.c_int]),
    "b200moe_kernel_times": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_double)]),
    "b200moe_row_size": (C.c_int64, [C.c_int, C.c_int64]),
    "b200moe_mul_mat_id_width_ok": (C.c_int, [C.c_int, C.c_int64]),
    "b200moe_quantize_nvfp4_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]),
    "b200moe_dequantize_host": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]),
    "b200moe_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p), C.c_char_p, C.c_size_t]),
    "b200moe_gguf_close": (None, [C.c_void_p]),
    "b200moe_gguf_n_tensors": (C.c_int64, [C.c_void_p]),
    "b200moe_gguf_tensor": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int32), C.POINTER(C.c_int64 * 4), C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]),
    "b200moe_gguf_metadata_u64": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]),
    "b200moe_gguf_moe_layer": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(Layer), C.c_char_p, C.c_size_t]),
    "b200moe_expert_blob_bytes_nvfp4": (C.c_int64, [C.c_int32, C.c_int32]),
    "b200moe_unpack_expert_blobs_nvfp4": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "b200moe_route": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_void_p, C.c_int, C.c_int32, C.c_void_p, C.c_void_p,
                                C.POINTER(Observe), C.c_void_p]),
    "b200moe_mul_mat_id": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int64,
                                     C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200moe_mul_mat": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_latent_down": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_void_p, C.c_int, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200moe_latent_up": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "b200moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "b200moe_gather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "b200moe_ep_slot_bytes": (C.c_int64, [C.c_int64]),
    "b200moe_ep_pack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_ep_expert_rows": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200moe_ep_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                     C.c_void_p, C.c_void_p]),
    "b200moe_ffn": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_void_p, C.c_int, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                              C.POINTER(Observe), C.c_void_p]),
    "b200moe_layer_forward": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_void_p, C.c_int, C.c_int32, C.c_void_p,
                                        C.POINTER(Observe), C.c_void_p]),
    "b200moe_op_binary": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]),
    "b200moe_op_unary": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Tensor), C.POINTER(Tensor), C.c_float, C.c_float, C.c_void_p]),
    "b200moe_op_repeat": (C.c_int, [C.c_void_p, C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]),
    "b200moe_op_get_rows": (C.c_int, [C.c_void_p, C.POINTER(Tensor), C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]),
    "b200moe_op_sum_rows": (C.c_int, [C.c_void_p, C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]),
    "b200moe_op_soft_max": (C.c_int, [C.c_void_p, C.POINTER(Tensor), C.POINTER(Tensor), C.c_float, C.c_void_p]),
    "b200moe_op_argsort_desc": (C.c_int, [C.c_void_p, C.POINTER(Tensor), C.POINTER(Tensor), C.c_void_p]),
    "b200moe_op_mul_mat_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200moe_probe_fp4_tile": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200moe_probe_fp4_rate": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double)]),
    "b200moe_route_noalloc": (C.c_int, [C.c_int, C.POINTER(Layer), C.c_void_p, C.c_int, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_char_p, C.c_size_t]),
    "b200moe_layer_forward_host": (C.c_int, [C.c_void_p, C.POINTER(Layer), C.c_void_p, C.c_int, C.c_int32, C.c_void_p,
                                             C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the built library; raises if it is missing (build it with `python -m edge0_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m edge0_b200.build` (needs nvcc). "
                               "There is no CPU or PyTorch fallback for this path.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(lib, name)
            f.restype, f.argtypes = res, args
        _lib = lib
    return _lib


class B200MoeError(RuntimeError):
    def __init__(self, status: int, detail: str):
        super().__init__(f"b200moe status {status} ({STATUS.get(status, '?')}): {detail}")
        self.status = status
