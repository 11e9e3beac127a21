"""ctypes binding of libek_b200.so -- one declaration per entry point of include/ek_b200.h.

The shared library is the product; there is no Python or CPU implementation behind these
names.  Loading fails loudly when the library has not been built."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("EK_B200_LIB") or os.path.join(os.path.dirname(_HERE), "lib", "libek_b200.so")

EK_OK = 0
STATUS_NAMES = {
    0: "EK_OK", 1: "EK_EXPERT_NOT_FOUND", 2: "EK_EXPERT_WEIGHT_NOT_FOUND", 3: "EK_INVALID_INPUT",
    4: "EK_SAFETENSOR", 5: "EK_NOT_FOUND", 16: "EK_CUDA", 17: "EK_TIMEOUT", 18: "EK_BOUNDS",
    19: "EK_NO_MEMORY", 20: "EK_UNSUPPORTED",
}
EK_BF16, EK_F32, EK_F8_E4M3, EK_I8, EK_I32, EK_F16, EK_U8, EK_I64 = range(8)
EK_SCORE_SOFTMAX, EK_SCORE_SIGMOID = 0, 1
EK_QUANT_BF16, EK_QUANT_FP8_BLOCK128, EK_QUANT_INT8_BLOCK128 = 0, 1, 2
EK_TILE_LAYOUT_VERSION = 5   # include/ek_b200.h
EK_EP_MAX_RANKS = 16


EK_IPC_HANDLE_BYTES = 64
EK_STAGE_COUNT = 5
STAGE_NAMES = ("route", "permute", "gateup", "down", "combine")


class TensorView(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * 4), ("data", C.c_void_p)]


class Config(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("intermediate", C.c_int32), ("n_experts", C.c_int32),
                ("top_k", C.c_int32), ("scoring", C.c_int32), ("n_group", C.c_int32),
                ("topk_group", C.c_int32), ("norm_topk_prob", C.c_int32), ("routed_scaling", C.c_float),
                ("n_shared_experts", C.c_int32), ("bf16_combine", C.c_int32), ("quant", C.c_int32),
                ("max_tokens", C.c_int32), ("max_layers", C.c_int32), ("device", C.c_int32),
                ("ep_rank", C.c_int32), ("ep_size", C.c_int32), ("replica_slots", C.c_int32),
                ("model_name", C.c_char * 64)]


class RouteDebug(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ids", C.c_void_p), ("weights", C.c_void_p),
                ("counts", C.c_void_p), ("offsets", C.c_void_p), ("perm", C.c_void_p)]


# name -> (restype, argtypes); mirrors include/ek_b200.h
SIGNATURES = {
    "ek_backend_create": (C.c_int32, [C.POINTER(Config), C.POINTER(C.c_void_p)]),
    "ek_backend_destroy": (None, [C.c_void_p]),
    "ek_create_error": (C.c_char_p, []),
    "ek_last_error": (C.c_char_p, [C.c_void_p]),
    "ek_status_name": (C.c_char_p, [C.c_int32]),
    "ek_expert_register": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(TensorView), C.c_int32]),
    "ek_expert_register_safetensors": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t]),
    "ek_expert_mark_loading": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int32)]),
    "ek_expert_evict": (C.c_int32, [C.c_void_p, C.c_char_p]),
    "ek_expert_has": (C.c_int32, [C.c_void_p, C.c_char_p]),
    "ek_expert_loaded": (C.c_int32, [C.c_void_p]),
    "ek_expert_loading": (C.c_int32, [C.c_void_p]),
    "ek_expert_keys": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "ek_router_register": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_expert_forward": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_moe_forward": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_moe_forward_fused": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.POINTER(RouteDebug)]),
    "ek_route_from_logits": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p]),
    "ek_combine": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "ek_w8a16_activate": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "ek_worker_forward_wire": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                           C.POINTER(C.c_size_t)]),
    "ek_expert_counts": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_last_routing": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "ek_stage_timing_enable": (C.c_int32, [C.c_void_p, C.c_int32]),
    "ek_stage_times": (C.c_int32, [C.c_void_p, C.POINTER(C.c_float)]),
    "ek_kernel_launches": (C.c_int64, [C.c_void_p]),
    "ek_ep_peer_alloc": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_ep_peer_open": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_ep_peer_close": (C.c_int32, [C.c_void_p]),
    "ek_ep_peer_push": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_uint32]),
    "ek_ep_peer_partial": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_uint32]),
    "ek_ep_peer_finish": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_uint32, C.c_void_p]),
    "ek_expert_export_tiles": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "ek_expert_register_tiles": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t]),
    "ek_worker_batch_stats": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "ek_debug_set_ffn_impl": (C.c_int32, [C.c_void_p, C.c_int32]),
    "ek_set_precise_dequant": (C.c_int32, [C.c_void_p, C.c_int32]),
    "ek_set_stream": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "ek_moe_forward_fused_async": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_sync": (C.c_int32, [C.c_void_p]),
    "ek_ep_route": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "ek_ep_ffn": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_ep_combine": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_ep_set_owners": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_ep_partial": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ek_ep_finish": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "ek_bucket_noalloc": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_char_p, C.c_size_t]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python expert-kit_b200/build.py` "
            "(this package has no CPU or pure-Python path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
