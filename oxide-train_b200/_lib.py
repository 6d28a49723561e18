"""ctypes binding of the C ABI in ``include/b200gemm.h``.

The library is the product; this module only loads it and declares the
signatures.  There is no fallback: if the shared library is missing, loading
raises, and on a machine without a B200 ``b200gemm_create`` fails.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# B200GEMM_LIB lets a developer point the binding at another build of the same library.
LIB_PATH = os.environ.get("B200GEMM_LIB") or os.path.join(HERE, "libb200gemm.so")

OK, ERR_INVALID, ERR_SHAPE, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE = range(6)
K_MAJOR, MN_MAJOR = 0, 1
OUT_F32, OUT_BF16 = 0, 1
STORE, ACCUMULATE = 0, 1
FLAG_CTA_GROUP_1, FLAG_CTA_GROUP_2, FLAG_WIDE_TILE, FLAG_NARROW_TILE = 0x1, 0x2, 0x4, 0x8
OP_NN, OP_NT, OP_TN = 0, 1, 2


class GemmDesc(C.Structure):
    """``b200gemm_desc_t``."""
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("a_layout", C.c_int32), ("b_layout", C.c_int32),
        ("out_type", C.c_int32), ("mode", C.c_int32),
        ("batch", C.c_int32), ("split_k", C.c_int32),
        ("batch_stride_a", C.c_int64), ("batch_stride_b", C.c_int64), ("batch_stride_c", C.c_int64),
        ("flags", C.c_uint32), ("reserved", C.c_uint32),
    ]


# name -> (restype, argtypes); every symbol include/b200gemm.h declares.
SIGNATURES = {
    "b200gemm_version": (C.c_int, []),
    "b200gemm_last_error_string": (C.c_char_p, []),
    "b200gemm_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "b200gemm_destroy": (C.c_int, [C.c_void_p]),
    "b200gemm_set_sm_limit": (C.c_int, [C.c_void_p, C.c_int32]),
    "b200gemm_set_exchange_ctas": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32]),
    "b200gemm_set_scheduler": (C.c_int, [C.c_void_p, C.c_int32]),
    "b200gemm_gemm_dual": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]),
    "b200gemm_gemm": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(GemmDesc)]),
    "b200gemm_gemm_host": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(GemmDesc)]),
    "b200gemm_launch_config": (C.c_int, [C.c_void_p, C.POINTER(GemmDesc)] + [C.POINTER(C.c_int32)] * 4),
    "b200gemm_sgemm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]),
    "b200gemm_convert_f32_to_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]),
    "b200gemm_convert_bf16_to_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]),
    "b200gemm_transpose_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]),
    "b200gemm_wait_selftest": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64]),
    "b200gemm_device_status": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
    "b200gemm_grouped_gemm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32,
                                        C.c_int64, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32,
                                        C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "b200gemm_moe_route": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                     C.c_int32, C.c_int64] + [C.c_void_p] * 7),
    "b200gemm_moe_ep_plan": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200gemm_moe_ep_push": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.POINTER(C.c_void_p), C.c_int64, C.c_int32, C.c_int32, C.c_int64,
                                       C.c_int32, C.c_int64]),
    "b200gemm_moe_ep_pull_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p,
                                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                               C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_int64,
                                               C.c_void_p, C.c_int32]),
    "b200gemm_moe_scatter": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                       C.c_int64, C.c_void_p]),
    "b200gemm_moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int64, C.c_int32, C.c_int64, C.c_void_p, C.c_int32]),
    "b200gemm_lmhead_ce_workspace_bytes": (C.c_size_t, [C.c_int64]),
    "b200gemm_lmhead_ce_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                             C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "b200gemm_lmhead_ce_forward_shard": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                                   C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "b200gemm_grouped_gemm_indexed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                                C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p,
                                                C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int64,
                                                C.c_int64, C.c_int64, C.c_int32]),
    "b200gemm_grouped_gemm_swiglu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                               C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p,
                                               C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                               C.c_int32, C.c_int64, C.c_int64, C.c_int64]),
    "b200gemm_grouped_gemm_silu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                             C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p,
                                             C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                             C.c_int32, C.c_int64, C.c_int64, C.c_int64]),
    "b200gemm_grouped_gemm_act_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                                     C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_void_p,
                                                     C.c_int32, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                                     C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64]),
    "b200gemm_grouped_wgrad": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                         C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32]),
    "b200gemm_moe_combine_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                                C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64,
                                                C.c_void_p, C.c_void_p]),
    "b200gemm_activation_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int64,
                                               C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                               C.c_int64]),
    "b200gemm_moe_route_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_int32,
                                              C.c_int32, C.c_void_p]),
    "b200gemm_router_logits": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                         C.c_int32, C.c_void_p]),
    "b200gemm_loss_mean_with_aux": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                              C.c_int32, C.c_float, C.c_void_p]),
    "b200gemm_lmhead_ce_merge_shards": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64,
                                                  C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200gemm_moe_ep_return_plan": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                              C.c_void_p, C.c_void_p]),
    "b200gemm_grouped_gemm_peer": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32,
                                             C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.POINTER(C.c_void_p),
                                             C.c_int32, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_int32, C.c_int64, C.c_int64, C.c_int64]),
    "b200gemm_peer_barrier": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32,
                                        C.c_uint64, C.c_int64, C.c_void_p, C.c_int32, C.POINTER(C.c_void_p)]),
    "b200gemm_sum_parts": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int64,
                                     C.c_void_p, C.c_int32, C.c_int32]),
    "b200gemm_lmhead_ce_forward_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                                     C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                                     C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200gemm_lmhead_ce_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                              C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_int64,
                                              C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_int32]),
}

_lib = None


def load() -> C.CDLL:
    """Load ``libb200gemm.so`` (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` "
                "(there is no fallback implementation)")
        lib = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


class B200GemmError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"b200gemm status {code}: {message}")
        self.code = code


def check(code: int) -> None:
    if code != OK:
        raise B200GemmError(code, load().b200gemm_last_error_string().decode())
