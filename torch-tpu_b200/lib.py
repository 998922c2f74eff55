"""ctypes binding of the C ABI declared in include/b200moe.h.

This is the only place the Python side touches the kernels; it passes raw device pointers and sizes.
There is no fallback: if ``libb200moe.so`` has not been built, importing the binding raises.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200moe.so")

ABI_VERSION = 3
OK, EINVAL, ESHAPE, EWORKSPACE, EALIGN, EDRIVER = 0, -1, -2, -3, -4, -5
F32, BF16, F16 = 0, 1, 2
SCORE_SOFTMAX, SCORE_SIGMOID = 0, 1
OUT_PER_SLOT, OUT_COMBINED, OUT_COMBINED_FUSED = 0, 1, 2
STAGE_PREP, STAGE_GATE_UP, STAGE_DOWN, STAGE_COMBINE, STAGE_ALL = 1, 2, 4, 8, 15
ACT_W8A8, ACT_W8A16 = 0, 1
IMPL_AUTO, IMPL_SIMPLE, IMPL_TCGEN05 = 0, 1, 2
STATUS_BAD_EXPERT, STATUS_WAIT_TIMEOUT, STATUS_PEER_TIMEOUT, STATUS_PEER_OVERFLOW = 1, 2, 4, 8


class ExpertsDesc(Structure):
    _fields_ = [("T", c_int64), ("H", c_int64), ("I", c_int64), ("E", c_int64), ("k", c_int64),
                ("I_shared", c_int64), ("out_mode", c_int), ("act_mode", c_int), ("impl", c_int),
                ("scale_dtype", c_int), ("w_dtype", c_int), ("impl_gate_up", c_int), ("impl_down", c_int),
                ("weights_bf16", c_int), ("stages", c_int), ("max_ctas", c_int)]


# name -> (restype, argtypes): every symbol include/b200moe.h declares
SIGNATURES = {
    "b200moe_abi_version": (c_int, []),
    "b200moe_error_string": (c_char_p, [c_int]),
    "b200moe_noaux_tc_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64,
                                      c_int64, c_void_p]),
    "b200moe_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "b200moe_router_logits": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "b200moe_route": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                              c_int64, c_int64, c_int, c_float, c_void_p]),
    "b200moe_permute_scratch_ints": (c_size_t, [c_int64, c_int64]),
    "b200moe_permute": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                c_void_p]),
    "b200moe_permute_static_max_scratch_ints": (c_size_t, []),
    "b200moe_permute_static": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "b200moe_gather_scatter_index": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                             c_int64, c_void_p]),
    "b200moe_quant_rows": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                   c_void_p]),
    "b200moe_experts_workspace_bytes": (c_size_t, [POINTER(ExpertsDesc)]),
    "b200moe_experts": (c_int, [c_void_p] * 16 + [POINTER(ExpertsDesc), c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200moe_combine": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64,
                                c_void_p]),
    "b200moe_combine_indexed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int64,
                                        c_int64, c_void_p]),
    "b200moe_combine_masked": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64,
                                       c_int64, c_int64, c_void_p]),
    "b200moe_grouped_mlp_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64, c_int64, c_int]),
    "b200moe_grouped_mlp": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p] + [c_void_p] * 6 +
                            [c_int, c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200moe_ep_packed_row_bytes": (c_int64, [c_int64]),
    "b200moe_ep_pack_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                     c_void_p]),
    "b200moe_ep_unpack_ids": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "b200moe_ep_unpack_rows": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "b200moe_invert_permutation": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "b200moe_linear_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int]),
    "b200moe_linear_w8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p,
                                  c_size_t, c_void_p, c_void_p]),
    "b200moe_scaled_mm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "b200moe_scaled_mm": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                  c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200moe_p2p_alloc": (c_int, [POINTER(c_void_p), c_size_t]),
    "b200moe_p2p_free": (c_int, [c_void_p]),
    "b200moe_p2p_export": (c_int, [c_char_p, c_void_p]),
    "b200moe_p2p_import": (c_int, [POINTER(c_void_p), c_char_p]),
    "b200moe_p2p_release": (c_int, [c_void_p]),
    "b200moe_p2p_barrier": (c_int, [c_void_p, c_int64, c_int64, c_uint32, c_void_p, c_void_p, c_void_p]),
    "b200moe_ep_exchange_counts": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_uint32, c_void_p,
                                           c_void_p, c_void_p]),
    "b200moe_ep_plan": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "b200moe_ep_dispatch": (c_int, [c_void_p] * 8 + [c_int64] * 7 + [c_void_p, c_void_p]),
    "b200moe_ep_transpose_scales": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "b200moe_grouped_mlp_remote": (c_int, [c_void_p] * 12 + [c_int, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                                             c_size_t, c_void_p, c_void_p]),
}

_lib = None


def lib():
    """The loaded library (loads on first use; raises if it is missing - there is no other path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python torch-tpu_b200/build.py` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these kernels.")
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        if l.b200moe_abi_version() != ABI_VERSION:
            raise RuntimeError("libb200moe.so ABI version mismatch; rebuild it")
        _lib = l
    return _lib


def error_string(code: int) -> str:
    return lib().b200moe_error_string(code).decode()


def check(code: int, what: str) -> None:
    if code != OK:
        raise RuntimeError(f"{what} failed: {error_string(code)} ({code})")
