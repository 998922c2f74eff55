"""torch-tpu_b200: the FP8 fused-MoE inference hot path of sophgo/torch-tpu (routing, permutation, grouped
gate/up GEMM with SiLU-and-mul, down GEMM, weighted combine), written for NVIDIA B200 (sm_100a) and exposed
behind the reference's own ``torch.ops.my_ops.*`` custom-op surface.

  lib      ctypes binding of the C ABI (include/b200moe.h)
  ops      functional wrappers over the C ABI for torch CUDA tensors
  layer    FusedMoE: route -> experts -> combine as one call, plus the expert-parallel variant
  weights  checkpoint-layout -> op-layout conversion and FP8 block quantisation
  load_ops()  registers torch.ops.my_ops.{fused_moe_fused_experts, fused_moe_fused_experts_v2,
              fused_moe_grouped_topk, noaux_tc_topk, mlp_w8a16_dq_forward, mlp_w8a8_quant_forward}
"""
import os

from . import lib  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
OPS_LIB_PATH = os.path.join(_HERE, "libb200_moe_ops.so")
_ops_loaded = False


def load_ops():
    """Load the TORCH_LIBRARY(my_ops) extension.  Raises if it has not been built: there is no fallback."""
    global _ops_loaded
    if not _ops_loaded:
        import torch
        if not os.path.exists(OPS_LIB_PATH):
            raise RuntimeError(f"{OPS_LIB_PATH} is missing: build it with `python torch-tpu_b200/build.py`")
        lib.lib()  # libb200moe.so first, so that the extension's dependency resolves to the in-tree copy
        torch.ops.load_library(OPS_LIB_PATH)
        _ops_loaded = True


def __getattr__(name):
    if name in ("ops", "layer", "weights", "ep"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
