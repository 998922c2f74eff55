"""No-GPU checks of the boundary: the C-ABI library loads and exports every symbol include/b200moe.h declares,
the op library registers the reference's op names with the reference's schemas, host-side argument checks run
before any launch, and the workspace size function behaves."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def m():
    import torch_tpu_b200
    if not os.path.exists(torch_tpu_b200.lib.LIB_PATH) or not os.path.exists(torch_tpu_b200.OPS_LIB_PATH):
        from importlib import import_module
        import_module("torch_tpu_b200.build").build_all()
    return torch_tpu_b200


def test_every_declared_symbol_is_exported(m):
    header = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    declared = set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    l = m.lib.lib()
    for name in sorted(declared):
        assert hasattr(l, name), f"{name} declared in include/b200moe.h but not exported"
    assert declared == set(m.lib.SIGNATURES), "ctypes binding and header disagree"
    assert l.b200moe_abi_version() == m.lib.ABI_VERSION == 3
    assert b"workspace" in l.b200moe_error_string(-3)


def test_host_side_rejections_need_no_gpu(m):
    l = m.lib.lib()
    null = ctypes.c_void_p(0)
    assert l.b200moe_topk(null, null, null, 0, 1, 8, 2, null) == m.lib.EINVAL
    one = ctypes.c_void_p(16)
    assert l.b200moe_topk(one, one, one, 0, 1, 2048, 2, null) == m.lib.ESHAPE
    assert l.b200moe_noaux_tc_topk(one, one, one, 0, 1, 256, 7, 4, 8, null) == m.lib.ESHAPE
    assert l.b200moe_quant_rows(one, one, 128, one, null, 1, 4, 100, null) == m.lib.ESHAPE
    assert l.b200moe_combine(one, one, one, 0, null, 4, 2, 12, null) == m.lib.ESHAPE
    assert l.b200moe_combine(ctypes.c_void_p(8), one, one, 0, null, 4, 2, 16, null) == m.lib.EALIGN
    # dense linear layer: K must be a multiple of 128, N of 64; an empty batch is fine without any pointer
    assert l.b200moe_linear_w8(one, one, one, one, 0, 4, 100, 128, one, 1 << 20, null, null) == m.lib.ESHAPE
    assert l.b200moe_linear_w8(one, one, one, one, 0, 4, 128, 100, one, 1 << 20, null, null) == m.lib.ESHAPE
    assert l.b200moe_linear_w8(null, null, null, null, 0, 0, 128, 128, null, 0, null, null) == m.lib.OK
    assert l.b200moe_linear_w8(null, one, one, one, 0, 4, 128, 128, one, 1 << 20, null, null) == m.lib.EINVAL
    assert l.b200moe_linear_workspace_bytes(4, 100, 128, 0) == 0
    assert l.b200moe_linear_workspace_bytes(32, 7168, 576, 1) >= 128 * 7168 + 56 * 128 * 4 + 5 * 56 * 4
    # peer-memory expert parallelism: at most 8 ranks, the rank inside the group, experts divisible by ranks
    assert l.b200moe_ep_plan(one, one, one, 256, 9, 0, null) == m.lib.EINVAL
    assert l.b200moe_ep_plan(one, one, one, 256, 8, 8, null) == m.lib.EINVAL
    assert l.b200moe_ep_plan(one, one, one, 250, 8, 0, null) == m.lib.ESHAPE
    assert l.b200moe_p2p_barrier(null, 2, 0, 1, null, null, null) == m.lib.EINVAL
    assert l.b200moe_ep_dispatch(one, one, one, one, one, one, one, one, 4, 2, 100, 8, 2, 0, 64, null, null) == m.lib.ESHAPE
    assert l.b200moe_ep_transpose_scales(one, 64, one, one, 256, 128, null) == m.lib.EINVAL   # ld < capacity


def test_workspace_bytes(m):
    ops = m.ops
    d = ops.make_desc(4096, 4096, 14336, 8, 2, out_mode=m.lib.OUT_COMBINED)
    n = ops.experts_workspace_bytes(d)
    P = 8192
    assert n >= P * 4096 + P * 14336 + P * 4096 * 2
    assert n < 2 * (P * 4096 + P * 14336 + P * 4096 * 2)
    assert ops.experts_workspace_bytes(ops.make_desc(4, 100, 128, 4, 2)) == 0       # H % 128 != 0
    d2 = ops.make_desc(16, 7168, 2048, 256, 8, I_shared=2048, out_mode=m.lib.OUT_COMBINED)
    assert ops.experts_workspace_bytes(d2) > ops.experts_workspace_bytes(
        ops.make_desc(16, 7168, 2048, 256, 8, out_mode=m.lib.OUT_COMBINED))


def test_workspace_bytes_never_shrink_with_tokens(m):
    """A layer sizes its workspace once for max_tokens and then runs any smaller batch in it."""
    ops = m.ops
    for kw in (dict(H=512, I=256, E=64, k=6, I_shared=256), dict(H=4096, I=14336, E=8, k=2)):
        prev = 0
        for T in (1, 2, 63, 64, 80, 85, 86, 128, 255, 256, 257, 600, 4096):
            d = ops.make_desc(T, kw["H"], kw["I"], kw["E"], kw["k"], I_shared=kw.get("I_shared", 0),
                              out_mode=m.lib.OUT_COMBINED)
            n = ops.experts_workspace_bytes(d)
            assert n >= prev, (kw, T, n, prev)
            prev = n


def test_op_surface_matches_reference_names_and_schemas(m):
    m.load_ops()
    want = {
        "fused_moe_fused_experts": 25, "fused_moe_fused_experts_v2": 27, "fused_moe_grouped_topk": 10,
        "noaux_tc_topk": 6, "mlp_w8a16_dq_forward": 9, "mlp_w8a8_quant_forward": 9,
        "mm_w8a16_dq_forward": 5, "enable_profile": 2, "disable_profile": 0}
    for name, nargs in want.items():
        op = getattr(torch.ops.my_ops, name)
        schema = op.default._schema
        assert len(schema.arguments) == nargs, (name, str(schema))
    s = str(torch.ops.my_ops.fused_moe_fused_experts.default._schema)
    # Tensor output, input, Tensor? x2, 3 weights, 3 optional scales, ids, weights, 3 optionals, 3 ints, bool, 2 ints,
    # 3 optionals, bool (torch_tpu/csrc/ops/my_ops/fusedMoE.cpp:117-130)
    assert s.count("Tensor?") == 11 and s.count("int ") == 5 and s.count("bool ") == 2, s
    with pytest.raises(RuntimeError, match="CUDA"):
        torch.ops.my_ops.noaux_tc_topk(torch.zeros(1, 8), torch.zeros(1, 8, dtype=torch.int32), torch.zeros(1, 256), 8, 4, 8)
