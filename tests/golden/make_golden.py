"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE'S OWN CPU CODE.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/torch-tpu

The reference's test modules ``import torch_tpu`` at the top, which needs vendor binaries; a stub
module that only provides ``torch_tpu.utils.compare`` (pure numpy/torch in the reference) makes
them importable.  Nothing else of the reference is touched.  The fixtures are ``.npz`` files of
raw bit patterns (bf16 as uint16, e4m3 as uint8) so that numpy can hold them.

What is recorded:
  noaux_topk.npz  - ``gt_noaux_tc_topk`` on the reference test's own inputs
                    (test_noaux_tc_topk.py:191-225: manual_seed(42), randperm(256) in bf16) and on
                    tie-free fp32 rows.
  topk.npz        - ``topk_cpu`` (test_topk.py:9-12) on randperm rows.
  moe_small.npz   - ``deepseek_moe_cpu`` (test_moe.py:162-166) on small stored inputs built the way
                    test_moe.py:255-274 builds them (bf16 default dtype, randn*0.1 weights, randn*0.1
                    bf16 scales that may be negative, distinct experts per token).
  moe_ref_shapes.npz - outputs of ``deepseek_moe_cpu`` on the reference's own parametrisation
                    (test_moe.py:218-227) with inputs regenerated from seed 1000 by
                    ``ref_moe_inputs`` below (the statements of test_moe.py:251-274).
  mlp_dense.npz   - ``mlp_w8a16_dq_cpu`` (test_mlp_w8a16_dq.py:53-85) on a small stored case.
  moe_bf16.npz    - ``QwenMoE`` (python/test/fused_moe_bf16.py:63-95: bf16 weights, no scales) on small stored inputs
                    built the way fused_moe_bf16.py:152-167 builds them (randn bf16 weights, distinct experts).
"""
import importlib.util
import os
import random
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def ref_moe_inputs(T, H, I, E, k, seed=1000):
    """The input statements of test_moe.py:251-274 (same order of RNG draws)."""
    torch.manual_seed(seed)
    random.seed(seed)
    sel = [random.sample(range(E), k) for _ in range(T)]
    ids = torch.tensor(sel, dtype=torch.int32).reshape(T, k)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        nI, nH = (I + 127) // 128, (H + 127) // 128
        rw = torch.randn(T, k, dtype=torch.bfloat16)
        w0 = torch.randn(E, I, H) * 0.1
        w1 = torch.randn(E, I, H) * 0.1
        w2 = torch.randn(E, H, I) * 0.1
        s0 = torch.randn(E, nI, nH) * 0.1
        s1 = torch.randn(E, nI, nH) * 0.1
        s2 = torch.randn(E, nH, nI) * 0.1
        w0 = w0.to(torch.float8_e4m3fn)
        w1 = w1.to(torch.float8_e4m3fn)
        w2 = w2.to(torch.float8_e4m3fn)
        x = torch.randn(T, H)
    finally:
        torch.set_default_dtype(old)
    return x, ids, rw, w0, w1, w2, s0, s1, s2


def main(ref_root: str) -> None:
    # stub torch_tpu: only utils.compare, loaded from the reference file itself
    tt = types.ModuleType("torch_tpu")
    tu = types.ModuleType("torch_tpu.utils")
    spec = importlib.util.spec_from_file_location(
        "torch_tpu.utils.compare", os.path.join(ref_root, "torch_tpu/utils/compare.py"))
    cmpm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cmpm)
    tt.utils, tu.compare = tu, cmpm
    sys.modules.update({"torch_tpu": tt, "torch_tpu.utils": tu, "torch_tpu.utils.compare": cmpm})
    sys.path.insert(0, os.path.join(ref_root, "python/regression/test_llm"))
    import test_moe as RM            # noqa: E402
    import test_noaux_tc_topk as RN  # noqa: E402
    import test_topk as RT           # noqa: E402
    import test_mlp_w8a16_dq as RD   # noqa: E402

    # ---- grouped top-k ------------------------------------------------------------------
    out = {}
    torch.manual_seed(42)
    scores = torch.stack([torch.randperm(256, dtype=torch.float32)]).reshape(1, -1).to(torch.bfloat16)
    v, i, _ = RN.gt_noaux_tc_topk(scores.clone(), 8, 4, 8)
    out["ref_scores_bf16"], out["ref_values_bf16"], out["ref_indices"] = _bits(scores), _bits(v), i.numpy()
    g = torch.Generator().manual_seed(7)
    sc32 = torch.rand(64, 256, generator=g)            # fp32, distinct with probability ~1
    v, i, _ = RN.gt_noaux_tc_topk(sc32.clone(), 8, 4, 8)
    out["f32_scores"], out["f32_values"], out["f32_indices"] = sc32.numpy(), v.numpy(), i.numpy()
    sc_b = torch.stack([torch.randperm(256, generator=g).float() for _ in range(64)]).to(torch.bfloat16)
    # bf16 group sums can tie, and the reference leaves tie order open (its own failing case is
    # parked at test_noaux_tc_topk.py:112-188): keep the rows whose group scores are all distinct
    gs = RN.gt_noaux_tc_topk(sc_b.clone(), 8, 4, 8)[2]["group_scores"].float()
    keep = torch.tensor([len(set(r.tolist())) == 8 for r in gs])
    sc_b = sc_b[keep][:32].contiguous()
    v, i, _ = RN.gt_noaux_tc_topk(sc_b.clone(), 8, 4, 8)
    out["bf16_scores"], out["bf16_values"], out["bf16_indices"] = _bits(sc_b), _bits(v), i.numpy()
    sc_c = torch.stack([torch.randperm(64, generator=g).float() for _ in range(48)])
    gs = RN.gt_noaux_tc_topk(sc_c.clone(), 4, 2, 6)[2]["group_scores"]
    sc_c = sc_c[torch.tensor([len(set(r.tolist())) == 4 for r in gs])][:16].contiguous()
    v, i, _ = RN.gt_noaux_tc_topk(sc_c.clone(), 4, 2, 6)
    out["g4_scores"], out["g4_values"], out["g4_indices"] = sc_c.numpy(), v.numpy(), i.numpy()
    np.savez_compressed(os.path.join(HERE, "noaux_topk.npz"), **out)

    # ---- plain top-k ---------------------------------------------------------------------
    g = torch.Generator().manual_seed(11)
    x = torch.stack([torch.randperm(256, generator=g).to(torch.bfloat16) for _ in range(16)])
    v, i = RT.topk_cpu(x, 8)
    x2 = torch.stack([torch.randperm(128, generator=g).float() for _ in range(8)])
    v2, i2 = RT.topk_cpu(x2, 8)
    np.savez_compressed(os.path.join(HERE, "topk.npz"), x_bf16=_bits(x), values=v.numpy(),
                        indices=i.numpy(), x2=x2.numpy(), values2=v2.numpy(), indices2=i2.numpy())

    # ---- fused experts, small stored inputs ----------------------------------------------
    cases = {}
    for name, (T, H, I, E, k) in {"a": (4, 256, 128, 4, 2), "b": (3, 384, 256, 5, 3)}.items():
        x, ids, rw, w0, w1, w2, s0, s1, s2 = ref_moe_inputs(T, H, I, E, k, seed=1000 + len(cases))
        torch.set_default_dtype(torch.bfloat16)
        try:
            o = torch.zeros(T, k, H)
            o = RM.deepseek_moe_cpu(x, ids, o, E, k, w0, w1, w2, s0, s1, s2, 128)
        finally:
            torch.set_default_dtype(torch.float32)
        for key, val in dict(x=x, ids=ids, rw=rw, w0=w0, w1=w1, w2=w2, s0=s0, s1=s1, s2=s2,
                             out=o).items():
            cases[f"{name}_{key}"] = _bits(val)
    np.savez_compressed(os.path.join(HERE, "moe_small.npz"), **cases)

    # ---- fused experts, the reference's own shapes (inputs regenerated from the seed) ------
    outs = {}
    for (T, H, I, E, k) in [(1, 7168, 256, 1, 1), (1, 7168, 256, 2, 2), (1, 7168, 256, 16, 8)]:
        x, ids, rw, w0, w1, w2, s0, s1, s2 = ref_moe_inputs(T, H, I, E, k, seed=1000)
        torch.set_default_dtype(torch.bfloat16)
        try:
            o = torch.zeros(T, k, H)
            o = RM.deepseek_moe_cpu(x, ids, o, E, k, w0, w1, w2, s0, s1, s2, 128)
        finally:
            torch.set_default_dtype(torch.float32)
        outs[f"out_{T}_{H}_{I}_{E}_{k}"] = _bits(o)
        outs[f"ids_{T}_{H}_{I}_{E}_{k}"] = ids.numpy()
        outs[f"xsum_{T}_{H}_{I}_{E}_{k}"] = np.float64(x.double().sum().item())
    np.savez_compressed(os.path.join(HERE, "moe_ref_shapes.npz"), **outs)

    # ---- dense FP8 gated MLP (the shared-expert op) ---------------------------------------
    torch.manual_seed(5)
    T, H, I = 5, 256, 384
    x = torch.randn(T, H).to(torch.bfloat16)
    wg = (torch.randn(I, H) * 0.1).to(torch.float8_e4m3fn)
    wu = (torch.randn(I, H) * 0.1).to(torch.float8_e4m3fn)
    wd = (torch.randn(H, I) * 0.1).to(torch.float8_e4m3fn)
    sg = (torch.randn(I // 128, H // 128) * 0.1).to(torch.bfloat16)
    su = (torch.randn(I // 128, H // 128) * 0.1).to(torch.bfloat16)
    sd = (torch.randn(H // 128, I // 128) * 0.1).to(torch.bfloat16)
    o = RD.mlp_w8a16_dq_cpu(x, wg, wu, wd, sg, su, sd, 128)
    np.savez_compressed(os.path.join(HERE, "mlp_dense.npz"), x=_bits(x), wg=_bits(wg), wu=_bits(wu),
                        wd=_bits(wd), sg=_bits(sg), su=_bits(su), sd=_bits(sd), out=o.numpy())
    # ---- bf16-weight experts ---------------------------------------------------------------
    sys.path.insert(0, os.path.join(ref_root, "python/test"))
    import fused_moe_bf16 as RB      # noqa: E402
    torch.manual_seed(11)
    random.seed(11)
    cases = {}
    for name, (T, H, I, E, k) in {"a": (6, 256, 128, 4, 2), "b": (3, 384, 128, 2, 2)}.items():
        ids = torch.tensor([random.sample(range(E), k) for _ in range(T)], dtype=torch.int32)
        w0 = torch.randn(E, I, H).to(torch.bfloat16)
        w1 = torch.randn(E, I, H).to(torch.bfloat16)
        w2 = torch.randn(E, H, I).to(torch.bfloat16)
        x = torch.randn(T, H).to(torch.bfloat16)
        o = RB.QwenMoE(E, k, w0, w1, w2)(x, ids)
        for key, t in (("x", x), ("w0", w0), ("w1", w1), ("w2", w2), ("out", o)):
            cases[f"{name}_{key}"] = _bits(t)
        cases[f"{name}_ids"] = ids.numpy()
    np.savez_compressed(os.path.join(HERE, "moe_bf16.npz"), **cases)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the torch-tpu checkout>")
    main(sys.argv[1])
