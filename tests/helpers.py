"""Shared helpers of the test-suite (bit-pattern fixtures <-> torch tensors)."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def f8_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)


def load(name: str):
    return np.load(os.path.join(GOLDEN, name))


def ref_moe_inputs(T, H, I, E, k, seed=1000):
    """Input statements of the reference's MoE test (python/regression/test_llm/test_moe.py:251-274),
    same order of RNG draws; used to regenerate the inputs whose outputs are stored in
    golden/moe_ref_shapes.npz."""
    import random
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


def moe_small_case(name: str):
    """One stored case of golden/moe_small.npz -> tensors in the op's device layout
    (down weight/scales transposed and contiguous, test_moe.py:285-288)."""
    z = load("moe_small.npz")
    x = bf16_from_bits(z[f"{name}_x"])
    ids = torch.from_numpy(z[f"{name}_ids"].copy())
    rw = bf16_from_bits(z[f"{name}_rw"])
    w0, w1, w2 = (f8_from_bits(z[f"{name}_w{i}"]) for i in range(3))
    s0, s1, s2 = (bf16_from_bits(z[f"{name}_s{i}"]) for i in range(3))
    out = bf16_from_bits(z[f"{name}_out"])
    wd = w2.transpose(1, 2).contiguous()
    sd = s2.transpose(1, 2).contiguous()
    return dict(x=x, ids=ids, rw=rw, wg=w0, wu=w1, wd=wd, sg=s0, su=s1, sd=sd, out=out)
