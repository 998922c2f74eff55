"""Routing kernels vs the oracle and the reference-generated golden vectors: indices bit-exact, values exact
copies (top-k) or within rtol 1e-5 / atol 1e-6 (normalised weights) - the tolerances of the reference's own tests
(python/regression/test_llm/test_noaux_tc_topk.py:141-154, test_topk.py:30-36)."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import bf16_from_bits, load

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    import torch_tpu_b200
    return torch_tpu_b200.ops


def test_noaux_tc_topk_reference_case(ops):
    z = load("noaux_topk.npz")
    scores = bf16_from_bits(z["ref_scores_bf16"])
    for B in (1, 8, 16, 64, 128):  # test_noaux_tc_topk.py:191-199
        v, i = ops.noaux_tc_topk(scores.repeat(B, 1).to(DEV), 8, 4, 8)
        assert torch.equal(i.cpu().long(), torch.from_numpy(z["ref_indices"]).repeat(B, 1))
        assert torch.equal(v.cpu().view(torch.int16), bf16_from_bits(z["ref_values_bf16"]).repeat(B, 1).view(torch.int16))


@pytest.mark.parametrize("key,groups,keep,k", [("f32", 8, 4, 8), ("bf16", 8, 4, 8), ("g4", 4, 2, 6)])
def test_noaux_tc_topk_golden(ops, key, groups, keep, k):
    z = load("noaux_topk.npz")
    sc = z[f"{key}_scores"]
    scores = bf16_from_bits(sc) if sc.dtype == np.uint16 else torch.from_numpy(sc.copy())
    v, i = ops.noaux_tc_topk(scores.to(DEV), groups, keep, k)
    assert torch.equal(i.cpu().long(), torch.from_numpy(z[f"{key}_indices"]))
    want = z[f"{key}_values"]
    want = bf16_from_bits(want) if want.dtype == np.uint16 else torch.from_numpy(want.copy())
    assert torch.equal(v.cpu().float(), want.float())


def test_plain_topk_golden(ops):
    z = load("topk.npz")
    v, i = ops.topk(bf16_from_bits(z["x_bf16"]).to(DEV), 8)
    assert torch.equal(i.cpu().float(), torch.from_numpy(z["indices"]))
    assert torch.equal(v.cpu().float(), torch.from_numpy(z["values"]))
    v, i = ops.topk(torch.from_numpy(z["x2"].copy()).to(DEV), 8)
    assert torch.equal(i.cpu().float(), torch.from_numpy(z["indices2"]))


@pytest.mark.parametrize("B,E,G,KG,k,dtype", [
    (1, 256, 8, 4, 8, torch.float32), (257, 256, 8, 4, 8, torch.float32), (33, 128, 1, 1, 8, torch.float32),
    (64, 8, 1, 1, 2, torch.float32), (19, 64, 4, 2, 6, torch.bfloat16), (5, 384, 8, 3, 8, torch.float16),
    (7, 1024, 16, 4, 32, torch.float32), (3, 24, 3, 2, 5, torch.float32)])
def test_grouped_topk_vs_oracle_with_ties(ops, B, E, G, KG, k, dtype):
    """Random scores INCLUDING ties (low-precision dtypes tie often): the lowest-index rule must match the oracle."""
    g = torch.Generator().manual_seed(B * 1000 + E)
    scores = (torch.randn(B, E, generator=g) * 2).to(dtype)
    if G > 1:
        wv, wi = O.noaux_tc_topk(scores, G, KG, k)
        v, i = ops.noaux_tc_topk(scores.to(DEV), G, KG, k)
    else:
        wv, wi = O.topk_lowest_index(scores, k)
        v, i = ops.topk(scores.to(DEV), k)
    assert torch.equal(i.cpu().long(), wi)
    assert torch.equal(v.cpu().float(), wv.float())


@pytest.mark.parametrize("T,H,E,k,mode", [
    (1, 512, 8, 2, "softmax"), (16, 1024, 8, 2, "softmax"), (300, 256, 128, 8, "softmax"),
    (300, 512, 8, 2, "softmax"), (100, 1280, 16, 4, "softmax"), (70, 4096, 5, 2, "softmax"),
    (3000, 512, 8, 2, "softmax"), (2500, 256, 12, 3, "softmax"),
    (1, 512, 256, 8, "deepseek"), (64, 512, 256, 8, "deepseek"), (1000, 256, 256, 8, "deepseek"),
    (40, 256, 64, 6, "sigmoid_nogroup")])
def test_route_chain(ops, T, H, E, k, mode):
    """Router GEMM on the device, then the routing chain on the device vs the oracle ON THE DEVICE'S LOGITS:
    ids bit-exact (inputs asserted tie-free at the top-k boundary), weights to 1e-5."""
    x, wr, logits_cpu = O.make_inputs(T, H, E, seed=T + E, router_std=0.2)
    logits = ops.router_logits(x.to(DEV), wr.to(DEV))
    torch.testing.assert_close(logits.cpu(), logits_cpu, rtol=1e-4, atol=1e-4)
    lg = logits.cpu()
    if mode == "softmax":
        ok = O.tie_free_rows(torch.softmax(lg, -1), k)
        wid, ww = O.route_softmax_topk(lg, k)
        ids, w = ops.route(logits, k, "softmax")
    elif mode == "deepseek":
        bias = torch.randn(E, generator=torch.Generator().manual_seed(5)) * 0.01
        ok = O.tie_free_rows(torch.sigmoid(lg) + bias, k, 8, 4)
        wid, ww = O.route_sigmoid_grouped(lg, bias, 8, 4, k, 2.5)
        ids, w = ops.route(logits, k, "sigmoid", bias.to(DEV), 8, 4, True, 2.5)
    else:
        ok = O.tie_free_rows(torch.sigmoid(lg), k)
        wid, ww = O.route_sigmoid_grouped(lg, None, 1, 1, k, 1.0)
        ids, w = ops.route(logits, k, "sigmoid")
    # rows whose top-k boundary is closer than 1e-6 relative are not decidable across exp implementations
    assert ok.float().mean() > 0.97
    assert torch.equal(ids.cpu()[ok], wid[ok])
    torch.testing.assert_close(w.cpu()[ok], ww[ok], rtol=1e-5, atol=1e-6)


def test_invalid_arguments_are_rejected(ops):
    s = torch.zeros(2, 256, device=DEV)
    with pytest.raises(RuntimeError):
        ops.noaux_tc_topk(s, 7, 4, 8)       # 256 % 7 != 0
    with pytest.raises(RuntimeError):
        ops.topk(torch.zeros(2, 2048, device=DEV), 8)  # n > 1024
    with pytest.raises(RuntimeError):
        ops.topk(s, 64)                      # k > 32


@pytest.mark.parametrize("H,E,k,mode", [(4096, 8, 2, "softmax"), (7168, 256, 8, "deepseek"), (2048, 128, 8, "softmax")])
def test_router_kernels_agree_across_batch_sizes_at_real_shapes(ops, H, E, k, mode):
    """The router has three kernels with three summation orders (T <= 16: one block per expert row; E <= 16: a block
    per 4 tokens; else the tensor-core GEMM), so the same token meets a different kernel in a different batch.
    Measured here at the benchmark's own hidden sizes, 2048 tokens routed as one batch and 16 at a time:
    - every kernel agrees with an fp64 product of the same bf16 operands: the CUDA-core kernels to 1e-5, the
      tensor-core GEMM (fp32 accumulation inside mma.sync) to 2e-5 of the largest logit;
    - a row whose selection gaps (between consecutive picks, at the top-k boundary and at the group boundary) are all
      wider than 1e-3 relative gets the same experts in the same order in either batch size, and rows that get another
      set of experts are below 2 % of the batch."""
    T_big = 2048
    x, wr, _ = O.make_inputs(T_big, H, E, seed=H + E, router_std=H ** -0.5)   # logits ~ N(0, 1)
    xd, wd = x.to(DEV), wr.to(DEV)
    big = ops.router_logits(xd, wd).cpu()
    small = torch.cat([ops.router_logits(xd[i:i + 16].contiguous(), wd).cpu() for i in range(0, T_big, 16)])
    one = torch.cat([ops.router_logits(xd[i:i + 1].contiguous(), wd).cpu() for i in range(4)])
    ref = x.double() @ wr.double().T
    scale = float(ref.abs().max())
    tc = E > 16                                           # the large batch goes through the tensor-core kernel
    assert float((big.double() - ref).abs().max()) <= (2e-5 if tc else 1e-6) * scale
    assert float((small.double() - ref).abs().max()) <= 1e-6 * scale
    assert float((one.double() - ref[:4]).abs().max()) <= 1e-6 * scale
    if mode == "softmax":
        wide = O.tie_free_rows(torch.softmax(ref.float(), -1), k, rel_gap=1e-3)
        route = lambda lg: ops.route(lg.to(DEV), k, "softmax")[0].cpu()
    else:
        bias = torch.randn(E, generator=torch.Generator().manual_seed(5)) * 0.01
        wide = O.tie_free_rows(torch.sigmoid(ref.float()) + bias, k, 8, 4, rel_gap=1e-3)
        route = lambda lg: ops.route(lg.to(DEV), k, "sigmoid", bias.to(DEV), 8, 4, True, 2.5)[0].cpu()
    ids_big, ids_small = route(big), route(small)
    differ = (ids_big != ids_small).any(-1)
    assert float(wide.float().mean()) > 0.2               # (8 ordered picks of 256 leave few rows with every gap wide)
    assert not bool((differ & wide).any())                # no row with decidable gaps routes differently
    other_set = (torch.sort(ids_big, -1)[0] != torch.sort(ids_small, -1)[0]).any(-1)
    assert float(other_set.float().mean()) <= 0.02        # rows that get another SET of experts in the other batch size
