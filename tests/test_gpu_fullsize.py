"""Parity at the benchmark's own sizes (Mixtral-8x7B shape, 4096 tokens; DeepSeek-V3 shape, 2048 tokens with the
shared expert).  The CPU oracle cannot redo a whole step at these sizes, so:

  - routing ids and the permutation are checked exactly for ALL tokens (they are cheap on the CPU);
  - size-independent properties are checked on the whole output: the step is bit-reproducible, and the combined
    output equals the weighted sum of the per-slot outputs;
  - the expert arithmetic is checked against the oracle on a fixed seeded subsample of tokens (256 for Mixtral,
    32 for DeepSeek, whose 256 experts make every sampled token pull new weights to the host), with only the
    activated experts' weights copied to the host.
"""
import os
import sys

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


def _layer(workload, T):
    sys.path.insert(0, ROOT)
    import bench
    wl = bench.WORKLOADS[workload]
    layer = bench.build_layer(wl, T, DEV, seed=0)
    x = bench.make_x(T, wl["H"], DEV, seed=100).to(DEV)
    return bench, wl, layer, x


@pytest.mark.parametrize("workload,T,n_sample", [("mixtral", 4096, 256), ("deepseek", 2048, 32)])
def test_full_size_step(workload, T, n_sample):
    import torch_tpu_b200  # noqa: F401
    from torch_tpu_b200 import ops
    bench, wl, layer, x = _layer(workload, T)
    E, k, H = wl["E"], wl["k"], wl["H"]
    y = layer.forward(x).clone()
    torch.cuda.synchronize()
    assert int(layer.status.item()) == 0
    ids, w = layer.ids[:T].clone(), layer.topk_w[:T].clone()
    logits = layer.logits[:T].cpu()

    # ---- routing, all tokens: exact on the device's own logits --------------------------------------------------
    if wl["score"] == "softmax":
        ok = O.tie_free_rows(torch.softmax(logits, -1), k)
        wid, ww = O.route_softmax_topk(logits, k)
    else:
        bias = layer.bias.cpu()
        ok = O.tie_free_rows(torch.sigmoid(logits) + bias, k, wl["groups"], wl["topk_groups"])
        wid, ww = O.route_sigmoid_grouped(logits, bias, wl["groups"], wl["topk_groups"], k, wl["scale"])
    assert ok.float().mean() > 0.97
    assert torch.equal(ids.cpu()[ok], wid[ok])
    torch.testing.assert_close(w.cpu()[ok], ww[ok], rtol=1e-5, atol=1e-6)

    # ---- permutation, all pairs: a stable sort by expert --------------------------------------------------------
    sorted_pair, offsets = ops.permute(ids, E)
    sp, off = sorted_pair.cpu().long(), offsets.cpu().long()
    flat = ids.cpu().long().reshape(-1)
    assert torch.equal(torch.sort(sp).values, torch.arange(T * k))                 # a permutation
    assert torch.equal(off[1:] - off[:-1], torch.bincount(flat, minlength=E))      # expert_offsets = counts
    e_sorted = flat[sp]
    assert bool((e_sorted[1:] >= e_sorted[:-1]).all())                             # grouped by expert
    same = e_sorted[1:] == e_sorted[:-1]
    assert bool((sp[1:][same] > sp[:-1][same]).all())                              # stable inside an expert

    # ---- properties of the whole output -------------------------------------------------------------------------
    y2 = layer.forward(x)
    torch.cuda.synchronize()
    assert torch.equal(y2, y)                                                      # bit-reproducible
    if layer.shared is None:
        wg, wu, wd, sg, su, sd = layer.w
        per_slot = torch.empty(T, k, H, dtype=torch.bfloat16, device=DEV)
        ops.experts(per_slot, x, wg, wu, wd, sg, su, sd, ids)
        comb = (per_slot.float() * w.float()[..., None]).sum(1)
        met = O.parity_metrics(y, comb)
        assert met["max_rel"] <= 4e-3 and met["cosine"] >= 0.99999, met           # one bf16 rounding apart

    # ---- expert arithmetic on a seeded subsample ----------------------------------------------------------------
    g = torch.Generator().manual_seed(7)
    idx = torch.randperm(T, generator=g)[:n_sample].sort().values
    xs, ids_s, w_s = x[idx.to(DEV)].cpu(), ids.cpu()[idx], w.cpu()[idx]
    used = torch.unique(ids_s.long())
    wts = [t[used.to(DEV)].cpu() for t in layer.w]                                 # only these experts travel
    remap = torch.full((E,), -1, dtype=torch.long)
    remap[used] = torch.arange(len(used))
    shared = tuple(t[0].cpu() for t in layer.shared) if layer.shared is not None else None
    want = O.moe_layer_w8a8(xs, remap[ids_s.long()].to(torch.int32), tuple(wts), shared=shared, topk_w=w_s)
    met = O.parity_metrics(y[idx.to(DEV)].cpu(), want)
    assert met["max_rel"] <= 2e-2 and met["cosine"] >= 0.9995, met
