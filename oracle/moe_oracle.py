"""CPU oracle for the FP8 fused-MoE hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package may import this module: it is the checker that
the parity tests, the smoke test and the CPU-baseline leg of the benchmark
compare the CUDA kernels against.  Everything here runs on CPU tensors with
plain torch ops.

Each function names the reference file (path inside sophgo/torch-tpu) whose
arithmetic it restates.  Two expert oracles exist because the reference op is
W8A16 (bf16 activations) while the CUDA path quantises activations to e4m3:

* ``experts_w8a16``  - "oracle-A": the reference CPU path
  (python/regression/test_llm/test_moe.py:10-98) with the same statement order
  and the same bf16 roundings.  Pinned against fixtures produced by the
  reference's own code (tests/golden/make_golden.py).
* ``experts_w8a8``   - "oracle-B": the same statements evaluated in fp32 with
  the activation quantise/dequantise steps (per token, per 128 columns, e4m3)
  inserted in front of the gate/up and the down projections.  This is the
  contract the FP8 tensor-core kernels are held to.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

BLOCK = 128
FP8_MAX = 448.0
AMAX_FLOOR = 1e-12  # floor of a group's max|x| before the scale is formed
F8 = torch.float8_e4m3fn


# --------------------------------------------------------------------------
# quantisation helpers
# --------------------------------------------------------------------------
def weight_dequant(w: torch.Tensor, s: torch.Tensor, block: int = BLOCK,
                   dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``y[r,c] = dtype(f32(w[r,c]) * s[r//block, c//block])``.

    Restates ``weight_dequant`` (python/regression/test_llm/test_moe.py:10-50):
    the product is formed in fp32 and rounded once into the result dtype (the
    reference allocates the result in torch's default dtype, bf16 in its test).
    """
    assert w.dim() == 2 and s.dim() == 2
    M, N = w.shape
    sf = s.to(torch.float32).repeat_interleave(block, 0)[:M].repeat_interleave(block, 1)[:, :N]
    return (w.to(torch.float32) * sf).to(dtype)


def quant_weight_128x128(w: torch.Tensor, block: int = BLOCK) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``[R,C]`` -> (e4m3 ``[R,C]``, fp32 scale ``[ceil(R/b), ceil(C/b)]``) with
    ``scale = amax(block)/448`` - the input-generation rule of the benchmark
    configurations (block amax / 448, fp32 scales)."""
    R, C = w.shape
    nr, nc = (R + block - 1) // block, (C + block - 1) // block
    wp = torch.zeros(nr * block, nc * block, dtype=torch.float32)
    wp[:R, :C] = w.to(torch.float32)
    blk = wp.view(nr, block, nc, block)
    amax = blk.abs().amax(dim=(1, 3)).clamp_min(AMAX_FLOOR)
    s = amax / FP8_MAX
    q = (blk / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(nr * block, nc * block)[:R, :C]
    return q.to(F8).contiguous(), s.contiguous()


def quant_act_1x128(x: torch.Tensor, block: int = BLOCK) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per row, per ``block`` columns: ``amax = max(max|x|, 1e-12)``, ``s = amax/448``,
    ``q = e4m3_rne(clamp(x * (448/amax), +-448))``.  fp32 arithmetic throughout; the
    CUDA kernels use the same two IEEE divisions and one multiply per element, so the
    bytes are expected to be identical."""
    x = x.to(torch.float32)
    R, C = x.shape
    assert C % block == 0
    g = x.view(R, C // block, block)
    amax = g.abs().amax(dim=-1).clamp_min(AMAX_FLOOR)
    inv = torch.tensor(FP8_MAX, dtype=torch.float32) / amax
    s = amax / torch.tensor(FP8_MAX, dtype=torch.float32)
    q = (g * inv[..., None]).clamp(-FP8_MAX, FP8_MAX).to(F8).view(R, C)
    return q.contiguous(), s.contiguous()


def dequant_act(q: torch.Tensor, s: torch.Tensor, block: int = BLOCK) -> torch.Tensor:
    R, C = q.shape
    return (q.to(torch.float32).view(R, C // block, block) * s[..., None]).view(R, C)


# --------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------
def topk_lowest_index(scores: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Descending top-k along the last dim; among equal values the LOWEST index wins.
    ``aten::topk`` as the reference uses it (native_ops/Topk.cpp:90-150, CPU twin
    python/regression/test_llm/test_topk.py:9-12) leaves tie order open; a stable
    descending sort pins it."""
    v, i = torch.sort(scores, dim=-1, descending=True, stable=True)
    return v[..., :k].contiguous(), i[..., :k].contiguous()


def noaux_tc_topk(scores: torch.Tensor, n_groups: int, topk_groups: int, top_k: int
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Grouped top-k of ``gt_noaux_tc_topk``
    (python/regression/test_llm/test_noaux_tc_topk.py:10-35): group score = sum of the
    two largest scores of the group, formed IN THE SCORES' DTYPE; keep ``topk_groups``
    groups; the others become -inf; top-``top_k`` of what is left.  Returns
    (values in the scores' dtype, int64 indices)."""
    bs, E = scores.shape
    g = scores.view(bs, n_groups, E // n_groups)
    top2 = topk_lowest_index(g, min(2, E // n_groups))[0]
    group_scores = top2.sum(dim=-1) if top2.shape[-1] > 1 else top2[..., 0]
    gidx = topk_lowest_index(group_scores, topk_groups)[1]
    mask = torch.ones(bs, n_groups, dtype=torch.bool).scatter_(1, gidx, False)
    masked = g.masked_fill(mask.unsqueeze(-1), float("-inf")).reshape(bs, E)
    return topk_lowest_index(masked, top_k)


def route_softmax_topk(logits: torch.Tensor, k: int, renorm: bool = True
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax (fp32) -> top-k -> optional renormalisation.  There is no reference test of
    this chain; it is the softmax twin of the sigmoid chain of
    python/regression/test_llm/test_torch_ops.py:439-455.  Returns (int32 ids, fp32 weights)."""
    p = torch.softmax(logits.to(torch.float32), dim=-1)
    w, ids = topk_lowest_index(p, k)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return ids.to(torch.int32), w


def route_sigmoid_grouped(logits: torch.Tensor, bias: Optional[torch.Tensor], n_groups: int,
                          topk_groups: int, k: int, scale: float
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """sigmoid -> (+bias for selection only) -> grouped top-k -> gather un-biased scores ->
    sum -> div -> mul(scale); op order of
    python/regression/test_llm/test_torch_ops.py:439-455 with the selection done by
    ``noaux_tc_topk``.  fp32 throughout.  Returns (int32 ids, fp32 weights)."""
    s = torch.sigmoid(logits.to(torch.float32))
    sel = s + bias.to(torch.float32) if bias is not None else s
    if n_groups > 1:
        _, ids = noaux_tc_topk(sel, n_groups, topk_groups, k)
    else:
        _, ids = topk_lowest_index(sel, k)
    w = torch.gather(s, 1, ids)
    w = w / w.sum(dim=-1, keepdim=True)
    w = w * scale
    return ids.to(torch.int32), w


def tie_free_rows(sel_scores: torch.Tensor, k: int, n_groups: int = 1, topk_groups: int = 1,
                  rel_gap: float = 1e-6) -> torch.Tensor:
    """Boolean mask of the rows whose selection is safe against ulp-level differences between exp
    implementations: the k-th and (k+1)-th largest selection scores (after group masking) and, with groups,
    the last kept and first dropped group score differ by more than ``rel_gap`` relative."""
    s = sel_scores.to(torch.float64)
    ok = torch.ones(s.shape[0], dtype=torch.bool)
    if n_groups > 1:
        g = s.view(s.shape[0], n_groups, -1)
        gs = torch.sort(g, dim=-1, descending=True)[0][..., :2].sum(-1)
        gv = torch.sort(gs, dim=-1, descending=True)[0]
        if topk_groups < n_groups:
            ok &= (gv[:, topk_groups - 1] - gv[:, topk_groups]) > rel_gap * gv[:, topk_groups - 1].abs().clamp_min(1e-30)
        keep = torch.sort(gs, dim=-1, descending=True, stable=True)[1][:, :topk_groups]
        mask = torch.ones(s.shape[0], n_groups, dtype=torch.bool).scatter_(1, keep, False)
        s = g.masked_fill(mask.unsqueeze(-1), float("-inf")).reshape(s.shape[0], -1)
    v = torch.sort(s, dim=-1, descending=True)[0]
    if v.shape[-1] > k:
        gap = v[:, k - 1] - v[:, k]
        ok &= ~torch.isfinite(gap) | (gap > rel_gap * v[:, k - 1].abs().clamp_min(1e-30))
    # ordering inside the top-k matters too (ids are compared position by position)
    inner = v[:, :k - 1] - v[:, 1:k]
    ok &= (inner > rel_gap * v[:, :k - 1].abs().clamp_min(1e-30)).all(-1)
    return ok


def assert_tie_free(sel_scores: torch.Tensor, k: int, rel_gap: float = 1e-6) -> None:
    """Generators call this: the k-th and (k+1)-th largest selection scores of every row
    must differ by more than ``rel_gap`` relative, so that ulp-level differences between
    exp implementations cannot change the selected set."""
    v = torch.sort(sel_scores.to(torch.float64), dim=-1, descending=True)[0]
    if v.shape[-1] <= k:
        return
    gap = v[..., : k] - v[..., 1: k + 1]
    finite = torch.isfinite(gap)
    ok = gap[finite] > rel_gap * v[..., :k][finite].abs().clamp_min(1e-30)
    assert bool(ok.all()), "routing scores are not tie-free at the top-k boundary"


# --------------------------------------------------------------------------
# permutation
# --------------------------------------------------------------------------
def permutation(ids: torch.Tensor, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable sort of the flat (token,slot) pairs by expert id.  Equivalent to the per-expert
    ``nonzero`` of the reference device kernel (my_ops/fusedMoE.pl:737-755): inside one
    expert the flat indices ``t*k+j`` ascend.  Returns (int32 sorted_pair[P], int32
    expert_offsets[E+1])."""
    flat = ids.reshape(-1).to(torch.int64)
    order = torch.sort(flat, stable=True)[1]
    counts = torch.bincount(flat, minlength=num_experts)
    offs = torch.zeros(num_experts + 1, dtype=torch.int64)
    offs[1:] = torch.cumsum(counts, 0)
    return order.to(torch.int32), offs.to(torch.int32)


def gather_scatter_index(ids: torch.Tensor, num_experts: int):
    """The reference kernel's scratch outputs (my_ops/fusedMoE.pl:737-755): for expert e,
    ``gather_index[e,:cnt]`` = ascending token ids routed to e, ``scatter_index[e,:cnt]`` =
    ascending flat ``t*k+j``; rows are padded with -1 here.  Returns (gather [E,T],
    scatter [E,T], num_per_expert [E]) as int32.  Assumes, like the reference, that the k
    experts of one token are distinct."""
    T, k = ids.shape
    gather = torch.full((num_experts, T), -1, dtype=torch.int32)
    scatter = torch.full((num_experts, T), -1, dtype=torch.int32)
    cnt = torch.zeros(num_experts, dtype=torch.int32)
    flat = ids.reshape(-1)
    for e in range(num_experts):
        nz = torch.nonzero(flat == e).flatten()
        n = nz.numel()
        cnt[e] = n
        scatter[e, :n] = nz.to(torch.int32)
        gather[e, :n] = (nz // k).to(torch.int32)
    return gather, scatter, cnt


# --------------------------------------------------------------------------
# experts
# --------------------------------------------------------------------------
def expert_mlp_w8a16(x: torch.Tensor, wg, wu, wd_ih, sg, su, sd_ih,
                     dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """One expert, rows ``x [m,H]`` -> ``[m,H]``; statement order of ``DeepseekMlp.forward``
    (python/regression/test_llm/test_moe.py:63-84): dequantise, gate linear, SiLU, up linear,
    multiply, down linear - every intermediate rounded to ``dtype``.  ``wd_ih``/``sd_ih`` are in
    the op's device layout ``[I,H]`` / ``[nI,nH]`` (the transposed, contiguous down projection,
    test_moe.py:285-288) and are transposed back so that the same ``F.linear`` call runs."""
    x = x.to(dtype)
    dq0 = weight_dequant(wg, sg, dtype=dtype)
    g = F.linear(x, dq0)
    a = F.silu(g)
    dq1 = weight_dequant(wu, su, dtype=dtype)
    u = F.linear(x, dq1)
    h = a * u
    dq2 = weight_dequant(wd_ih.t().contiguous(), sd_ih.t().contiguous(), dtype=dtype)
    return F.linear(h, dq2)


def experts_w8a16(x, ids, wg, wu, wd, sg, su, sd, dtype: torch.dtype = torch.bfloat16,
                  per_token: bool = False) -> torch.Tensor:
    """oracle-A.  ``out[t,j,:] = expert[ids[t,j]](x[t])`` (``DeepseekMoE.forward``,
    python/regression/test_llm/test_moe.py:93-98), un-weighted, ``[T,k,H]``.  By default the rows
    of one expert are batched through one dequantisation ("hoisted"); the reference dequantises
    per (token,slot) and hands the expert the 1-D row ``x[t]``, which changes nothing in the
    statements but the cost and, possibly, the blocking of the bf16 matrix products (so the last
    bit of a few elements).  ``per_token=True`` walks the pairs exactly as the reference does."""
    T, k = ids.shape
    H = x.shape[1]
    out = torch.zeros(T, k, H, dtype=dtype)
    if per_token:
        for t in range(T):
            for j in range(k):
                e = int(ids[t, j])
                out[t, j, :] = expert_mlp_w8a16(x[t], wg[e], wu[e], wd[e], sg[e], su[e], sd[e], dtype=dtype)
        return out
    flat = ids.reshape(-1).to(torch.int64)
    for e in torch.unique(flat).tolist():
        pos = torch.nonzero(flat == e).flatten()
        rows = x[pos // k]
        y = expert_mlp_w8a16(rows, wg[e], wu[e], wd[e], sg[e], su[e], sd[e], dtype=dtype)
        out.view(T * k, H)[pos] = y
    return out


def experts_bf16(x, ids, wg, wu, wd_ih, per_token: bool = False) -> torch.Tensor:
    """bf16-weight experts, un-weighted ``[T,k,H]``: ``QwenMlp.forward`` / ``QwenMoE.forward``
    (python/test/fused_moe_bf16.py:63-95) - gate linear, SiLU, up linear, multiply, down linear, all in bf16.
    ``wd_ih`` is the op's layout ``[E,I,H]`` (the transposed, contiguous down projection, :178) and is transposed
    back so that the same ``F.linear`` call runs.  ``per_token`` walks the pairs as the reference does."""
    T, k = ids.shape
    H = x.shape[1]
    x = x.to(torch.bfloat16)
    out = torch.zeros(T, k, H, dtype=torch.bfloat16)

    def mlp(rows, e):
        a = F.silu(F.linear(rows, wg[e]))
        return F.linear(a * F.linear(rows, wu[e]), wd_ih[e].t().contiguous())
    if per_token:
        for t in range(T):
            for j in range(k):
                out[t, j, :] = mlp(x[t], int(ids[t, j]))
        return out
    flat = ids.reshape(-1).to(torch.int64)
    for e in torch.unique(flat).tolist():
        pos = torch.nonzero(flat == e).flatten()
        out.view(T * k, H)[pos] = mlp(x[pos // k], e)
    return out


def expert_mlp_w8a8(x: torch.Tensor, wg, wu, wd_ih, sg, su, sd_ih) -> torch.Tensor:
    """One expert under the W8A8 contract, fp32 arithmetic: the statements of
    ``DeepseekMlp.forward`` (test_moe.py:63-84) with ``x`` and the SwiGLU product each replaced
    by their per-row 1x128 e4m3 quantise->dequantise image.  Returns fp32 ``[m,H]``."""
    xq, xs = quant_act_1x128(x)
    xd = dequant_act(xq, xs)
    g = F.linear(xd, weight_dequant(wg, sg, dtype=torch.float32))
    u = F.linear(xd, weight_dequant(wu, su, dtype=torch.float32))
    h = F.silu(g) * u
    hq, hs = quant_act_1x128(h)
    hd = dequant_act(hq, hs)
    wd = weight_dequant(wd_ih, sd_ih, dtype=torch.float32)  # [I,H]
    return hd @ wd


def experts_w8a8(x, ids, wg, wu, wd, sg, su, sd) -> torch.Tensor:
    """oracle-B.  ``[T,k,H]`` bf16, un-weighted."""
    T, k = ids.shape
    H = x.shape[1]
    out = torch.zeros(T * k, H, dtype=torch.float32)
    flat = ids.reshape(-1).to(torch.int64)
    for e in torch.unique(flat).tolist():
        pos = torch.nonzero(flat == e).flatten()
        out[pos] = expert_mlp_w8a8(x[pos // k].to(torch.float32), wg[e], wu[e], wd[e],
                                   sg[e], su[e], sd[e])
    return out.view(T, k, H).to(torch.bfloat16)


def combine(out_tkh: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Weighted combine ``y[t,:] = sum_j w[t,j] * out[t,j,:]`` as the caller-side ``bmm`` of
    python/regression/test_llm/test_bmm.py:118-134: bf16 operands, one bf16 rounding of the
    result."""
    o = out_tkh.to(torch.bfloat16)
    ww = w.to(torch.bfloat16)
    return torch.bmm(o.transpose(1, 2), ww.unsqueeze(-1)).squeeze(-1)


def moe_layer_w8a8(x, logits_or_ids, weights, *, shared=None, topk_w=None) -> torch.Tensor:
    """Whole layer under the W8A8 contract: experts (oracle-B) -> combine (+ shared expert with
    weight 1 added in fp32 before the final bf16 rounding)."""
    wg, wu, wd, sg, su, sd = weights
    out = experts_w8a8(x, logits_or_ids, wg, wu, wd, sg, su, sd)
    y = (out.to(torch.float32) * topk_w.to(torch.float32)[..., None]).sum(1)
    if shared is not None:
        swg, swu, swd, ssg, ssu, ssd = shared
        ys = expert_mlp_w8a8(x.to(torch.float32), swg, swu, swd, ssg, ssu, ssd)
        y = y + ys.to(torch.bfloat16).to(torch.float32)
    return y.to(torch.bfloat16)


# --------------------------------------------------------------------------
# metrics
# --------------------------------------------------------------------------
def cos_sim(a, b) -> float:
    """``0.5 + 0.5*cos`` (torch_tpu/utils/compare.py:5-15)."""
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    d = np.linalg.norm(a) * np.linalg.norm(b)
    c = 0.0 if d == 0 else float(a @ b) / d
    return 0.5 + 0.5 * c


def cal_diff(x: torch.Tensor, y: torch.Tensor):
    """(cos_diff, RMSE, amax_diff) (torch_tpu/utils/compare.py:17-21)."""
    x, y = x.double(), y.double()
    rmse = ((x - y) ** 2).mean().sqrt().item()
    cos_diff = 1 - 2 * (x * y).sum().item() / max((x * x + y * y).sum().item(), 1e-12)
    return cos_diff, rmse, (x - y).abs().max().item()


def parity_metrics(got: torch.Tensor, want: torch.Tensor) -> dict:
    """The tolerance the FP8 path is held to: ``max_rel = max|a-b| / max|b|`` (<= 2e-2) and
    plain cosine (>= 0.9995), plus the reference's own two metrics."""
    a = got.detach().to(torch.float64).reshape(-1).cpu()
    b = want.detach().to(torch.float64).reshape(-1).cpu()
    denom = float(b.abs().max().clamp_min(1e-30))
    cosine = float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-30))
    cd, rmse, amax = cal_diff(a, b)
    return {"max_rel": float((a - b).abs().max()) / denom, "cosine": cosine,
            "cos_sim": 0.5 + 0.5 * cosine, "cos_diff": cd, "rmse": rmse}


# --------------------------------------------------------------------------
# seeded synthetic inputs
# --------------------------------------------------------------------------
def make_expert_weights(E: int, H: int, I: int, seed: int, first_expert: int = 0,
                        std: float = 0.02):
    """Expert weights of the benchmark configurations: N(0, std) fp32 -> e4m3 with fp32 scale =
    block amax / 448 per 128x128 block.  Each (expert, matrix) has its own seed so that an
    expert-parallel rank can generate just its experts and the bits do not depend on the
    number of ranks.  Layout: gate/up ``[E,I,H]``; down generated as ``[H,I]`` and stored
    transposed ``[E,I,H]`` (python/regression/test_llm/test_moe.py:285)."""
    nI, nH = (I + BLOCK - 1) // BLOCK, (H + BLOCK - 1) // BLOCK
    wg = torch.empty(E, I, H, dtype=F8)
    wu = torch.empty(E, I, H, dtype=F8)
    wd = torch.empty(E, I, H, dtype=F8)
    sg = torch.empty(E, nI, nH)
    su = torch.empty(E, nI, nH)
    sd = torch.empty(E, nI, nH)
    for e in range(E):
        for m, (wq, sq) in enumerate(((wg, sg), (wu, su), (wd, sd))):
            g = torch.Generator().manual_seed((seed * 1000003 + (first_expert + e)) * 3 + m)
            if m < 2:
                w = torch.randn(I, H, generator=g) * std
            else:
                w = (torch.randn(H, I, generator=g) * std).t().contiguous()
            q, s = quant_weight_128x128(w)
            wq[e], sq[e] = q, s
    return wg, wu, wd, sg, su, sd


def make_inputs(T: int, H: int, E: int, seed: int = 0, router_std: float = 0.02):
    """x ``[T,H]`` bf16 ~ N(0,1), router weights ``[E,H]`` bf16 ~ N(0, router_std), fp32 logits
    computed from the bf16 values."""
    g = torch.Generator().manual_seed(seed * 7919 + 17)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    wr = (torch.randn(E, H, generator=g) * router_std).to(torch.bfloat16)
    logits = x.to(torch.float32) @ wr.to(torch.float32).t()
    return x, wr, logits


def zipf_bias(E: int, seed: int = 0, s: float = 1.2, mult: float = 3.0) -> torch.Tensor:
    """Per-expert logit bias ``mult * log(p_e)``, ``p_e`` proportional to ``rank_e**-s`` with a
    seeded random assignment of ranks 1..E to experts (the load-skew configuration)."""
    g = torch.Generator().manual_seed(seed * 31 + 5)
    ranks = (torch.randperm(E, generator=g) + 1).to(torch.float64)
    p = ranks ** (-s)
    p = p / p.sum()
    return (mult * torch.log(p)).to(torch.float32)
