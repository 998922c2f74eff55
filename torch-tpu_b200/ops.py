"""Functional wrappers over the C ABI taking torch CUDA tensors (device memory and streams are torch's;
the arithmetic is all in libb200moe).  Every function enqueues on torch's current stream and returns
without synchronising.  Inputs must be contiguous CUDA tensors; nothing here falls back to PyTorch math."""
import ctypes

import torch

from . import lib as L

_DT = {torch.float32: L.F32, torch.bfloat16: L.BF16, torch.float16: L.F16}


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _chk(t, name, dtype=None):
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.is_contiguous()):
        raise ValueError(f"{name} must be a contiguous CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


def noaux_tc_topk(scores, n_groups, topk_groups, top_k):
    """Grouped top-k (reference op my_ops.noaux_tc_topk, my_ops/NoauxTcTopk.cpp:9-67).
    Returns (values [B,k] in scores' dtype, indices [B,k] int32)."""
    _chk(scores, "scores")
    B, E = scores.shape
    values = torch.empty(B, top_k, dtype=scores.dtype, device=scores.device)
    indices = torch.empty(B, top_k, dtype=torch.int32, device=scores.device)
    L.check(L.lib().b200moe_noaux_tc_topk(_ptr(values), _ptr(indices), _ptr(scores), _DT[scores.dtype], B, E,
                                          n_groups, topk_groups, top_k, _stream()), "b200moe_noaux_tc_topk")
    return values, indices


def topk(x, k):
    """Descending top-k along the last dim with int32 indices (aten::topk on the reference device,
    native_ops/Topk.cpp:90-150)."""
    _chk(x, "x")
    B, n = x.shape
    values = torch.empty(B, k, dtype=x.dtype, device=x.device)
    indices = torch.empty(B, k, dtype=torch.int32, device=x.device)
    L.check(L.lib().b200moe_topk(_ptr(values), _ptr(indices), _ptr(x), _DT[x.dtype], B, n, k, _stream()),
            "b200moe_topk")
    return values, indices


def router_logits(x, wr, out=None):
    _chk(x, "x", torch.bfloat16)
    _chk(wr, "wr", torch.bfloat16)
    T, H = x.shape
    E = wr.shape[0]
    if out is None:
        out = torch.empty(T, E, dtype=torch.float32, device=x.device)
    L.check(L.lib().b200moe_router_logits(_ptr(out), _ptr(x), _ptr(wr), T, H, E, _stream()), "b200moe_router_logits")
    return out


def route(logits, k, score_func="softmax", bias=None, n_groups=1, topk_groups=1, renorm=True, scale=1.0,
          ids=None, w=None, w_bf16=None, logit_bias=None):
    """(+logit_bias) -> score -> (+bias, selection only) -> group-limited top-k -> normalise -> scale.  Returns (ids int32 [T,k], w fp32 [T,k])."""
    _chk(logits, "logits", torch.float32)
    T, E = logits.shape
    if ids is None:
        ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    if w is None:
        w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    sf = L.SCORE_SOFTMAX if score_func == "softmax" else L.SCORE_SIGMOID
    L.check(L.lib().b200moe_route(_ptr(ids), _ptr(w), _ptr(w_bf16), _ptr(logits), _ptr(logit_bias), _ptr(bias), T, E, k, sf, n_groups,
                                  topk_groups, int(renorm), float(scale), _stream()), "b200moe_route")
    return ids, w


def permute(ids, num_experts, status=None):
    """Stable sort of the (token,slot) pairs by expert.  Returns (sorted_pair int32 [P], expert_offsets int32 [E+1])."""
    _chk(ids, "ids", torch.int32)
    T, k = ids.shape
    P = T * k
    sorted_pair = torch.empty(P, dtype=torch.int32, device=ids.device)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=ids.device)
    scratch = torch.empty(max(1, L.lib().b200moe_permute_scratch_ints(P, num_experts)), dtype=torch.int32,
                          device=ids.device)
    L.check(L.lib().b200moe_permute(_ptr(sorted_pair), _ptr(offsets), _ptr(ids), T, k, num_experts, _ptr(scratch),
                                    _ptr(status), _stream()), "b200moe_permute")
    return sorted_pair, offsets


def gather_scatter_index(sorted_pair, offsets, T, k, num_experts):
    dev = sorted_pair.device
    gather = torch.full((num_experts, T), -1, dtype=torch.int32, device=dev)
    scatter = torch.full((num_experts, T), -1, dtype=torch.int32, device=dev)
    cnt = torch.empty(num_experts, dtype=torch.int32, device=dev)
    L.check(L.lib().b200moe_gather_scatter_index(_ptr(gather), _ptr(scatter), _ptr(cnt), _ptr(sorted_pair),
                                                 _ptr(offsets), T, k, num_experts, _stream()),
            "b200moe_gather_scatter_index")
    return gather, scatter, cnt


def quant_rows(x, row_map=None, div=1):
    """Row gather + 1x128 e4m3 quantisation.  Returns (q e4m3 [rows,H], scales fp32 [H/128, ld]) - scales are stored
    group-major with ld = rows rounded up to 128."""
    _chk(x, "x", torch.bfloat16)
    H = x.shape[1]
    rows = row_map.numel() if row_map is not None else x.shape[0]
    ld = (rows + 127) // 128 * 128
    q = torch.empty(rows, H, dtype=torch.float8_e4m3fn, device=x.device)
    s_t = torch.zeros(H // 128, ld, dtype=torch.float32, device=x.device)
    L.check(L.lib().b200moe_quant_rows(_ptr(q), _ptr(s_t), ld, _ptr(x), _ptr(row_map), div, rows, H, _stream()),
            "b200moe_quant_rows")
    return q, s_t


def make_desc(T, H, I, E, k, *, I_shared=0, out_mode=L.OUT_PER_SLOT, act_mode=L.ACT_W8A8, impl=L.IMPL_AUTO,
              scale_dtype=torch.float32, w_dtype=torch.float32, impl_gate_up=L.IMPL_AUTO, impl_down=L.IMPL_AUTO,
              weights_bf16=False, stages=0, max_ctas=0):
    return L.ExpertsDesc(T, H, I, E, k, I_shared, out_mode, act_mode, impl, _DT[scale_dtype], _DT[w_dtype],
                         impl_gate_up, impl_down, int(weights_bf16), stages, max_ctas)


def experts_workspace_bytes(desc):
    return L.lib().b200moe_experts_workspace_bytes(ctypes.byref(desc))


def experts(out, x, wg, wu, wd, sg, su, sd, ids, topk_w=None, *, shared=None, act_mode=L.ACT_W8A8,
            impl=L.IMPL_AUTO, workspace=None, status=None, fused_combine=False, impl_gate_up=L.IMPL_AUTO,
            impl_down=L.IMPL_AUTO, stages=0, max_ctas=0):
    """Everything after routing (reference op my_ops.fused_moe_fused_experts, my_ops/fusedMoE.cpp:117-236).
    ``out`` [T,k,H] -> un-weighted per-slot rows; ``out`` [T,H] -> weighted combine with ``topk_w`` (+ ``shared`` =
    (wg,wu,wd,sg,su,sd) of a dense expert applied to every token), formed by a separate kernel in slot order or,
    with ``fused_combine``, inside the down GEMM's epilogue (fp32 reductions, order not fixed).  ``stages``: a
    mask of ``L.STAGE_*`` to re-run part of a call on a workspace that a whole call has filled.  ``max_ctas`` > 0
    caps the tensor-core kernels' persistent grids (SMs left to another stream's kernels).  Returns ``out``."""
    _chk(out, "out", torch.bfloat16)
    _chk(x, "x", torch.bfloat16)
    bf16w = wg.dtype == torch.bfloat16      # bf16 weights carry no scales: sg/su/sd may be None
    for n, t in (("wg", wg), ("wu", wu), ("wd", wd)):
        _chk(t, n, torch.bfloat16 if bf16w else torch.float8_e4m3fn)
    if bf16w:
        act_mode = L.ACT_W8A16
    else:
        for n, t in (("sg", sg), ("su", su), ("sd", sd)):
            _chk(t, n, sg.dtype)
    _chk(ids, "ids", torch.int32)
    T, H = x.shape
    E, I, _ = wg.shape
    k = ids.shape[1]
    out_mode = L.OUT_PER_SLOT if out.dim() == 3 else (L.OUT_COMBINED_FUSED if fused_combine else L.OUT_COMBINED)
    I_shared = shared[0].shape[-2] if shared is not None else 0
    d = make_desc(T, H, I, E, k, I_shared=I_shared, out_mode=out_mode, act_mode=act_mode, impl=impl,
                  scale_dtype=torch.float32 if bf16w else sg.dtype,
                  w_dtype=topk_w.dtype if topk_w is not None else torch.float32,
                  impl_gate_up=impl_gate_up, impl_down=impl_down, weights_bf16=bf16w, stages=stages,
                  max_ctas=max_ctas)
    need = experts_workspace_bytes(d)
    if need == 0 and T > 0:
        raise ValueError("unsupported sizes for b200moe_experts (H, I multiples of 128; see include/b200moe.h)")
    if workspace is None:
        workspace = torch.empty(need + 256, dtype=torch.uint8, device=x.device)
    base = (workspace.data_ptr() + 255) // 256 * 256
    avail = workspace.numel() - (base - workspace.data_ptr())
    sh = [_ptr(t) for t in shared] if shared is not None else [ctypes.c_void_p(0)] * 6
    L.check(L.lib().b200moe_experts(_ptr(out), _ptr(x), _ptr(wg), _ptr(wu), _ptr(wd), _ptr(sg), _ptr(su), _ptr(sd),
                                    _ptr(ids), _ptr(topk_w), *sh, ctypes.byref(d), ctypes.c_void_p(base), avail,
                                    _ptr(status), _stream()), "b200moe_experts")
    return out


def combine(y, w, add=None, out=None):
    _chk(y, "y", torch.bfloat16)
    T, k, H = y.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=y.device)
    L.check(L.lib().b200moe_combine(_ptr(out), _ptr(y), _ptr(w), _DT[w.dtype], _ptr(add), T, k, H, _stream()),
            "b200moe_combine")
    return out


def combine_indexed(y, pos, w, add=None, out=None, ids=None, num_experts=0):
    """out[t,:] = sum_j w[t,j] * y[pos[t*k+j], :] (+ add[t,:]); y bf16 [R,H], pos int32 [T*k] or None.  Slots with a
    negative ``pos`` or (when ``ids`` is given) an expert id outside [0, num_experts) contribute nothing."""
    _chk(y, "y", torch.bfloat16)
    T, k = w.shape
    H = y.shape[-1]
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=y.device)
    L.check(L.lib().b200moe_combine_masked(_ptr(out), _ptr(y), _ptr(pos), _ptr(w), _DT[w.dtype], _ptr(add), _ptr(ids),
                                           num_experts, T, k, H, _stream()), "b200moe_combine_masked")
    return out


def grouped_mlp_workspace_bytes(R, H, I, E, ld, scale_dtype=torch.float32):
    return L.lib().b200moe_grouped_mlp_workspace_bytes(R, H, I, E, ld, _DT[scale_dtype])


def grouped_mlp(y, xq, xs_t, expert_offsets, wg, wu, wd, sg, su, sd, R, row_map=None, impl=L.IMPL_AUTO,
                workspace=None, status=None):
    """Gate/up GEMM + SiLU*up + requantise + down GEMM on rows already quantised and sorted by (local) expert."""
    E, I, H = wg.shape
    ld = xs_t.shape[1]
    need = grouped_mlp_workspace_bytes(R, H, I, E, ld, sg.dtype)
    if workspace is None:
        workspace = torch.empty(need + 256, dtype=torch.uint8, device=y.device)
    base = (workspace.data_ptr() + 255) // 256 * 256
    avail = workspace.numel() - (base - workspace.data_ptr())
    L.check(L.lib().b200moe_grouped_mlp(_ptr(y), _ptr(xq), _ptr(xs_t), ld, _ptr(expert_offsets), _ptr(row_map),
                                        _ptr(wg), _ptr(wu), _ptr(wd), _ptr(sg), _ptr(su), _ptr(sd), _DT[sg.dtype], R, H,
                                        I, E, impl, ctypes.c_void_p(base), avail, _ptr(status), _stream()),
            "b200moe_grouped_mlp")
    return y


def linear_w8(x, w, scale, out=None, workspace=None, status=None):
    """out[M,N] = x[M,K] . dequant(w [N,K] e4m3, scale [ceil(N/128), K/128])^T on the FP8 tensor cores (activations
    quantised 1x128 on the fly).  Reference op: my_ops.mm_w8a16_dq_forward (my_ops/MmW8A16Dq.cpp:185-229)."""
    _chk(x, "x", torch.bfloat16)
    _chk(w, "w")
    _chk(scale, "scale")
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    need = L.lib().b200moe_linear_workspace_bytes(M, K, N, _DT[scale.dtype])
    if workspace is None:
        workspace = torch.empty(need + 256, dtype=torch.uint8, device=x.device)
    base = (workspace.data_ptr() + 255) // 256 * 256
    avail = workspace.numel() - (base - workspace.data_ptr())
    L.check(L.lib().b200moe_linear_w8(_ptr(out), _ptr(x), _ptr(w), _ptr(scale), _DT[scale.dtype], M, K, N,
                                      ctypes.c_void_p(base), avail, _ptr(status), _stream()), "b200moe_linear_w8")
    return out


def ep_packed_row_bytes(H):
    return L.lib().b200moe_ep_packed_row_bytes(H)


def ep_pack_rows(rows, x, sorted_pair, ids, experts_per_rank):
    T, H = x.shape
    k = ids.shape[1]
    L.check(L.lib().b200moe_ep_pack_rows(_ptr(rows), _ptr(x), _ptr(sorted_pair), _ptr(ids), T, k, experts_per_rank, H,
                                         _stream()), "b200moe_ep_pack_rows")
    return rows


def ep_unpack_ids(eid, rows, R, H):
    L.check(L.lib().b200moe_ep_unpack_ids(_ptr(eid), _ptr(rows), R, H, _stream()), "b200moe_ep_unpack_ids")
    return eid


def ep_unpack_rows(xq, xs_t, rows, order, R, H):
    L.check(L.lib().b200moe_ep_unpack_rows(_ptr(xq), _ptr(xs_t), xs_t.shape[1], _ptr(rows), _ptr(order), R, H,
                                           _stream()), "b200moe_ep_unpack_rows")


def invert_permutation(inv, perm, n):
    L.check(L.lib().b200moe_invert_permutation(_ptr(inv), _ptr(perm), n, _stream()), "b200moe_invert_permutation")
    return inv
