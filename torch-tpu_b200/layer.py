"""FusedMoE: the caller-side wrapper that the reference leaves to model code - router matmul, routing chain
(python/regression/test_llm/test_torch_ops.py:439-455), the fused experts op
(python/regression/test_llm/test_moe.py:131-140) and the weighted combine (test_bmm.py:118-134) - as one call
that allocates nothing after construction (all buffers are sized for ``max_tokens`` up front)."""
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import lib as L
from . import ops


@dataclass
class MoEConfig:
    hidden: int
    intermediate: int
    num_experts: int
    top_k: int
    score_func: str = "softmax"      # "softmax" | "sigmoid"
    n_groups: int = 1                # group-limited routing (DeepSeek-V3: 8)
    topk_groups: int = 1             # groups kept (DeepSeek-V3: 4)
    renorm: bool = True              # weights / sum(weights)
    routed_scale: float = 1.0        # DeepSeek-V3: 2.5
    shared_intermediate: int = 0     # 0 = no shared expert


class FusedMoE:
    """One MoE layer on one GPU.  Weights are in the op layout: gate/up/down ``[E,I,H]`` float8_e4m3fn (down =
    W_down^T contiguous), scales ``[E,I/128,H/128]`` fp32 or bf16, router ``[E,H]`` bf16, optional selection bias
    ``[E]`` fp32 (added to the scores for selection only), optional ``logit_bias`` ``[E]`` fp32 (added to the logits), optional shared expert ``(wg,wu,wd,sg,su,sd)`` with a leading dim of 1."""

    def __init__(self, cfg: MoEConfig, router_w, wg, wu, wd, sg, su, sd, bias=None, shared: Optional[Tuple] = None,
                 logit_bias=None, max_tokens: int = 4096, act_mode: int = L.ACT_W8A8, impl: int = L.IMPL_AUTO,
                 alloc_workspace: bool = True, fused_combine: bool = False):
        self.cfg = cfg
        self.router_w, self.bias, self.logit_bias = router_w, bias, logit_bias
        self.w = (wg, wu, wd, sg, su, sd)
        self.shared = shared
        self.act_mode, self.impl = act_mode, impl
        self.fused_combine = fused_combine  # weighted combine inside the down GEMM's epilogue (see ops.experts)
        dev = wg.device
        self.device = dev
        self.max_tokens = max_tokens
        E, k, H = cfg.num_experts, cfg.top_k, cfg.hidden
        self.logits = torch.empty(max_tokens, E, dtype=torch.float32, device=dev)
        self.ids = torch.empty(max_tokens, k, dtype=torch.int32, device=dev)
        self.topk_w = torch.empty(max_tokens, k, dtype=torch.float32, device=dev)
        self.out = torch.empty(max_tokens, H, dtype=torch.bfloat16, device=dev)
        self.x_dev = torch.empty(max_tokens, H, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._graphs = {}
        self.workspace = None
        if alloc_workspace:  # an expert-parallel shard runs its experts through other entry points
            d = ops.make_desc(max_tokens, H, cfg.intermediate, E, k, I_shared=cfg.shared_intermediate,
                              out_mode=L.OUT_COMBINED_FUSED if fused_combine else L.OUT_COMBINED, act_mode=act_mode, impl=impl, scale_dtype=sg.dtype)
            self.workspace = torch.empty(ops.experts_workspace_bytes(d) + 256, dtype=torch.uint8, device=dev)

    def route(self, x):
        T = x.shape[0]
        c = self.cfg
        logits = ops.router_logits(x, self.router_w, out=self.logits[:T])
        return ops.route(logits, c.top_k, c.score_func, self.bias, c.n_groups, c.topk_groups, c.renorm,
                         c.routed_scale, ids=self.ids[:T], w=self.topk_w[:T], logit_bias=self.logit_bias)

    def forward(self, x, out=None):
        """x bf16 [T,H] on the device -> bf16 [T,H] (a view of an internal buffer unless ``out`` is given)."""
        T = x.shape[0]
        if T > self.max_tokens:
            raise ValueError(f"{T} tokens > max_tokens={self.max_tokens}")
        ids, w = self.route(x)
        if out is None:
            out = self.out[:T]
        wg, wu, wd, sg, su, sd = self.w
        return ops.experts(out, x, wg, wu, wd, sg, su, sd, ids, w, shared=self.shared, act_mode=self.act_mode,
                           impl=self.impl, workspace=self.workspace, status=self.status,
                           fused_combine=self.fused_combine)

    __call__ = forward

    def capture(self, T: int):
        """Capture forward() for exactly T tokens into a CUDA graph (the call allocates nothing and never touches the
        host, so the whole layer replays as one launch - what matters at decode sizes, where a dozen small kernels
        would otherwise cost more in launch gaps than in work).  Use forward_graph() afterwards."""
        x_static = self.x_dev[:T]
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):           # first calls set function attributes: keep them out of the capture
                self.forward(x_static)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y = self.forward(x_static)
        self._graphs[T] = (g, y)
        return g

    def forward_graph(self, x):
        """Replay the graph captured for x.shape[0] tokens (captures it on first use)."""
        T = x.shape[0]
        if T not in self._graphs:
            self.capture(T)
        g, y = self._graphs[T]
        self.x_dev[:T].copy_(x, non_blocking=True)
        g.replay()
        return y

    def forward_host(self, x_host, out_host):
        """End-to-end call with HOST buffers (pinned, so that the copies are asynchronous): H2D of x on a copy stream,
        the layer on the current stream, D2H of the result on a second copy stream, with two device buffers each way -
        the copies of neighbouring calls overlap the compute of this one, as a serving loop would run it.  out_host is
        valid after host_join() + a stream synchronise (or torch.cuda.synchronize())."""
        return _host_pipeline_call(self, self.forward, x_host, out_host)

    def host_join(self):
        """Make the current stream wait for every copy that forward_host has enqueued."""
        _host_pipeline_join(self)


def _host_pipeline_state(obj, T, H, dev):
    st = getattr(obj, "_hp", None)
    if st is None or st["x"][0].shape[0] < T:
        cap = max(T, getattr(obj, "max_tokens", T))
        st = dict(i=0, h2d=torch.cuda.Stream(device=dev), d2h=torch.cuda.Stream(device=dev),
                  x=[torch.empty(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(2)],
                  y=[torch.empty(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(2)],
                  x_free=[torch.cuda.Event() for _ in range(2)], x_ready=[torch.cuda.Event() for _ in range(2)],
                  y_ready=[torch.cuda.Event() for _ in range(2)], y_free=[torch.cuda.Event() for _ in range(2)])
        cur = torch.cuda.current_stream(dev)
        for e in st["x_free"] + st["y_free"]:
            e.record(cur)
        obj._hp = st
    return st


def _host_pipeline_call(obj, fwd, x_host, out_host):
    T, H = x_host.shape
    dev = obj.device if hasattr(obj, "device") else obj.layer.device
    st = _host_pipeline_state(obj, T, H, dev)
    i = st["i"] & 1
    st["i"] += 1
    cur = torch.cuda.current_stream(dev)
    xb, yb = st["x"][i][:T], st["y"][i][:T]
    st["h2d"].wait_event(st["x_free"][i])            # the compute that read this input buffer two calls ago is done
    with torch.cuda.stream(st["h2d"]):
        xb.copy_(x_host, non_blocking=True)
        st["x_ready"][i].record(st["h2d"])
    cur.wait_event(st["x_ready"][i])
    cur.wait_event(st["y_free"][i])                  # the D2H that read this output buffer two calls ago is done
    fwd(xb, out=yb)                                  # the layer writes straight into the pipeline's output buffer
    st["x_free"][i].record(cur)
    st["y_ready"][i].record(cur)
    st["d2h"].wait_event(st["y_ready"][i])
    with torch.cuda.stream(st["d2h"]):
        out_host.copy_(yb, non_blocking=True)
        st["y_free"][i].record(st["d2h"])
    return out_host


def _host_pipeline_join(obj):
    st = getattr(obj, "_hp", None)
    if st is not None:
        dev = obj.device if hasattr(obj, "device") else obj.layer.device
        cur = torch.cuda.current_stream(dev)
        for e in st["y_free"]:
            cur.wait_event(e)
