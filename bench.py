"""Benchmark of the FP8 fused-MoE layer (route -> permute -> gate/up GEMM + SiLU*up -> down GEMM -> combine).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload mixtral|deepseek|qwen|small] [--tokens T]
    python bench.py --impl reference ...     # the reference's CPU arithmetic (oracle port) on the host cores

One "step" is one pass of the layer over one batch of T synthetic tokens per GPU.  Prints ONE JSON line:
  value      tokens/s with inputs resident in HBM (whole job, all GPUs)
  e2e        tokens/s through FusedMoE.forward_host: pinned host x -> H2D -> layer -> D2H of the result, every step
  roofline   the dominant kernel (gate/up GEMM) timed alone with CUDA events, algorithmic FLOPs or bytes / time / peak
  sweep      the same layer at the other token counts of the workload (decode sizes are HBM-bound)
  cpu_baseline  the CPU oracle (a port of the reference's CPU path) on a bounded sample, host cores stated
Inputs are seeded synthetic tensors of the named model shape (no datasets or checkpoints are involved).
Weights (>= 0.6 GB) are far larger than the 126 MB L2, so consecutive steps cannot be served from cache.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: H, I, E, k, routing, tokens (headline first), shared I
    "small": dict(H=1024, I=512, E=8, k=2, score="softmax", tokens=[16], desc="T16 H1024 I512 E8 top2"),
    "mixtral": dict(H=4096, I=14336, E=8, k=2, score="softmax", tokens=[4096, 1, 32, 512],
                    desc="Mixtral-8x7B-shaped layer"),
    "deepseek": dict(H=7168, I=2048, E=256, k=8, score="sigmoid", groups=8, topk_groups=4, scale=2.5, shared=2048,
                     tokens=[2048, 1, 64], desc="DeepSeek-V3-shaped layer (256 routed + 1 shared expert)"),
    "qwen": dict(H=2048, I=768, E=128, k=8, score="softmax", zipf=True, tokens=[8192],
                 desc="Qwen3-30B-A3B-shaped layer, Zipf(1.2)-skewed routing"),
}


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel (gate/up GEMM) at the headline
# size, taken from an ncu capture of this very command (profiles/moe_gemm_tc_dram_traffic.md); bench.py cannot run ncu
# itself, so the figure is carried here and is null for sizes that were not captured.
NCU_TRAFFIC_BYTES = {("mixtral", 4096): 1295.8e6, ("qwen", 8192): 245.3e6}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sus=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    src="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sus=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.stop, self.max_mhz = [], set(), False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake": 0x80}
        while not self.stop:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.05)

    def __enter__(self):
        if self.nv:
            self.t.start()
        return self

    def __exit__(self, *a):
        self.stop = True
        if self.nv:
            self.t.join(timeout=1)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def algorithmic(wl, T, e_act):
    H, I, k = wl["H"], wl["I"], wl["k"]
    Is = wl.get("shared", 0)
    flops = 6.0 * T * k * H * I + 6.0 * T * H * Is
    nH, nI = H // 128, I // 128
    wbytes = e_act * (3 * H * I + 12 * nH * nI) + (3 * H * Is + 12 * nH * (Is // 128) if Is else 0)
    abytes = 4 * T * H + 2 * wl["E"] * H + 8 * T * k
    return flops, wbytes + abytes


def build_layer(wl, T_max, dev, seed, first_expert=0, n_local=None, fused_combine=False):
    import torch
    import torch_tpu_b200
    from torch_tpu_b200 import weights as W
    from torch_tpu_b200.layer import FusedMoE, MoEConfig
    E = wl["E"]
    n_local = E if n_local is None else n_local
    w = W.random_experts(n_local, wl["H"], wl["I"], dev, seed=seed * 1000 + first_expert)
    g = torch.Generator(device=dev).manual_seed(seed + 12345)
    wr = (torch.randn(E, wl["H"], generator=g, device=dev) * 0.02).to(torch.bfloat16)
    bias = None
    if wl["score"] == "sigmoid":
        bias = torch.randn(E, generator=g, device=dev) * 0.01
    logit_bias = None
    if wl.get("zipf"):
        # per-expert logit bias 3*log(p_e), p_e ~ rank_e^-1.2 with a seeded random assignment of ranks to experts
        ranks = (torch.randperm(E, generator=torch.Generator().manual_seed(seed * 31 + 5)) + 1).double()
        p = ranks ** -1.2
        logit_bias = (3.0 * torch.log(p / p.sum())).float().to(dev)
    shared = W.random_experts(1, wl["H"], wl["shared"], dev, seed=seed + 777) if wl.get("shared") else None
    cfg = MoEConfig(wl["H"], wl["I"], E, wl["k"], wl["score"], wl.get("groups", 1), wl.get("topk_groups", 1), True,
                    wl.get("scale", 1.0), wl.get("shared", 0))
    layer = FusedMoE(cfg, wr, *w, bias=bias, shared=shared, logit_bias=logit_bias, max_tokens=T_max,
                     fused_combine=fused_combine)
    return layer


def make_x(T, H, dev, seed, zipf_bias=None):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, H, generator=g).to(torch.bfloat16)


def time_steps(fn, steps, warmup, barrier=None, finish=None):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    if finish:
        finish()   # e.g. make the timed stream wait for copies running on side streams
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1) / steps  # ms per step


def launches_per_step(wl, T, world=1, ep="nccl"):
    P = T * wl["k"]
    if world > 1 and ep == "p2p":
        # router, route, permute | counts exchange, plan, dispatch, barrier | scales, tiles, 2 GEMMs, barrier | combine
        n = 2 + (1 if P <= 1024 else 3) + 4 + 5 + 1
        if wl.get("shared"):
            n += (1 if T <= 1024 else 3) + 1 + 1 + 2
        return n
    if world > 1:
        # router, route, permute, pack | unpack ids, permute (received rows), unpack rows, tiles, 2 GEMMs | invert, combine
        n = 2 + (1 if P <= 1024 else 3) + 1 + 1 + 3 + 1 + 1 + 2 + 2
        if wl.get("shared"):
            n += (1 if T <= 1024 else 3) + 1 + 1 + 2      # permute (identity ids), tiles, quant, 2 GEMMs
        return n
    n = 2 + (1 if P <= 1024 else 3) + 1 + 1 + 2 + 1   # router, route, permute, tiles, quant, 2 GEMMs, combine
    if wl.get("shared"):
        n += 2 + 1 + 2                                  # identity offsets + tiles, quant, 2 GEMMs
    return n


def cpu_baseline(wl, layer, sample_tokens, kind_arith="w8a8"):
    """Oracle on the host cores over `sample_tokens` tokens of the same workload (weights copied from the device)."""
    import torch
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count())
    T = sample_tokens
    x = make_x(T, wl["H"], "cpu", seed=4242)
    wr = layer.router_w.cpu()
    t0 = time.perf_counter()
    logits = x.float() @ wr.float().t()
    if wl["score"] == "softmax":
        if layer.logit_bias is not None:
            logits = logits + layer.logit_bias.cpu()
        ids, w = O.route_softmax_topk(logits, wl["k"])
    else:
        ids, w = O.route_sigmoid_grouped(logits, layer.bias.cpu(), wl["groups"], wl["topk_groups"], wl["k"], wl["scale"])
    used = torch.unique(ids.long())
    wts = [t[used].cpu() for t in layer.w]           # only the activated experts travel to the host
    remap = torch.full((wl["E"],), -1, dtype=torch.long)
    remap[used] = torch.arange(len(used))
    ids_l = remap[ids.long()].to(torch.int32)
    t1 = time.perf_counter()
    if kind_arith == "w8a8":
        out = O.experts_w8a8(x, ids_l, *wts)
    else:
        out = O.experts_w8a16(x, ids_l, *wts)
    y = O.combine(out, w)
    if layer.shared is not None:
        sh = [t[0].cpu() for t in layer.shared]
        y = y + O.expert_mlp_w8a8(x.float(), *sh).to(torch.bfloat16)
    t2 = time.perf_counter()
    secs = t2 - t1  # routing and the weight download are excluded; the expert arithmetic + combine is what is timed
    return T / secs, secs


def run_reference(args, wl):
    """`--impl reference`: the reference's CPU arithmetic (W8A16, bf16 roundings: oracle-A, a port of
    python/regression/test_llm/test_moe.py:10-98 with the dequantisation hoisted per expert) on the host cores."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = wl["tokens"][0] if args.tokens is None else args.tokens
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    sample = args.sample_tokens
    small_wl = dict(wl)
    layer = build_layer(small_wl, 16, dev, seed=0)
    times = []
    for i in range(args.warmup + args.steps):
        tps, secs = cpu_baseline(wl, layer, sample, "w8a16")
        if i >= args.warmup:
            times.append(secs)
    ms = 1000 * sum(times) / len(times)
    val = sample / (ms / 1000)
    line = {"impl": "reference", "metric": "fp8_fused_moe_layer_tokens_per_s", "value": val, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations x e4m3 weights (cpu)",
            "data": "synthetic", "config": {"workload": f"{args.workload}: {wl['desc']}, {T} tokens/GPU"},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                             "sample": f"{sample} tokens per step through the activated experts (dequantised once per expert)"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="mixtral", choices=list(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=None, help="tokens per GPU (default: the workload's headline size)")
    ap.add_argument("--sample-tokens", type=int, default=32, help="tokens of the CPU sample")
    ap.add_argument("--ep", default="p2p", choices=["p2p", "nccl"],
                    help="exchange of the expert-parallel runs (N > 1): peer-memory stores or NCCL all-to-all")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        return run_reference(args, wl)

    # Libraries (NCCL prints its version banner) write to stdout; the contract is ONE JSON line there.  Everything
    # but that line goes to stderr: fd 1 is pointed at fd 2 and the line is written to the saved descriptor.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch_tpu_b200
    from torch_tpu_b200 import lib as L
    from torch_tpu_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    barrier = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(dev))
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())  # noqa: E731
    peaks = load_peaks()
    T = wl["tokens"][0] if args.tokens is None else args.tokens
    T_max = max([T] + ([] if args.tokens else wl["tokens"]))

    if world > 1:
        from torch_tpu_b200.ep import build_ep_layer
        try:
            layer = build_ep_layer(wl, T, dev, rank, world, seed=0, transport=args.ep)
        except RuntimeError as exc:
            # peer memory cannot be mapped on this machine (the set-up fails on every rank together): run the
            # all-to-all exchange instead and say so in the line
            if args.ep != "p2p" or "peer memory" not in str(exc):
                raise
            sys.stderr.write(f"bench: {exc}; using the NCCL all-to-all exchange\n")
            args.ep = "nccl"
            layer = build_ep_layer(wl, T, dev, rank, world, seed=0, transport="nccl")
    else:
        layer = build_layer(wl, T_max, dev, seed=0)

    # ---- device-resident throughput ---------------------------------------------------------------------------
    xs = [make_x(T, wl["H"], dev, seed=100 + rank * 10 + i).to(dev) for i in range(4)]
    it = [0]

    def step():
        layer.forward(xs[it[0] % 4])
        it[0] += 1

    with ClockSampler(local) as cs:
        ms = time_steps(step, args.steps, args.warmup, barrier)
    clocks = cs.summary()
    status = int((layer.layer if world > 1 else layer).status.item())
    if world > 1 and args.ep == "p2p":
        status |= int(layer.status.item())

    # ---- end to end with host buffers ---------------------------------------------------------------------------
    xh = [x.cpu().pin_memory() for x in xs]
    oh = torch.empty(T, wl["H"], dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        layer.forward_host(xh[it[0] % 4], oh)
        it[0] += 1

    ms_e2e = time_steps(step_e2e, args.steps, args.warmup, barrier, finish=layer.host_join)

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    line = {"metric": "fp8_fused_moe_layer_tokens_per_s", "value": T * world / (ms / 1000), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: {wl['desc']}, {T} tokens/GPU", "H": wl["H"], "I": wl["I"],
                       "E": wl["E"], "top_k": wl["k"], "parallelism": f"ep{world} ({args.ep})" if world > 1 else "single",
                       "l2": "weights >> 126 MB L2, 4 rotating input batches"},
            "e2e": {"value": T * world / (ms_e2e / 1000), "unit": "tokens/s", "h2d_bytes_per_step": T * wl["H"] * 2,
                    "d2h_bytes_per_step": T * wl["H"] * 2},
            "gpu_launches": launches_per_step(wl, T, world, args.ep) * args.steps, "clocks": clocks, "device_status": status}

    if rank == 0 and world == 1:
        # ---- roofline of the dominant kernel: gate/up GEMM alone on the filled workspace ---------------------------
        ids = layer.ids[:T]
        e_act = int(torch.unique(ids).numel())
        wg, wu, wd, sg, su, sd = layer.w
        out = layer.out[:T]

        def only(mask):
            def f():
                ops.experts(out, xs[0], wg, wu, wd, sg, su, sd, ids, layer.topk_w[:T], shared=layer.shared,
                            workspace=layer.workspace, stages=mask)
            return f
        layer.forward(xs[0])
        ms_g1 = time_steps(only(L.STAGE_GATE_UP), args.steps, 3)
        ms_g2 = time_steps(only(L.STAGE_DOWN), args.steps, 3)
        flops, nbytes = algorithmic(wl, T, e_act)
        Is = wl.get("shared", 0)
        f_g1 = 4.0 * T * wl["k"] * wl["H"] * wl["I"] + 4.0 * T * wl["H"] * Is
        b_g1 = e_act * 2 * wl["H"] * wl["I"] + 2 * wl["H"] * Is + T * wl["k"] * (wl["H"] + wl["I"])
        fp8_peak = 2 * peaks["bf16"]
        t_tc, t_hbm = f_g1 / (fp8_peak * 1e12), b_g1 / (peaks["hbm"] * 1e9)
        if t_tc >= t_hbm:
            roof = {"bound": "tensor", "achieved": f_g1 / (ms_g1 / 1000) / 1e12, "peak": fp8_peak, "unit": "TFLOP/s"}
        else:
            roof = {"bound": "hbm", "achieved": b_g1 / (ms_g1 / 1000) / 1e9, "peak": peaks["hbm"], "unit": "GB/s"}
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["traffic"] = NCU_TRAFFIC_BYTES.get((args.workload, T))
        roof["traffic_unit"] = "bytes per launch (ncu dram read + write)"
        roof["algorithmic_bytes"] = b_g1
        roof["kernel"] = "moe_gemm_tc_kernel<false> (gate/up GEMM + SiLU*up + requantise)"
        roof["ms_per_launch"] = ms_g1
        roof["peak_source"] = (f"{peaks['src']}: FP8 dense taken as 2 x the bf16 cuBLAS burst figure"
                               if roof["bound"] == "tensor" else f"{peaks['src']} copy bandwidth")
        roof["down_gemm_ms"] = ms_g2
        line["roofline"] = roof
        line["layer"] = {"flops_per_step": flops, "bytes_per_step": nbytes,
                         "tflops": flops / (ms / 1000) / 1e12, "gbs": nbytes / (ms / 1000) / 1e9,
                         "activated_experts": e_act}

        # ---- the other token counts of the workload ---------------------------------------------------------------
        if not args.no_sweep and args.tokens is None:
            sweep = []
            for Ts in wl["tokens"][1:]:
                xx = [make_x(Ts, wl["H"], dev, seed=300 + i).to(dev) for i in range(4)]
                j = [0]

                use_graph = Ts <= 1024   # launch-bound sizes: one graph launch instead of a dozen small ones

                def st():
                    (layer.forward_graph if use_graph else layer.forward)(xx[j[0] % 4])
                    j[0] += 1
                m = time_steps(st, max(args.steps, 30), 5)
                ea = int(torch.unique(layer.ids[:Ts]).numel())
                fl, nb = algorithmic(wl, Ts, ea)
                t_tc, t_hbm = fl / (fp8_peak * 1e12), nb / (peaks["hbm"] * 1e9)
                sweep.append({"tokens": Ts, "cuda_graph": use_graph, "ms_per_step": m, "tokens_per_s": Ts / (m / 1000),
                              "bound": "tensor" if t_tc >= t_hbm else "hbm", "activated_experts": ea,
                              "frac": (fl / (m / 1000) / 1e12 / fp8_peak) if t_tc >= t_hbm else
                              (nb / (m / 1000) / 1e9 / peaks["hbm"])})
            line["sweep"] = sweep

        # ---- CPU baseline -----------------------------------------------------------------------------------------
        if not args.no_cpu:
            tps, secs = cpu_baseline(wl, layer, args.sample_tokens, "w8a8")
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"{args.sample_tokens} tokens through the oracle's expert arithmetic "
                                              f"({secs:.1f} s; activated experts dequantised once each)"}
    if rank == 0:
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        import torch.distributed as dist
        if hasattr(layer, "close"):
            layer.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
