"""Expert-parallel host logic on CPU ranks (gloo, world_size 2 and 3): split computation, dispatch/return ordering,
inverse-permutation combine.  The kernels are replaced by a CPU backend built from the oracle, so what is tested is
exactly the code of torch-tpu_b200/ep.py that also runs on GPUs.  Also: a rank that never joins is detected through
the process-group timeout (failure injected on the host)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class CpuBackend:
    """Same interface as ep.CudaBackend, arithmetic from the oracle (test infrastructure only)."""

    def __init__(self):
        from oracle import moe_oracle as O
        self.O = O

    def route(self, layer, x):
        logits = x.float() @ layer.router_w.float().t()
        c = layer.cfg
        if c.score_func == "softmax":
            return self.O.route_softmax_topk(logits, c.top_k)
        return self.O.route_sigmoid_grouped(logits, layer.bias, c.n_groups, c.topk_groups, c.top_k, c.routed_scale)

    def permute(self, ids, E):
        return self.O.permutation(ids, E)

    def row_bytes(self, H):
        return (H + 4 * (H // 128) + 4 + 15) // 16 * 16

    def pack(self, x, sorted_pair, ids, experts_per_rank):
        P, (T, H), k = sorted_pair.numel(), x.shape, ids.shape[1]
        rows = torch.zeros(P, self.row_bytes(H), dtype=torch.uint8)
        tok = (sorted_pair // k).long()
        q, s = self.O.quant_act_1x128(x[tok].float())
        rows[:, :H] = q.view(torch.uint8)
        rows[:, H:H + 4 * (H // 128)] = s.contiguous().view(torch.uint8).view(P, -1)
        eid = (ids.reshape(-1)[sorted_pair.long()] % experts_per_rank).to(torch.int32)
        rows[:, H + 4 * (H // 128):H + 4 * (H // 128) + 4] = eid.view(torch.uint8).view(P, 4)
        return rows

    def local_mlp(self, rows, R, H, weights):
        O = self.O
        wg, wu, wd, sg, su, sd = weights
        nH = H // 128
        rows = rows[:R]
        q = rows[:, :H].contiguous().view(torch.float8_e4m3fn)
        s = rows[:, H:H + 4 * nH].contiguous().view(torch.float32).view(R, nH)
        eid = rows[:, H + 4 * nH:H + 4 * nH + 4].contiguous().view(torch.int32).view(R)
        xd = O.dequant_act(q, s)
        y = torch.zeros(R, H)
        for e in torch.unique(eid).tolist():
            m = eid == e
            g = torch.nn.functional.linear(xd[m], O.weight_dequant(wg[e], sg[e], dtype=torch.float32))
            u = torch.nn.functional.linear(xd[m], O.weight_dequant(wu[e], su[e], dtype=torch.float32))
            hq, hs = O.quant_act_1x128(torch.nn.functional.silu(g) * u)
            y[m] = O.dequant_act(hq, hs) @ O.weight_dequant(wd[e], sd[e], dtype=torch.float32)
        return y.to(torch.bfloat16)

    def shared_mlp(self, x, shared):
        return self.O.expert_mlp_w8a8(x.float(), *[t[0] for t in shared]).to(torch.bfloat16)

    def combine(self, y_back, sorted_pair, w, add):
        T, k = w.shape
        inv = torch.empty_like(sorted_pair)
        inv[sorted_pair.long()] = torch.arange(sorted_pair.numel(), dtype=torch.int32)
        y = y_back[inv.long()].view(T, k, -1).float()
        out = (y * w.float()[..., None]).sum(1)
        if add is not None:
            out = out + add.float()
        return out.to(torch.bfloat16)


def _worker(rank, world, port, cfgname, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torch_tpu_b200  # noqa: F401
        from oracle import moe_oracle as O
        from torch_tpu_b200.ep import EPFusedMoE
        from torch_tpu_b200.layer import FusedMoE, MoEConfig
        H, I, E = 256, 128, 12
        if cfgname == "softmax":
            cfg = MoEConfig(H, I, E, 3)
            bias, shared = None, None
        else:
            cfg = MoEConfig(H, I, E, 4, "sigmoid", 4, 2, True, 2.5, shared_intermediate=128)
            bias = torch.randn(E, generator=torch.Generator().manual_seed(3)) * 0.01
            shared = O.make_expert_weights(1, H, 128, seed=99)
        El = E // world
        full = O.make_expert_weights(E, H, I, seed=5)                      # every rank can build all experts ...
        local = tuple(t[rank * El:(rank + 1) * El].contiguous() for t in full)   # ... and keeps its shard
        T = 17 + 5 * rank                                                  # ragged token counts per rank
        x, _, _ = O.make_inputs(T, H, E, seed=10 + rank, router_std=0.2)
        _, wr, _ = O.make_inputs(1, H, E, seed=1, router_std=0.2)          # replicated router
        layer = FusedMoE(cfg, wr, *local, bias=bias, shared=shared, max_tokens=64, alloc_workspace=False)
        ep = EPFusedMoE(layer, E, backend=CpuBackend())
        y = ep(x)
        # single-process reference over ALL experts for this rank's tokens
        be = CpuBackend()
        ids, w = be.route(layer, x)
        want = O.moe_layer_w8a8(x, ids, full, shared=tuple(t[0] for t in shared) if shared else None, topk_w=w)
        m = O.parity_metrics(y, want)
        counts = ep.last_counts
        ok = m["max_rel"] < 1e-2 and m["cosine"] > 0.9999 and int(counts.sum()) == sum(
            (17 + 5 * r) * cfg.top_k for r in range(world))
        q.put((rank, ok, m["max_rel"], m["cosine"]))
    except Exception as e:  # report instead of letting the parent wait for its time-out
        import traceback
        q.put((rank, False, "exception", traceback.format_exc()[-800:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,cfgname", [(2, "softmax"), (2, "deepseek_like"), (3, "softmax")])
def test_ep_layer_matches_single_process_oracle(world, cfgname):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, cfgname, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert all(r[1] for r in res), res


def _absent_worker(rank, world, port, q):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        if rank == 1:
            q.put((1, "left"))          # leaves between steps: no collective of this rank is in flight
            return
        t = torch.zeros(world, dtype=torch.int64)
        out = torch.empty(world * world, dtype=torch.int64)
        try:
            dist.all_gather_into_tensor(out, t)
            q.put((0, "no error"))
        except Exception as e:          # the short process-group timeout ends the collective with an error
            q.put((0, "error: " + type(e).__name__))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_absent_rank_is_detected_by_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_absent_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert res[1] == "left" and res[0].startswith("error"), res


def test_ep_rejects_indivisible_expert_count():
    from torch_tpu_b200.ep import EPFusedMoE

    class G:
        pass
    import unittest.mock as um
    with um.patch("torch.distributed.get_world_size", return_value=4), um.patch("torch.distributed.get_rank", return_value=0):
        with pytest.raises(ValueError):
            EPFusedMoE(G(), 10, backend=object())
