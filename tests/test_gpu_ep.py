"""Expert-parallel CUDA paths: the all-to-all one (pack, NCCL all-to-all, unpack, grouped MLP, indexed combine) and
the peer-memory one (counts exchange, plan, dispatch stores, grouped MLP with peer output, flag barriers).  With one
visible GPU both run on a single-rank group; with two or more GPUs a 2-rank job is spawned and every rank is checked
against the oracle over ALL experts."""
import os
import socket
import sys

import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run_rank(rank, world, port, q, mode):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    try:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(dev))
    except Exception as exc:                       # e.g. the rendezvous port was taken in the meantime
        q.put((rank, False, "rendezvous", repr(exc)[-300:]))
        return
    try:
        import torch_tpu_b200  # noqa: F401
        from torch_tpu_b200.ep import EPFusedMoE
        from torch_tpu_b200.layer import FusedMoE, MoEConfig
        H, I, E, k, Is = 512, 256, 16, 4, 256
        cfg = MoEConfig(H, I, E, k, "sigmoid", 4, 2, True, 2.5, shared_intermediate=Is)
        bias = torch.randn(E, generator=torch.Generator().manual_seed(3)) * 0.01
        shared = O.make_expert_weights(1, H, Is, seed=99)
        full = O.make_expert_weights(E, H, I, seed=5)
        El = E // world
        local = tuple(t[rank * El:(rank + 1) * El].contiguous().to(dev) for t in full)
        T = 150 + 37 * rank
        x, _, _ = O.make_inputs(T, H, E, seed=10 + rank, router_std=0.2)
        _, wr, _ = O.make_inputs(1, H, E, seed=1, router_std=0.2)
        layer = FusedMoE(cfg, wr.to(dev), *local, bias=bias.to(dev), shared=tuple(t.to(dev) for t in shared),
                         max_tokens=256, alloc_workspace=False)
        bad = mode.endswith("_badids")
        inline = mode.endswith("_inline")    # shared expert in line (default: on a side stream beside the dispatch)
        mode = mode.split("_")[0]
        if bad:
            # expert ids outside [0,E) reach the exchange: those (token,slot) pairs must be skipped everywhere
            # (no row dispatched, nothing summed) and the status word says so
            route = layer.route
            # made here, outside any stream capture; the patch itself is one kernel (the call is replayed from a graph)
            bad_pos = torch.tensor([3 * k + 1, 7 * k, 20 * k + k - 1], device=dev)
            bad_val = torch.tensor([E + 5, -2, 1 << 20], dtype=torch.int32, device=dev)

            def route_with_bad_ids(xx):
                ids_, w_ = route(xx)
                if xx.shape[0] > 20:
                    ids_.view(-1).index_copy_(0, bad_pos, bad_val)
                return ids_, w_
            layer.route = route_with_bad_ids
        if mode == "p2p":
            from torch_tpu_b200.ep_p2p import P2PFusedMoE
            ep = P2PFusedMoE(layer, E, max_tokens=256)
            if inline:
                ep.shared_ctas = 0
            ep(x[:40].to(dev))             # a first call of another size: epochs and buffers are reused after it
            y = ep(x.to(dev)).clone()
            torch.cuda.synchronize()
            assert int(ep.status.item()) == (1 if bad else 0), int(ep.status.item())
            ep.status.zero_()
            # the same call captured into a CUDA graph (device-side epochs, no allocation) and replayed twice
            for _ in range(2):
                yg = ep.forward_graph(x.to(dev))
                torch.cuda.synchronize()
                assert torch.equal(yg, y)
            assert int(ep.status.item()) == (1 if bad else 0), int(ep.status.item())
            ep.close()
        else:
            ep = EPFusedMoE(layer, E)
            y = ep(x.to(dev))
            torch.cuda.synchronize()
        ids, w = layer.ids[:T].cpu(), layer.topk_w[:T].cpu()
        wid, _ = O.route_sigmoid_grouped(layer.logits[:T].cpu(), bias, 4, 2, k, 2.5)
        dropped = (ids < 0) | (ids >= E)
        assert bool(dropped.any()) == bad
        ids_or, w_or = ids.clone(), w.clone()
        ids_or[dropped], w_or[dropped] = 0, 0.0          # a dropped slot contributes nothing
        want = O.moe_layer_w8a8(x, ids_or, full, shared=tuple(t[0] for t in shared), topk_w=w_or)
        assert bool(torch.isfinite(y.float()).all())
        m = O.parity_metrics(y, want)
        ok_rows = O.tie_free_rows(torch.sigmoid(layer.logits[:T].cpu()) + bias, k, 4, 2) & ~dropped.any(-1)
        ids_ok = bool(torch.equal(ids[ok_rows], wid[ok_rows]))
        q.put((rank, ids_ok and m["max_rel"] <= 2e-2 and m["cosine"] >= 0.9995, m["max_rel"], m["cosine"]))
    except Exception:
        import traceback
        q.put((rank, False, "exception", traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(1, "nccl"), (2, "nccl"), (1, "p2p"), (2, "p2p"), (1, "nccl_badids"),
                                        (1, "p2p_badids"), (2, "p2p_badids"), (1, "p2p_inline"), (2, "p2p_inline")])
def test_ep_cuda_path(world, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import queue
    import time
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    for attempt in range(3):                       # a taken rendezvous port is retried with another one
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_run_rank, args=(r, world, port, q, mode)) for r in range(world)]
        for p in procs:
            p.start()
        res, deadline = [], time.time() + 300
        while len(res) < world and time.time() < deadline:
            try:
                res.append(q.get(timeout=2))
            except queue.Empty:
                if not any(p.is_alive() for p in procs) and q.empty():
                    break                          # every rank is gone and none reported: do not sit out the limit
        for p in procs:
            p.join(timeout=60)
        if not any(len(r) > 2 and r[2] == "rendezvous" for r in res):
            break
    assert len(res) == world and all(r[1] for r in res), res


def test_ep_plan_tiles_every_destination_buffer():
    """b200moe_ep_plan for every rank of an 8-rank job on one GPU (the plan needs only the count matrix): the row
    ranges the ranks are given on each destination are disjoint, in (local expert, source rank) order, and end at the
    destination's own recv_offsets."""
    import ctypes
    import numpy as np
    sys.path.insert(0, ROOT)
    import torch_tpu_b200  # noqa: F401
    from torch_tpu_b200 import lib as L
    lib = L.lib()
    N, E = 8, 256
    El = E // N
    rng = np.random.default_rng(3)
    cnt = rng.integers(0, 300, size=(N, E)).astype(np.int32)
    cnt[:, 5] = 0                                    # an expert nobody routes to
    cnt_d = torch.from_numpy(cnt).cuda()
    dst = torch.empty(N, E, dtype=torch.int32, device="cuda")
    rcv = torch.empty(N, El + 1, dtype=torch.int32, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for r in range(N):
        L.check(lib.b200moe_ep_plan(ctypes.c_void_p(dst[r].data_ptr()), ctypes.c_void_p(rcv[r].data_ptr()),
                                    ctypes.c_void_p(cnt_d.data_ptr()), E, N, r, st), "b200moe_ep_plan")
    torch.cuda.synchronize()
    dst, rcv = dst.cpu().numpy(), rcv.cpu().numpy()
    tot = cnt.sum(0)
    for d in range(N):
        want_off = np.concatenate([[0], np.cumsum(tot[d * El:(d + 1) * El])])
        assert np.array_equal(rcv[d], want_off)
        pos = 0
        for le in range(El):
            e = d * El + le
            for r in range(N):                       # inside an expert: sources in rank order, back to back
                assert dst[r, e] == pos, (d, le, r)
                pos += cnt[r, e]
        assert pos == rcv[d, El]


def test_peer_flag_wait_runs_out_and_reports():
    """Failure detection without a fault: a 2-rank flag barrier whose peer never announces itself (its flag word is a
    piece of this process's own memory that nothing sets).  The kernel gives up after its time limit, raises status
    bit 2 (value 4) and returns; the context stays usable."""
    import ctypes
    import time
    sys.path.insert(0, ROOT)
    import torch_tpu_b200  # noqa: F401
    from torch_tpu_b200 import lib as L
    lib = L.lib()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")            # [0:8] mine, [32:40] the absent peer's
    table = torch.tensor([flags.data_ptr(), flags.data_ptr() + 128], dtype=torch.int64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.time()
    L.check(lib.b200moe_p2p_barrier(ctypes.c_void_p(table.data_ptr()), 2, 0, ctypes.c_uint32(1), None,
                                    ctypes.c_void_p(status.data_ptr()), st), "b200moe_p2p_barrier")
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert int(status.item()) == L.STATUS_PEER_TIMEOUT
    assert 1.0 < waited < 10.0, waited
    assert int(flags[0].item()) == 1 and int(flags[32].item()) == 1      # both announcements were made
    # the same barrier completes at once when the peer's word is there
    flags[1] = 2
    status.zero_()
    L.check(lib.b200moe_p2p_barrier(ctypes.c_void_p(table.data_ptr()), 2, 0, ctypes.c_uint32(2), None,
                                    ctypes.c_void_p(status.data_ptr()), st), "b200moe_p2p_barrier")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
