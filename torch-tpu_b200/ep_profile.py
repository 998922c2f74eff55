"""Timing helper for the peer-memory expert-parallel layer (one rank per GPU; launch with torch.distributed.run).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29521 \
        torch-tpu_b200/ep_profile.py phases <workload> <tokens per GPU>
    python -m torch.distributed.run ... torch-tpu_b200/ep_profile.py decode <workload> <tokens per GPU>

``phases``: per-phase device time of P2PFusedMoE.forward on every rank (CUDA events recorded between the steps of
the call, 6 steps averaged).  ``decode``: the whole step eager versus replayed as one CUDA graph per rank, max over
ranks.  Workloads are bench.py's (synthetic seeded tensors of the named model shape).
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import bench
    mode, name, T = sys.argv[1], sys.argv[2], int(sys.argv[3])
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    import torch_tpu_b200  # noqa: F401
    from torch_tpu_b200.ep import build_ep_layer
    wl = bench.WORKLOADS[name]
    layer = build_ep_layer(wl, T, dev, rank, world, seed=0, transport="p2p")
    xs = [bench.make_x(T, wl["H"], dev, seed=100 + rank * 10 + i).to(dev) for i in range(4)]
    if mode == "phases":
        for i in range(4):
            layer(xs[i])
        torch.cuda.synchronize()
        dist.barrier()
        acc, steps = {}, 6
        for i in range(steps):
            layer.phase_events = []
            layer(xs[i % 4])
            torch.cuda.synchronize()
            ev = layer.phase_events
            for (_, e0), (n1, e1) in zip(ev[:-1], ev[1:]):
                acc[n1] = acc.get(n1, 0.0) + e0.elapsed_time(e1) / steps
        layer.phase_events = None
        print(f"rank {rank} received rows {int(layer.recv_offsets[-1])}: "
              + "  ".join(f"{k} {v * 1000:.0f}us" for k, v in acc.items()), flush=True)
    else:
        it = [0]

        def bar():
            dist.barrier()
            torch.cuda.synchronize()

        def eager():
            layer(xs[it[0] % 4])
            it[0] += 1

        def graph():
            layer.forward_graph(xs[it[0] % 4])
            it[0] += 1
        ms_e = bench.time_steps(eager, 30, 5, bar)
        ms_g = bench.time_steps(graph, 30, 5, bar)
        t = torch.tensor([ms_e, ms_g], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(f"{name}, {T} tokens/GPU x {world} GPUs: eager {float(t[0]) * 1e3:.0f} us, graph "
                  f"{float(t[1]) * 1e3:.0f} us, status {int(layer.status.item())}", flush=True)
    layer.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
