"""Expert parallelism for the fused-MoE layer: one process per GPU, experts sharded contiguously over the ranks
(rank r owns experts [r*E/N, (r+1)*E/N)), tokens data-parallel, router and shared expert replicated.

    route (local) -> permute by GLOBAL expert id (rows come out grouped by destination rank)
      -> pack: gather + 1x128 e4m3 quantise + append scales and the destination-local expert id
      -> all-to-all (variable splits) of packed rows                                   [dispatch]
      -> permute the received rows by local expert -> unpack into the GEMM layout
      -> grouped gate/up GEMM + SiLU*up + requantise + down GEMM, rows scattered back to receive order
      -> all-to-all of bf16 result rows with the splits reversed                       [combine]
      -> weighted combine through the inverse permutation (+ local shared expert)

The reference has no expert-parallel code (its only MoE-adjacent collective is the equal-split all_to_all_single of
python/dist_test2260/test_all_to_all.py:19-44 over ProcessGroupSCCL::alltoall_base); the collective here is
``torch.distributed.all_to_all_single`` with per-rank split sizes (NCCL over NVLink on GPUs, gloo in the CPU tests).
Split sizes are needed on the host, so each call synchronises once on a [N,N] count matrix.

The arithmetic lives behind a small backend interface so that the host logic (splits, index plumbing, ordering) is
testable with CPU ranks: ``CudaBackend`` calls the C ABI; tests supply their own.
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist


class CudaBackend:
    """The product path: every step is a kernel of libb200moe called through the C ABI."""

    def __init__(self, layer_cfg, device, act_impl=0):
        from . import ops
        self.ops, self.dev, self.impl = ops, device, act_impl

    def route(self, layer, x):
        return layer.route(x)

    def permute(self, ids, E):
        return self.ops.permute(ids, E)

    def row_bytes(self, H):
        return self.ops.ep_packed_row_bytes(H)

    def pack(self, x, sorted_pair, ids, experts_per_rank):
        P = sorted_pair.numel()
        rows = torch.empty(P, self.row_bytes(x.shape[1]), dtype=torch.uint8, device=x.device)
        return self.ops.ep_pack_rows(rows, x, sorted_pair, ids, experts_per_rank)

    def local_mlp(self, rows, R, H, weights):
        """received packed rows -> bf16 results in receive order"""
        ops = self.ops
        wg, wu, wd, sg, su, sd = weights
        El = wg.shape[0]
        dev = rows.device
        eid = torch.empty(max(R, 1), 1, dtype=torch.int32, device=dev)
        ops.ep_unpack_ids(eid, rows, R, H)
        order, offsets = ops.permute(eid[:R], El)
        ld = (R + 127) // 128 * 128
        xq = torch.empty(max(R, 1), H, dtype=torch.uint8, device=dev)
        xs_t = torch.empty(H // 128, max(ld, 128), dtype=torch.float32, device=dev)
        ops.ep_unpack_rows(xq, xs_t, rows, order, R, H)
        y = torch.empty(max(R, 1), H, dtype=torch.bfloat16, device=dev)
        ops.grouped_mlp(y, xq, xs_t, offsets, wg, wu, wd, sg, su, sd, R, row_map=order, impl=self.impl)
        return y[:R]

    def shared_mlp(self, x, shared):
        T, H = x.shape
        out = torch.empty(T, 1, H, dtype=torch.bfloat16, device=x.device)
        ids = torch.zeros(T, 1, dtype=torch.int32, device=x.device)
        self.ops.experts(out, x, *shared, ids)
        return out.view(T, H)

    def combine(self, y_back, sorted_pair, w, add, out=None):
        inv = torch.empty_like(sorted_pair)
        self.ops.invert_permutation(inv, sorted_pair, sorted_pair.numel())
        return self.ops.combine_indexed(y_back, inv, w, add=add, out=out)


class EPFusedMoE:
    """Expert-parallel MoE layer.  ``layer`` is a FusedMoE holding the replicated router (its expert weights are the
    LOCAL shard); ``group`` the process group (default: world)."""

    def __init__(self, layer, num_experts_global: int, backend=None, group=None):
        self.layer, self.E, self.group = layer, num_experts_global, group
        self.N = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts_global % self.N:
            raise ValueError("the number of experts must be divisible by the number of ranks")
        self.El = num_experts_global // self.N
        self.backend = backend or CudaBackend(layer.cfg, layer.device, layer.impl)
        self.last_counts = None

    def split_sizes(self, offsets: torch.Tensor) -> Tuple[list, list]:
        """From expert_offsets [E+1] of the local permutation: rows this rank sends to every rank and, after one
        exchange of the count vectors, rows it receives from every rank."""
        N, El = self.N, self.El
        bounds = offsets[torch.arange(0, N + 1, device=offsets.device) * El].to(torch.int64)
        send = bounds[1:] - bounds[:-1]                               # [N] on the device
        allc = torch.empty(N * N, dtype=torch.int64, device=offsets.device)
        dist.all_gather_into_tensor(allc, send.contiguous(), group=self.group)
        allc = allc.view(N, N).cpu()                                  # the one host synchronisation of the call
        self.last_counts = allc
        return allc[self.rank].tolist(), allc[:, self.rank].tolist()

    def forward(self, x, out=None):
        be, layer = self.backend, self.layer
        T, H = x.shape
        ids, w = be.route(layer, x)                                   # ids over GLOBAL experts
        sorted_pair, offsets = be.permute(ids, self.E)
        send, recv = self.split_sizes(offsets)
        rows = be.pack(x, sorted_pair, ids, self.El)
        RB = rows.shape[1]
        R, S = int(sum(recv)), int(sum(send))   # S < T*k when ids outside [0,E) were dropped by the permutation
        recv_rows = torch.empty(max(R, 1), RB, dtype=torch.uint8, device=x.device)
        dist.all_to_all_single(recv_rows[:R], rows[:S], recv, send, group=self.group)
        y_recv = be.local_mlp(recv_rows, R, H, layer.w)
        y_back = torch.empty(max(T * ids.shape[1], 1), H, dtype=torch.bfloat16, device=x.device)
        dist.all_to_all_single(y_back[:S], y_recv.contiguous(), send, recv, group=self.group)
        add = be.shared_mlp(x, layer.shared) if layer.shared is not None else None
        return be.combine(y_back, sorted_pair, w, add) if out is None else be.combine(y_back, sorted_pair, w, add, out=out)

    __call__ = forward

    def forward_host(self, x_host, out_host):
        """Host-buffer entry point, pipelined like FusedMoE.forward_host."""
        from .layer import _host_pipeline_call
        return _host_pipeline_call(self, self.forward, x_host, out_host)

    def host_join(self):
        from .layer import _host_pipeline_join
        _host_pipeline_join(self)
