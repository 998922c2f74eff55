"""Expert parallelism over peer memory: the dispatch and combine exchanges are stores issued by the producing
kernels themselves (quantise-and-scatter into the owner's GEMM operand buffers; the down GEMM's epilogue into the
origin's per-slot buffer), with three flag barriers per call and no library collective or host synchronisation on
the data path.  See torch-tpu_b200/csrc/ep_p2p.cu for the kernels and include/b200moe.h for the C ABI.

``torch.distributed`` is used once, at construction, to exchange the 64-byte memory handles.  The reference has no
expert-parallel path (torch_tpu/csrc/distributed/c10d/ProcessGroupSCCL.cpp:714-743 is an equal-split all-to-all).
"""
import ctypes

import torch
import torch.distributed as dist

from . import lib as L
from . import ops


def _round_up(n, m):
    return (n + m - 1) // m * m


class _RawCuda:
    """Lets torch view a raw device range (``__cuda_array_interface__``) without copying."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerArena:
    """One zero-filled device allocation per rank, mapped into every rank of ``group`` (same node), carved into
    named regions.  ``table(name)`` is a device int64 array: entry r = address of rank r's region."""

    def __init__(self, regions, device, group=None):
        self.group, self.device = group, torch.device(device)
        self.N, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.offsets, off = {}, 0
        for name, nbytes in regions:
            self.offsets[name] = (off, nbytes)
            off = _round_up(off + nbytes, 256)
        self.nbytes = max(off, 256)
        lib = L.lib()
        p = ctypes.c_void_p()
        L.check(lib.b200moe_p2p_alloc(ctypes.byref(p), self.nbytes), "b200moe_p2p_alloc")
        self.base = p.value
        h = ctypes.create_string_buffer(64)
        L.check(lib.b200moe_p2p_export(h, ctypes.c_void_p(self.base)), "b200moe_p2p_export")
        handles = [None] * self.N
        dist.all_gather_object(handles, bytes(h.raw), group=group)
        self.peer_base, self._imported = [], []
        failed = 0
        for r, hb in enumerate(handles):
            if r == self.rank:
                self.peer_base.append(self.base)
                continue
            q = ctypes.c_void_p()
            rc = lib.b200moe_p2p_import(ctypes.byref(q), hb)
            if rc != 0:
                failed = rc
                break
            self.peer_base.append(q.value)
            self._imported.append(q.value)
        # every rank learns whether every mapping exists before anyone goes on (a rank that raised alone would
        # leave the others waiting for it)
        flag = torch.tensor([1 if failed else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        if int(flag.item()):
            for q in self._imported:
                lib.b200moe_p2p_release(ctypes.c_void_p(q))
            self._imported = []
            dist.barrier(group=group)
            lib.b200moe_p2p_free(ctypes.c_void_p(self.base))
            self.base = None
            raise RuntimeError("peer memory could not be mapped on every rank"
                               + (f" (this rank: {L.error_string(failed)})" if failed else ""))
        self._whole = torch.as_tensor(_RawCuda(self.base, self.nbytes), device=self.device)
        self._tables = {name: torch.tensor([b + o for b in self.peer_base], dtype=torch.int64, device=self.device)
                        for name, (o, _) in self.offsets.items()}
        dist.barrier(group=group)   # nobody stores into a peer before every mapping exists

    def table(self, name):
        return self._tables[name]

    def local(self, name, dtype, shape):
        o, n = self.offsets[name]
        return self._whole[o:o + n].view(dtype).view(*shape)

    def close(self):
        """Unmap the peers' memory, wait until every rank has done so, free the own allocation."""
        if self.base is None:
            return
        torch.cuda.synchronize(self.device)
        lib = L.lib()
        for q in self._imported:
            lib.b200moe_p2p_release(ctypes.c_void_p(q))
        self._imported = []
        dist.barrier(group=self.group)
        self._whole = None
        lib.b200moe_p2p_free(ctypes.c_void_p(self.base))
        self.base = None


class P2PFusedMoE:
    """Expert-parallel MoE layer over peer memory.  ``layer`` is a FusedMoE holding the replicated router and the
    LOCAL expert shard (rank r owns experts [r*E/N, (r+1)*E/N)); every rank may pass up to ``max_tokens`` tokens per
    call.  Capacity is the worst case (every row of every rank routed to one rank), so no row is ever dropped."""

    def __init__(self, layer, num_experts_global: int, max_tokens: int, group=None):
        self.layer, self.E, self.group = layer, num_experts_global, group
        self.N, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.N > 8:
            raise ValueError("peer-memory expert parallelism spans one node: at most 8 ranks")
        if num_experts_global % self.N:
            raise ValueError("the number of experts must be divisible by the number of ranks")
        self.El = num_experts_global // self.N
        cfg = layer.cfg
        self.H, self.k, self.max_tokens = cfg.hidden, cfg.top_k, max_tokens
        self.dev = torch.device(layer.device)
        self.cap = self.N * max_tokens * self.k
        self.ld = _round_up(self.cap, 128)
        nH = self.H // 128
        self.arena = PeerArena([("flags", 256), ("cnt", self.N * self.E * 4), ("xq", self.cap * self.H),
                                ("xs_rows", self.cap * nH * 4), ("src", self.cap * 4),
                                ("y", max_tokens * self.k * self.H * 2)], self.dev, group)
        a = self.arena
        self.cnt = a.local("cnt", torch.int32, (self.N, self.E))
        self.xq = a.local("xq", torch.uint8, (self.cap, self.H))
        self.xs_rows = a.local("xs_rows", torch.float32, (self.cap, nH))
        self.xs = torch.empty(nH, self.ld, dtype=torch.float32, device=self.dev)   # local: the GEMMs' layout
        self.src = a.local("src", torch.int32, (self.cap,))
        self.y = a.local("y", torch.bfloat16, (max_tokens, self.k, self.H))
        self.dst_row0 = torch.empty(self.E, dtype=torch.int32, device=self.dev)
        self.recv_offsets = torch.empty(self.El + 1, dtype=torch.int32, device=self.dev)
        wg, sg = layer.w[0], layer.w[3]
        self.I = wg.shape[1]
        need = ops.grouped_mlp_workspace_bytes(self.cap, self.H, self.I, self.El, self.ld, sg.dtype)
        self.workspace = torch.empty(need + 256, dtype=torch.uint8, device=self.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.epoch = 0
        self.epoch_dev = None      # device-side epoch counter: set by enable_graphs(), see there
        self._static = None        # buffers of the allocation-free (graph-capturable) form of forward()
        self.phase_events = None   # set to [] to have forward() record (name, event) after every phase
        # > 0: the shared expert runs on a side stream beside routing and dispatch, its GEMMs capped at this many
        # CTAs (the dispatch is bound by the links and needs few SMs); 0: in line, on every SM, after the dispatch.
        # Two thirds of the SMs measured best at the DeepSeek-V3 shape (3.24 against 3.38 ms per step on 2 GPUs).
        self.shared_ctas = 2 * torch.cuda.get_device_properties(self.dev).multi_processor_count // 3
        self._side = None

    def _next_epoch(self):
        self.epoch = (self.epoch + 1) & 0xFFFFFFFF
        return ctypes.c_uint32(self.epoch)

    def _mark(self, name):
        if self.phase_events is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.phase_events.append((name, e))

    def forward(self, x, out=None):
        """x bf16 [T,H] on the device -> bf16 [T,H] (``out`` if given, else a buffer of this object / a new tensor)."""
        layer, a, lib = self.layer, self.arena, L.lib()
        T, H = x.shape
        if T > self.max_tokens or H != self.H:
            raise ValueError("x must be [T <= max_tokens, hidden]")
        N, rank, E = self.N, self.rank, self.E
        p, st = ops._ptr, ops._stream
        self._mark("start")
        add, out1 = None, None
        if layer.shared is not None:                               # buffers of the shared expert's pass
            if self._static is None:
                out1 = torch.empty(T, 1, H, dtype=torch.bfloat16, device=x.device)
                ids0 = torch.zeros(T, 1, dtype=torch.int32, device=x.device)
                shared_ws = None
            else:
                out1, ids0, shared_ws = (self._static["shared_out"][:T], self._static["zero_ids"][:T],
                                         self._static["shared_ws"])
        beside = layer.shared is not None and self.shared_ctas > 0
        if beside:
            # The shared expert needs nothing but x: it runs beside routing, permutation and dispatch on part of the
            # SMs (a fork/join of two streams, capturable); the grouped GEMMs, which want every SM, wait for it.
            # The fork has to come first: a persistent CTA of the GEMMs needs a whole SM, and once the dispatch's
            # many small blocks are spread over every SM it finds none until they have drained (forked after the
            # router, the join waited 0.35 ms for a shared expert that had only started after the dispatch).
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.dev)
            self._side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side):
                ops.experts(out1, x, *layer.shared, ids0, workspace=shared_ws, max_ctas=self.shared_ctas)
            add = out1.view(T, H)
        ids, w = layer.route(x)                                    # ids over GLOBAL experts
        if self._static is None:
            sorted_pair, offsets = ops.permute(ids, E, status=self.status)
        else:                                                      # graph mode: nothing is allocated per call
            sorted_pair, offsets = self._static["sorted_pair"][:T * self.k], self._static["offsets"]
            L.check(lib.b200moe_permute(p(sorted_pair), p(offsets), p(ids), T, self.k, E, p(self._static["scratch"]),
                                        p(self.status), st()), "b200moe_permute")
        self._mark("route+permute")
        L.check(lib.b200moe_ep_exchange_counts(p(a.table("cnt")), p(a.table("flags")), p(offsets), E, N, rank,
                                               self._next_epoch(), p(self.epoch_dev), p(self.status), st()),
                "b200moe_ep_exchange_counts")
        L.check(lib.b200moe_ep_plan(p(self.dst_row0), p(self.recv_offsets), p(self.cnt), E, N, rank, st()),
                "b200moe_ep_plan")
        self._mark("counts+plan")
        L.check(lib.b200moe_ep_dispatch(p(a.table("xq")), p(a.table("xs_rows")), p(a.table("src")), p(x),
                                        p(sorted_pair), p(ids), p(offsets), p(self.dst_row0), T, self.k, H, E, N, rank,
                                        self.cap, p(self.status), st()), "b200moe_ep_dispatch")
        self._mark("dispatch")
        if layer.shared is not None and not beside:
            # in line: between this rank's dispatch and the barrier, so that the wait for the slowest sender passes
            # under it instead of leaving the SMs idle
            ops.experts(out1, x, *layer.shared, ids0, workspace=shared_ws)
            add = out1.view(T, H)
            self._mark("shared")
        L.check(lib.b200moe_p2p_barrier(p(a.table("flags")), N, rank, self._next_epoch(), p(self.epoch_dev),
                                        p(self.status), st()), "b200moe_p2p_barrier")
        self._mark("barrier")
        if beside:
            torch.cuda.current_stream().wait_stream(self._side)
            self._mark("shared (join)")
        L.check(lib.b200moe_ep_transpose_scales(p(self.xs), self.ld, p(self.xs_rows), p(self.recv_offsets[self.El:]),
                                                H, self.cap, st()), "b200moe_ep_transpose_scales")
        wg, wu, wd, sg, su, sd = layer.w
        base = (self.workspace.data_ptr() + 255) // 256 * 256
        avail = self.workspace.numel() - (base - self.workspace.data_ptr())
        L.check(lib.b200moe_grouped_mlp_remote(p(a.table("y")), p(self.src), p(self.xq), p(self.xs), self.ld,
                                               p(self.recv_offsets), p(wg), p(wu), p(wd), p(sg), p(su), p(sd),
                                               ops._DT[sg.dtype], self.cap, H, self.I, self.El,
                                               ctypes.c_void_p(base), avail, p(self.status), st()),
                "b200moe_grouped_mlp_remote")
        self._mark("grouped_mlp")
        L.check(lib.b200moe_p2p_barrier(p(a.table("flags")), N, rank, self._next_epoch(), p(self.epoch_dev),
                                        p(self.status), st()), "b200moe_p2p_barrier")
        self._mark("barrier2")
        # slots whose expert id was out of range were never dispatched: their rows of y hold nothing and are skipped
        out = ops.combine_indexed(self.y[:T].view(T * self.k, H), None, w, add=add, ids=ids, num_experts=E,
                                  out=out if out is not None else
                                  (None if self._static is None else self._static["out"][:T]))
        self._mark("combine")
        return out

    __call__ = forward

    def enable_graphs(self):
        """Switch to the allocation-free form of forward(): every buffer is made once here, and the barriers count
        their epochs in a device word instead of taking them from the host, so that a call holds no per-call value
        and can be captured into a CUDA graph.  Every rank of the group must switch at the same point of its call
        sequence (the device counter starts from the host's current epoch)."""
        if self._static is not None:
            return
        dev, T, k, H, E = self.dev, self.max_tokens, self.k, self.H, self.E
        st = dict(sorted_pair=torch.empty(T * k, dtype=torch.int32, device=dev),
                  offsets=torch.empty(E + 1, dtype=torch.int32, device=dev),
                  scratch=torch.empty(max(1, L.lib().b200moe_permute_scratch_ints(T * k, E)), dtype=torch.int32,
                                      device=dev),
                  out=torch.empty(T, H, dtype=torch.bfloat16, device=dev),
                  x=torch.empty(T, H, dtype=torch.bfloat16, device=dev))
        if self.layer.shared is not None:
            Is = self.layer.shared[0].shape[-2]
            d = ops.make_desc(T, H, Is, 1, 1, out_mode=L.OUT_PER_SLOT, scale_dtype=self.layer.shared[3].dtype)
            st.update(shared_out=torch.empty(T, 1, H, dtype=torch.bfloat16, device=dev),
                      zero_ids=torch.zeros(T, 1, dtype=torch.int32, device=dev),
                      shared_ws=torch.empty(ops.experts_workspace_bytes(d) + 256, dtype=torch.uint8, device=dev))
        self.epoch_dev = torch.tensor([self.epoch], dtype=torch.int32, device=dev)
        self._static, self._graphs = st, {}

    def capture(self, T: int):
        """Capture forward() for exactly T tokens per rank into a CUDA graph (every rank captures and later replays
        the same sequence; the flag barriers inside the graph keep the ranks in step)."""
        self.enable_graphs()
        x_static = self._static["x"][:T]
        side = torch.cuda.Stream(device=self.dev)
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
        if self._static is None or T not in self._graphs:
            self.capture(T)
        g, y = self._graphs[T]
        self._static["x"][:T].copy_(x, non_blocking=True)
        g.replay()
        return y

    def forward_host(self, x_host, out_host):
        """Host-buffer entry point, pipelined like FusedMoE.forward_host."""
        from .layer import _host_pipeline_call
        return _host_pipeline_call(self, self.forward, x_host, out_host)

    def host_join(self):
        from .layer import _host_pipeline_join
        _host_pipeline_join(self)

    def close(self):
        self.arena.close()
