"""Expert-parallel execution of the routed-expert layer across the GPUs of one node.

The reference is single-process and has no sharding (its routed block is
crates/beholdd-model/src/qwen3moe/forward.rs:1299-1407); this module adds the one exchange
step each way that splitting experts across ranks needs:

  * experts e in [r*E/N, (r+1)*E/N) live on rank r; the router weights are replicated;
  * every rank owns its own positions, routes them locally (bit-exact selection), and
    sends each route's input row to the rank that holds the selected expert
    (all-to-all-v "dispatch"), together with the expert id and the route weight;
  * the expert rank runs gate/up/SiLU/down for the rows it received and returns one output
    row per route, already scaled by the route weight (all-to-all-v "combine");
  * the owner adds the returned rows in selection order into a zeroed row, which is the
    reference's accumulation order, so the result does not depend on N.

Index bookkeeping (sorting routes by destination, split sizes) is done with torch on small
integer tensors; all arithmetic on activations runs in the CUDA library. The class takes
the process group and the compute callables as parameters so the exchange logic can be
tested with gloo on CPU ranks.
"""
from __future__ import annotations

import numpy as np


def route_plan(experts, n_experts: int, world: int):
    """For local routes experts[T, k] -> (dest rank per route, stable permutation that sorts
    routes by destination, per-destination counts). Pure integer work."""
    import torch

    per = n_experts // world
    flat = experts.reshape(-1).to(torch.int64)
    dest = torch.div(flat, per, rounding_mode="floor")
    order = torch.sort(dest, stable=True).indices
    counts = torch.bincount(dest, minlength=world)
    return dest, order, counts


class ExpertParallelLayer:
    """One routed-expert layer with experts split across `world` ranks."""

    def __init__(self, dev, router, gate, up, down, n_experts, dim, ff, top_k, rank=0, world=1, group=None,
                 exchange="gather", exchange_owner=None):
        """`exchange_owner`: another layer of the same shape whose peer-memory exchange this one uses (the layers of
        a model run one after the other, so one exchange block serves them all)."""
        self.dev, self.router, self.gate, self.up, self.down = dev, router, gate, up, down
        self.n_experts, self.dim, self.ff, self.top_k = n_experts, dim, ff, top_k
        self.rank, self.world, self.group = rank, world, group
        self.per = n_experts // world
        assert n_experts % world == 0
        assert exchange in ("gather", "alltoall", "peer")
        self.exchange = exchange
        self._ep = None        # the library's exchange object ("peer")
        self._ep_max_t = 0
        self._ep_owner = exchange_owner
        self.last_counts = None
        self._marks = None  # (name, event) pairs of an instrumented forward

    #: whether forward() can be captured into a CUDA graph (the NCCL exchanges here read split sizes on the host)
    @property
    def capturable(self) -> bool:
        return self.world == 1 or self.exchange == "peer"

    #: whether the result equals the single-GPU layer over the same global batch to the bit
    @property
    def bit_identical(self) -> bool:
        return self.world == 1 or self.exchange in ("alltoall", "peer")

    def _peer_exchange(self, T: int):
        """The library's peer-memory exchange (bhd_ep_*), created on first use for T positions per rank; the
        64-byte handles of the ranks' blocks travel through the process group."""
        import ctypes as C

        import torch
        import torch.distributed as dist

        if self._ep_owner is not None:
            return self._ep_owner._peer_exchange(T)
        if self._ep is not None and T <= self._ep_max_t:
            return self._ep
        self._free_peer_exchange()
        lib, ctx = self.dev.lib, self.dev.ctx
        handle = (C.c_uint8 * 64)()
        ep = C.c_void_p()
        self.dev._check(lib.bhd_ep_create(ctx, self.rank, self.world, self.n_experts, self.dim, self.top_k, T, C.byref(ep), handle))
        mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda" if dist.get_backend(self.group) == "nccl" else "cpu")
        everyone = torch.empty((self.world, 64), dtype=torch.uint8, device=mine.device)
        dist.all_gather_into_tensor(everyone.view(-1), mine, group=self.group)
        blob = bytes(everyone.cpu().numpy().reshape(-1).tolist())
        self.dev._check(lib.bhd_ep_connect(ep, C.c_char_p(blob)))
        dist.barrier(group=self.group)  # every rank has mapped every block before anyone writes
        self._ep, self._ep_max_t = ep, T
        return ep

    def _free_peer_exchange(self):
        if self._ep is not None:
            import torch
            import torch.distributed as dist

            torch.cuda.synchronize()
            dist.barrier(group=self.group)  # nobody still writes into a block that is about to go
            self.dev.lib.bhd_ep_destroy(self._ep)
            self._ep = None

    def _mark(self, name):
        if self._marks is not None:
            import torch

            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def timed_phases(self, x, y, repeats: int = 5):
        """Device time of each phase of forward() in microseconds (median over a few eager runs;
        the collectives are timed where the compute stream waits for them)."""
        import statistics

        import torch

        runs = []
        for _ in range(repeats + 1):
            self._marks = []
            self._mark("start")
            self.forward(x, y)
            self._mark("end")
            torch.cuda.synchronize()
            marks, self._marks = self._marks, None
            runs.append({b[0]: a[1].elapsed_time(b[1]) * 1e3 for a, b in zip(marks[:-1], marks[1:])})
        runs = runs[1:]  # the first run warms the allocator up
        return {k: round(statistics.median(r[k] for r in runs), 1) for k in runs[0]}

    @classmethod
    def from_synthetic(cls, dev, seed, n_experts, dim, ff, top_k, rank=0, world=1, group=None, exchange="gather"):
        """Seeded weights of the benchmark configuration; this rank uploads only its experts."""
        from . import synth
        from .device import Weight

        per = n_experts // world
        router = synth.router_weights(seed, n_experts, dim)
        gu_slab, d_slab = synth.packed_bytes(8, ff, dim), synth.packed_bytes(8, dim, ff)

        def local(stream, rows, cols, slab):
            # Expert slabs are generated per expert so that every rank sees the bytes the
            # single-GPU run sees for the same expert.
            parts = [synth.q8_0_matrix(seed, rows, cols, stream=stream * 1000 + e) for e in range(rank * per, (rank + 1) * per)]
            return np.concatenate(parts)

        return cls(dev, dev.upload_weight(Weight(router.view(np.uint8).reshape(-1), 0, n_experts, dim)),
                   dev.upload_weight(Weight(local(21, ff, dim, gu_slab), 8, ff, dim), slabs=per),
                   dev.upload_weight(Weight(local(22, ff, dim, gu_slab), 8, ff, dim), slabs=per),
                   dev.upload_weight(Weight(local(23, dim, ff, d_slab), 8, dim, ff), slabs=per),
                   n_experts, dim, ff, top_k, rank, world, group, exchange)

    def free(self):
        self._free_peer_exchange()
        for w in (self.router, self.gate, self.up, self.down):
            w.free()

    # ---- the two device steps, replaceable in CPU tests ------------------------------------
    def _route(self, x, experts, weights, counts):
        self.dev.moe_route(self.router, x, self.top_k, experts, weights, counts)

    def _local_experts(self, rows, expert_ids, route_weights, out):
        """rows [R, dim] each with one (global) expert id and weight -> out[r] = w * down(silu(gate)*up)."""
        self.dev.moe_experts(self.gate, self.up, self.down, rows, expert_ids.view(-1, 1), route_weights.view(-1, 1), out,
                             first_expert=self.rank * self.per, n_local=self.per, n_experts=self.n_experts)

    def _local_partial(self, x_all, experts_all, weights_all, out):
        """All positions of all ranks, only this rank's experts: out[t] = sum over the local
        routes of t, in selection order (routes of other ranks contribute nothing)."""
        self.dev.moe_experts(self.gate, self.up, self.down, x_all, experts_all, weights_all, out,
                             first_expert=self.rank * self.per, n_local=self.per, n_experts=self.n_experts)

    def _combine(self, per_route, y, accumulate):
        """per_route [k, T, dim] -> y[t] (+)= ((0 + r[0][t]) + r[1][t]) + ... in route order."""
        self.dev.moe_combine(per_route, y, accumulate)

    # ---- forward ---------------------------------------------------------------------------
    def forward(self, x, y, accumulate=False):
        import torch

        T = x.shape[0]
        experts = torch.empty((T, self.top_k), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, self.top_k), dtype=torch.float32, device=x.device)
        counts = torch.empty((self.n_experts,), dtype=torch.int32, device=x.device)
        if self.world == 1:
            self.dev.moe_layer(self.router, self.gate, self.up, self.down, x, y, self.top_k, experts, weights, counts,
                               accumulate=accumulate)
            self.last_counts = counts
            return experts, weights

        import torch.distributed as dist

        if self.exchange == "peer":
            ep = self._peer_exchange(T)
            self.dev._check(self.dev.lib.bhd_ep_layer(ep, self.router.handle, self.gate.handle, self.up.handle, self.down.handle,
                                                      x.data_ptr(), y.data_ptr(), T, experts.data_ptr(), weights.data_ptr(),
                                                      counts.data_ptr(), 1 if accumulate else 0, self.dev._stream()))
            self.last_counts = counts
            self._mark("layer")
            return experts, weights

        self._route(x, experts, weights, counts)
        self.last_counts = counts
        self._mark("route")
        if self.exchange == "gather":
            return self._forward_gather(x, y, experts, weights, accumulate)
        _, order, send_counts = route_plan(experts, self.n_experts, self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_list, recv_list = send_counts.tolist(), recv_counts.tolist()  # one host sync per layer
        n_recv = int(sum(recv_list))

        token_of_route = torch.div(order, self.top_k, rounding_mode="floor")
        rows_send = x.index_select(0, token_of_route)                       # dispatch gather
        # expert id and route weight (as raw bits) travel together, one int32 pair per route
        meta_send = torch.stack([experts.reshape(-1)[order], weights.reshape(-1)[order].view(torch.int32)],
                                dim=1).contiguous()
        rows_recv = torch.empty((n_recv, self.dim), dtype=x.dtype, device=x.device)
        meta_recv = torch.empty((n_recv, 2), dtype=torch.int32, device=x.device)
        dist.all_to_all_single(rows_recv, rows_send, recv_list, send_list, group=self.group)
        dist.all_to_all_single(meta_recv, meta_send, recv_list, send_list, group=self.group)
        self._mark("dispatch")

        out_recv = torch.empty((n_recv, self.dim), dtype=x.dtype, device=x.device)
        if n_recv:
            self._local_experts(rows_recv, meta_recv[:, 0].contiguous(), meta_recv[:, 1].contiguous().view(torch.float32),
                                out_recv)
        self._mark("experts")
        out_back = torch.empty((T * self.top_k, self.dim), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out_back, out_recv, send_list, recv_list, group=self.group)
        self._mark("return")

        # Un-permute into route-major [k, T, dim], then add in selection order.
        j_of_route = order % self.top_k
        slot = j_of_route * T + token_of_route
        per_route = torch.empty((self.top_k * T, self.dim), dtype=x.dtype, device=x.device)
        per_route.index_copy_(0, slot, out_back)
        self._combine(per_route.view(self.top_k, T, self.dim), y, accumulate)
        self._mark("combine")
        return experts, weights

    def _forward_gather(self, x, y, experts, weights, accumulate):
        """Exchange without a host round trip: all-gather the positions and their routes,
        every rank applies its own experts to all positions, reduce-scatter the partial
        outputs. Dispatch volume is the same order as the all-to-all (a position's 8 routes
        reach most ranks anyway) and nothing depends on counts known only on the device, so
        the whole layer stays asynchronous. The cross-rank sum is NCCL's reduction order, not
        the selection order: identical to the single-GPU result within f32 rounding."""
        import torch
        import torch.distributed as dist

        T, W = x.shape[0], self.world
        x_all = torch.empty((W * T, self.dim), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(x_all, x.contiguous(), group=self.group)
        meta = torch.cat([experts, weights.view(torch.int32)], dim=1).contiguous()
        meta_all = torch.empty((W * T, 2 * self.top_k), dtype=torch.int32, device=x.device)
        dist.all_gather_into_tensor(meta_all, meta, group=self.group)
        experts_all = meta_all[:, : self.top_k].contiguous()
        weights_all = meta_all[:, self.top_k:].contiguous().view(torch.float32)
        self._mark("all_gather")
        partial = torch.empty((W * T, self.dim), dtype=x.dtype, device=x.device)
        self._local_partial(x_all, experts_all, weights_all, partial)
        self._mark("experts")
        mine = torch.empty((T, self.dim), dtype=x.dtype, device=x.device) if accumulate else y
        if dist.get_backend(self.group) == "gloo":  # gloo has no reduce-scatter
            dist.all_reduce(partial, group=self.group)
            mine.copy_(partial[self.rank * T:(self.rank + 1) * T])
        else:
            dist.reduce_scatter_tensor(mine, partial, group=self.group)
        if accumulate:
            y.add_(mine)
        self._mark("reduce_scatter")
        return experts, weights
