"""Expert-parallel dispatch / combine logic on CPU ranks (gloo, world_size 2 and 4).

The exchange code of ExpertParallelLayer is run unchanged; only its three device steps
(route, local experts, combine) are replaced by the CPU oracle, so the test checks the index
bookkeeping and the all-to-all plumbing: every rank must get, for its own positions, exactly
what the single-process reference computes with all experts present.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_experts, dim, ff, top_k, T, out_dir, exchange):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import oracle
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.expert_parallel import ExpertParallelLayer, route_plan

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = oracle.load()
    router = synth.router_weights(7, n_experts, dim)
    gate = synth.expert_slabs(7, n_experts, ff, dim, 21)
    up = synth.expert_slabs(7, n_experts, ff, dim, 22)
    down = synth.expert_slabs(7, n_experts, dim, ff, 23)
    per = n_experts // world
    gu, dn = ff * (dim // 32) * 34, dim * (ff // 32) * 34

    class OracleLayer(ExpertParallelLayer):
        def _route(self, x, experts, weights, counts):
            _, e, w, _, c = orc.moe_route(router, x.numpy(), top_k)
            experts.copy_(torch.from_numpy(e)); weights.copy_(torch.from_numpy(w)); counts.copy_(torch.from_numpy(c))

        def _local_experts(self, rows, expert_ids, route_weights, out):
            lo = self.rank * per
            ids = expert_ids.numpy().reshape(-1, 1) - lo
            assert ids.min() >= 0 and ids.max() < per, "a route was sent to the wrong rank"
            res = orc.moe_experts(gate[lo * gu:(lo + per) * gu], up[lo * gu:(lo + per) * gu], down[lo * dn:(lo + per) * dn],
                                  per, dim, ff, rows.numpy(), ids.astype(np.int32), route_weights.numpy().reshape(-1, 1))
            out.copy_(torch.from_numpy(res))

        def _local_partial(self, x_all, experts_all, weights_all, out):
            lo = self.rank * per
            e = experts_all.numpy().astype(np.int64)
            w = weights_all.numpy().copy()
            local = (e >= lo) & (e < lo + per)
            res = np.zeros(out.shape, dtype=np.float32)
            for t in range(e.shape[0]):       # only this rank's routes, in selection order
                js = np.nonzero(local[t])[0]
                if js.size:
                    res[t] = orc.moe_experts(gate[lo * gu:(lo + per) * gu], up[lo * gu:(lo + per) * gu],
                                             down[lo * dn:(lo + per) * dn], per, dim, ff, x_all.numpy()[t:t + 1],
                                             (e[t:t + 1, js] - lo).astype(np.int32), w[t:t + 1, js])
            out.copy_(torch.from_numpy(res))

        def _combine(self, per_route, y, accumulate):
            acc = np.zeros(y.shape, dtype=np.float32)
            for j in range(per_route.shape[0]):
                acc = (acc + per_route[j].numpy()).astype(np.float32)
            y.copy_(torch.from_numpy(acc) + (y if accumulate else 0))

    layer = OracleLayer(None, None, None, None, None, n_experts, dim, ff, top_k, rank, world, exchange=exchange)
    x = synth.activations(100 + rank, (T, dim))
    y = torch.zeros((T, dim))
    experts, weights = layer.forward(torch.from_numpy(x), y)
    want, w_experts, w_weights, _ = orc.moe_layer(router, gate, up, down, ff, x, top_k)
    ok = np.array_equal(experts.numpy(), w_experts) and np.array_equal(weights.numpy(), w_weights)
    if exchange == "alltoall":  # rows come back per route and are added in selection order: same bits
        ok = ok and np.array_equal(y.numpy().view(np.uint32), want.view(np.uint32))
    else:                       # partial sums per rank are added by the collective: same value to f32 rounding
        ok = ok and float(np.abs(y.numpy() - want).max()) <= 1e-5 * float(np.abs(want).max())
    # the integer plan: destinations are the owning ranks, permutation is stable
    dest, order, counts = route_plan(experts, n_experts, world)
    ok = ok and bool((dest == experts.reshape(-1) // per).all()) and int(counts.sum()) == T * top_k
    ok = ok and bool((dest[order][1:] >= dest[order][:-1]).all())
    open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["alltoall", "gather"])
@pytest.mark.parametrize("world,n_experts,top_k,T", [(2, 8, 2, 5), (4, 16, 4, 7), (2, 4, 4, 3)])
def test_dispatch_and_combine_reproduce_the_single_process_layer(tmp_path, world, n_experts, top_k, T, exchange):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(world, port, n_experts, 64, 32, top_k, T, str(tmp_path), exchange), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok", f"rank {r}"
