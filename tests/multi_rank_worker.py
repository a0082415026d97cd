"""One rank of the multi-GPU parity test (launched by test_gpu_multi_rank.py through
torch.distributed.run, one rank per GPU, NCCL). Every rank computes; rank 0 checks against the CPU
oracle and against its own single-GPU layer and prints one JSON line. Exit code 0 = parity holds."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

TOL = 2e-3


def max_rel_err(got, want):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    den = np.maximum(np.abs(want), np.sqrt((want ** 2).mean()))
    return float((np.abs(got - want) / den).max())


def main():
    import torch
    import torch.distributed as dist

    import oracle
    from exec_beholdd_b200 import CudaDevice, Weight, synth
    from exec_beholdd_b200.expert_parallel import ExpertParallelLayer
    from exec_beholdd_b200.row_parallel import RowSplitLinear

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    dev = CudaDevice(local)
    orc = oracle.load()
    report, ok = {"world": world}, True
    ne, dim, ff, k, seed = 128, 2048, 768, 8, 31

    # ---- routed layer, experts split over the ranks ------------------------------------------
    single = ExpertParallelLayer.from_synthetic(dev, seed, ne, dim, ff, k) if rank == 0 else None
    host = None
    if rank == 0:  # the same per-expert bytes as from_synthetic, for the oracle
        cat = lambda stream, rows, cols: np.concatenate([synth.q8_0_matrix(seed, rows, cols, stream=stream * 1000 + e) for e in range(ne)])
        host = (synth.router_weights(seed, ne, dim), cat(21, ff, dim), cat(22, ff, dim), cat(23, dim, ff))
    for T in (1, 16, 40):
        x_np = synth.activations(seed + 5 + 100 * rank, (T, dim), outliers=True)
        x = torch.from_numpy(x_np).cuda()
        x_all = torch.empty((world * T, dim), device="cuda")
        dist.all_gather_into_tensor(x_all, x)
        want_single = want_oracle = None
        if rank == 0:
            y_all = torch.empty((world * T, dim), device="cuda")
            single.forward(x_all, y_all)
            want_single = y_all[:T].clone()
            want_oracle, experts_o, _, _ = orc.moe_layer(host[0], host[1], host[2], host[3], ff, x_np, k)
        for exchange in [v for v in os.environ.get("BHD_TEST_EXCHANGES", "peer,alltoall,gather").split(",") if v]:
            layer = ExpertParallelLayer.from_synthetic(dev, seed, ne, dim, ff, k, rank, world, exchange=exchange)
            y = torch.full((T, dim), float("nan"), device="cuda")
            for _ in range(2):  # twice: buffers and flags of the first call are reused by the second
                experts, _ = layer.forward(x, y)
            torch.cuda.synchronize()
            dev.check_status()
            if rank == 0:
                e_or = max_rel_err(y.cpu().numpy(), want_oracle)
                same = bool(torch.equal(y, want_single))
                idx = bool(np.array_equal(experts.cpu().numpy(), experts_o))
                good = e_or <= TOL and idx and (same or not layer.bit_identical)
                report[f"moe_T{T}_{exchange}"] = {"max_rel_err_vs_oracle": e_or, "bit_identical_to_single_gpu": same,
                                                  "indices_exact": idx, "ok": good}
                ok &= good
            layer.free()
    if single is not None:
        single.free()

    # ---- large projection, rows split over the ranks -------------------------------------------
    rows, cols = 12288, 4096
    for kind, batch in ((12, 1), (12, 4), (8, 2), (14, 1)):
        packed = synth.matrix(kind, seed + kind, rows, cols)
        lin = RowSplitLinear.from_host(dev, packed, kind, rows, cols, rank, world)
        x_np = synth.activations(seed + 9, (batch, cols))
        x = torch.from_numpy(x_np).cuda()
        y = torch.full((batch, rows), float("nan"), device="cuda")
        for _ in range(2):
            lin.forward(x, y)
        torch.cuda.synchronize()
        dev.check_status()
        if rank == 0:
            picks = np.arange(0, rows, 257)
            rb = synth.packed_bytes(kind, 1, cols)
            sub = np.ascontiguousarray(packed.reshape(rows, rb)[picks]).reshape(-1)
            err = max_rel_err(y.cpu().numpy()[:, picks], orc.matvec_batch(sub, kind, len(picks), cols, x_np))
            good = err <= TOL and bool(torch.isfinite(y).all())
            report[f"row_split_kind{kind}_b{batch}"] = {"max_rel_err_vs_oracle": err, "ok": good}
            ok &= good
        lin.free()

    flag = torch.tensor([0 if ok else 1], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if rank == 0:
        report["ok"] = bool(ok)
        print("MULTI_RANK_REPORT " + json.dumps(report), flush=True)
    dev.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    import faulthandler

    faulthandler.enable()
    main()
