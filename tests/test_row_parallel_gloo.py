"""Row-split dense projection on CPU ranks (gloo, world_size 2 and 4).

RowSplitLinear's exchange code runs unchanged; only its device step is replaced by the CPU
oracle on the rank's shard. Row splitting keeps every packed row whole, so each rank must end
with exactly the bits the single-process matvec produces for the full matrix.
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


def _worker(rank, world, port, kind, rows, cols, batch, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import oracle
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.row_parallel import RowSplitLinear, shard_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = oracle.load()
    packed = synth.matrix(kind, 11, rows, cols)
    mine = shard_rows(packed, kind, rows, cols, rank, world)

    class OracleLinear(RowSplitLinear):
        def _local(self, x, y_local):
            y_local.copy_(torch.from_numpy(orc.matvec_batch(mine, kind, rows // world, cols, x.numpy())))

    lin = OracleLinear(None, None, rows, cols, rank, world, exchange="all_gather")
    x = synth.activations(5, (batch, cols))          # the same activations on every rank
    y = torch.full((batch, rows), float("nan"))
    lin.forward(torch.from_numpy(x), y)
    want = orc.matvec_batch(packed, kind, rows, cols, x)
    ok = np.array_equal(y.numpy().view(np.uint32), want.view(np.uint32))
    open(os.path.join(out_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    dist.destroy_process_group()


@pytest.mark.parametrize("world,kind,rows,cols,batch", [(2, 12, 64, 512, 1), (2, 8, 96, 256, 3), (4, 14, 64, 256, 2)])
def test_row_split_reproduces_the_single_process_matvec_bit_for_bit(tmp_path, world, kind, rows, cols, batch):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(world, port, kind, rows, cols, batch, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "ok", f"rank {r}"


def test_rows_that_do_not_split_evenly_are_refused():
    sys.path.insert(0, ROOT)
    from exec_beholdd_b200 import synth
    from exec_beholdd_b200.row_parallel import RowSplitLinear, shard_rows

    packed = synth.matrix(8, 3, 10, 64)
    with pytest.raises(ValueError):
        shard_rows(packed, 8, 10, 64, 0, 4)
    with pytest.raises(ValueError):
        RowSplitLinear(None, None, 10, 64, 0, 4)
