"""Row-split execution of one large dense projection across the GPUs of one node.

The reference is single-process; its projections are `Device::matvec` calls over a whole
row-major weight (crates/beholdd-backend/src/lib.rs:182-198, cpu.rs:415-507). Output rows are
independent, so the weight splits by rows without touching the arithmetic of any row:

  * rank r holds rows [r*N/P, (r+1)*N/P) of the packed weight, whole packed rows each (no
    split along the columns, hence no cross-GPU reduction and no change of summation order);
  * every rank has the full activation vector(s), computes its slice of y, and one all-gather
    assembles y on every rank.

The result is bit-identical to the single-GPU result for every P. At decode the gathered slice
is N/P floats per rank (48 KB in total for N = 12288), so the collective's latency exceeds the
matvec itself; the class exists for weights that do not fit one GPU and for prefill, and the
benchmark reports the gathered time as it is.

The compute step is a replaceable method so that the exchange logic is testable with gloo on
CPU ranks.
"""
from __future__ import annotations

import numpy as np


def shard_rows(packed: np.ndarray, kind: int, rows: int, cols: int, rank: int, world: int) -> np.ndarray:
    """The packed bytes of this rank's rows (rows must divide evenly: packed rows stay whole)."""
    from . import synth

    if rows % world:
        raise ValueError(f"{rows} rows do not split evenly over {world} ranks")
    row_bytes = synth.packed_bytes(kind, 1, cols)
    per = rows // world
    flat = packed.reshape(-1)
    if flat.size != rows * row_bytes:
        raise ValueError(f"expected {rows * row_bytes} packed bytes, got {flat.size}")
    return flat[rank * per * row_bytes:(rank + 1) * per * row_bytes]


class RowSplitLinear:
    """y = W x with W's rows split over `world` ranks; every rank ends with the whole y."""

    def __init__(self, dev, shard, rows: int, cols: int, rank: int = 0, world: int = 1, group=None):
        if rows % world:
            raise ValueError(f"{rows} rows do not split evenly over {world} ranks")
        self.dev, self.shard = dev, shard
        self.rows, self.cols, self.rank, self.world, self.group = rows, cols, rank, world, group
        self.per = rows // world

    #: how the slices of y travel, and whether forward() can be captured into a CUDA graph
    exchange = "all_gather (NCCL)"

    @property
    def capturable(self) -> bool:
        return self.world == 1

    @classmethod
    def from_host(cls, dev, packed: np.ndarray, kind: int, rows: int, cols: int, rank: int = 0, world: int = 1, group=None):
        """Upload only this rank's rows of a host-resident packed weight."""
        from .device import Weight

        mine = shard_rows(packed, kind, rows, cols, rank, world)
        shard = dev.upload_weight(Weight(np.ascontiguousarray(mine), kind, rows // world, cols))
        return cls(dev, shard, rows, cols, rank, world, group)

    def free(self):
        self.shard.free()

    # ---- the device step, replaceable in CPU tests -----------------------------------------
    def _local(self, x, y_local):
        """y_local[b, :] = W[rank's rows] @ x[b, :] for every activation row b."""
        if x.shape[0] <= 8:
            self.dev.matvec_resident(self.shard, x, y_local)
        else:
            self.dev.matmul_resident(self.shard, x, y_local)

    # ---- forward ---------------------------------------------------------------------------
    def forward(self, x, y):
        """x [B, cols] -> y [B, rows], both on this rank's device, y complete on every rank."""
        import torch

        B = x.shape[0]
        if self.world == 1:
            self._local(x, y)
            return y
        import torch.distributed as dist

        y_local = torch.empty((B, self.per), dtype=x.dtype, device=x.device)
        self._local(x, y_local)
        if B == 1:
            # rank-major order is row order: gather straight into y
            dist.all_gather_into_tensor(y.view(-1), y_local.view(-1), group=self.group)
            return y
        gathered = torch.empty((self.world, B, self.per), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(gathered.view(-1), y_local.view(-1), group=self.group)
        y.view(B, self.world, self.per).copy_(gathered.permute(1, 0, 2))
        return y
