"""Row-split execution of one large dense projection across the GPUs of one node.

The reference is single-process; its projections are `Device::matvec` calls over a whole
row-major weight (crates/beholdd-backend/src/lib.rs:182-198, cpu.rs:415-507). Output rows are
independent, so the weight splits by rows without touching the arithmetic of any row:

  * rank r holds rows [r*N/P, (r+1)*N/P) of the packed weight, whole packed rows each (no
    split along the columns, hence no cross-GPU reduction and no change of summation order);
  * every rank has the full activation vector(s), computes its slice of y, and one all-gather
    assembles y on every rank.

No row's sum crosses a GPU. Two exchanges: "peer" (default) lets one library kernel after the matvec store
the slice into every rank's y over NVLink peer memory, signal and wait (no collective library, capturable
into a CUDA graph); "all_gather" is one NCCL all-gather, whose latency at decode sizes (48 KB of y for
N = 12288) exceeds the matvec itself.

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

    def __init__(self, dev, shard, rows: int, cols: int, rank: int = 0, world: int = 1, group=None, exchange: str = "peer"):
        """`exchange`: "peer" = the library's kernel stores every slice into every rank's y over peer memory
        (bhd_rowsplit_*, capturable into a CUDA graph); "all_gather" = one NCCL all-gather."""
        if rows % world:
            raise ValueError(f"{rows} rows do not split evenly over {world} ranks")
        assert exchange in ("peer", "all_gather")
        self.dev, self.shard = dev, shard
        self.rows, self.cols, self.rank, self.world, self.group = rows, cols, rank, world, group
        self.per = rows // world
        self.exchange = exchange
        self._rs = None
        self._rs_batch = 0

    @property
    def capturable(self) -> bool:
        """Whether forward() can be captured into a CUDA graph."""
        return self.world == 1 or self.exchange == "peer"

    @classmethod
    def from_host(cls, dev, packed: np.ndarray, kind: int, rows: int, cols: int, rank: int = 0, world: int = 1, group=None,
                  exchange: str = "peer"):
        """Upload only this rank's rows of a host-resident packed weight."""
        from .device import Weight

        mine = shard_rows(packed, kind, rows, cols, rank, world)
        shard = dev.upload_weight(Weight(np.ascontiguousarray(mine), kind, rows // world, cols))
        return cls(dev, shard, rows, cols, rank, world, group, exchange)

    def _peer_exchange(self, batch: int):
        """The library's exchange object, created on first use; the 64-byte handles of the ranks' blocks travel
        through the process group."""
        import ctypes as C

        import torch
        import torch.distributed as dist

        if self._rs is not None and batch <= self._rs_batch:
            return self._rs
        self._free_peer_exchange()
        lib = self.dev.lib
        handle = (C.c_uint8 * 64)()
        rs = C.c_void_p()
        self.dev._check(lib.bhd_rowsplit_create(self.dev.ctx, self.rank, self.world, self.rows, max(batch, 8), C.byref(rs), handle))
        mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda" if dist.get_backend(self.group) == "nccl" else "cpu")
        everyone = torch.empty((self.world, 64), dtype=torch.uint8, device=mine.device)
        dist.all_gather_into_tensor(everyone.view(-1), mine, group=self.group)
        self.dev._check(lib.bhd_rowsplit_connect(rs, C.c_char_p(bytes(everyone.cpu().numpy().reshape(-1).tolist()))))
        dist.barrier(group=self.group)  # every rank has mapped every block before anyone writes
        self._rs, self._rs_batch = rs, max(batch, 8)
        return rs

    def _free_peer_exchange(self):
        if self._rs is not None:
            import torch
            import torch.distributed as dist

            torch.cuda.synchronize()
            dist.barrier(group=self.group)  # nobody still writes into a block that is about to go
            self.dev.lib.bhd_rowsplit_destroy(self._rs)
            self._rs = None

    def free(self):
        self._free_peer_exchange()
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

        if self.exchange == "peer":
            rs = self._peer_exchange(B)
            self.dev._check(self.dev.lib.bhd_rowsplit_matvec(rs, self.shard.handle, 0, x.data_ptr(), y.data_ptr(), B, 1.0,
                                                             self.dev._stream()))
            return y
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
