"""Multi-GPU parity: the expert-parallel routed layer and the row-split projection on real NCCL
ranks, one process per GPU, checked against the CPU oracle and the single-GPU layer.

Skipped when fewer than two GPUs are visible. The ranks run tests/multi_rank_worker.py."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_and_row_split_parity_on_nccl_ranks(world):
    import torch

    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 29700 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "multi_rank_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    tail = (res.stdout + res.stderr)[-4000:]
    assert res.returncode == 0, tail
    lines = [l for l in res.stdout.splitlines() if l.startswith("MULTI_RANK_REPORT ")]
    assert lines, tail
    report = json.loads(lines[-1][len("MULTI_RANK_REPORT "):])
    print(json.dumps(report, indent=1))
    assert report["ok"], report
