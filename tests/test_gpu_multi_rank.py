"""Multi-GPU path on real GPUs: the row-sharded producer with its in-kernel exchange feeding column-sharded
GEMMs, one process per GPU (tests/multi_rank_worker.py).  Needs at least two GPUs; the CPU-side logic of the
shard helpers is covered by tests/test_multi_rank_cpu.py."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_row_sharded_producer_exchange_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29577", str(ROOT / "tests" / "multi_rank_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "MULTI_RANK_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
