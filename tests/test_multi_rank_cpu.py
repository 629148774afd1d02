"""The N > 1 host logic on CPU: two gloo ranks shard a weight by columns on
scale-group boundaries, run the oracle on their shard, all-gather, and must
reproduce the unsharded oracle result exactly; the producer's row shards tile
the rows on 128-row boundaries."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "flashrt-hf-kernels_b200" / "torch-ext" / "flashrt_b200_core"))

import sharding  # noqa: E402
from oracle import nvfp4_oracle as O  # noqa: E402


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 48, 512, 256
        rng = np.random.default_rng(0)                      # same bytes on every rank
        ap = rng.integers(0, 256, (m, k // 2), dtype=np.uint8)
        bp = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
        al = rng.integers(32, 80, (m, k // 16), dtype=np.uint8)
        bl = rng.integers(32, 80, (n, k // 16), dtype=np.uint8)
        b_swz = O.sf_linear_to_swizzled(bl)
        lo, hi = sharding.column_shard_bounds(n, world, rank)
        bp_loc, sf_loc = sharding.shard_weight(torch.from_numpy(bp), torch.from_numpy(b_swz), n, k, world, rank)
        # the contiguous scale slice IS the swizzle of the shard's linear scales
        np.testing.assert_array_equal(sf_loc.numpy(), O.sf_linear_to_swizzled(bl[lo:hi]))
        out_loc = O.gemm_bf16(ap, al, bp_loc.numpy(), O.sf_swizzled_to_linear(sf_loc.numpy(), hi - lo, k), alpha=0.5)
        full = sharding.gather_columns(dist, out_loc, world)
        want = O.gemm_bf16(ap, al, bp, bl, alpha=0.5)
        assert torch.equal(full, want)
        # the max-over-ranks timing reduction the benchmark uses
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
        if rank == 0:
            Path(tmp).write_text("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_column_sharded_gemm(tmp_path):
    flag = tmp_path / "done"
    mp.spawn(_worker, args=(2, 29591, str(flag)), nprocs=2, join=True)
    assert flag.read_text() == "ok"


def test_row_shards_tile_the_rows():
    for m in (128, 4096, 1000, 130, 7):
        for world in (1, 2, 4, 8):
            spans = [sharding.row_shard_bounds(m, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(lo % 128 == 0 or lo == m for lo, _ in spans)
    try:
        sharding.column_shard_bounds(4096 + 128, 8, 0)
    except ValueError:
        pass
    else:
        raise AssertionError("column shard off a scale-group boundary must be refused")
