"""Host-side logic of the column-sharded GEMM, on CPU ranks over gloo (world size 2 and 4).

The GPU kernel is replaced by the CPU oracle here (no GPU in this test); what is under test is
the partitioning, the per-rank weight re-packing, the all-gather re-interleave and that the
sharded result equals the unsharded one bit for bit (each output column is computed by the same
K-ordered accumulation whichever rank owns it).
"""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    from numr_b200 import sharding
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k, n = 96, 80, 64 * world
        rng = np.random.default_rng(4)                       # same stream on every rank
        x = rng.standard_normal((m, k)).astype(np.float32)
        w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
        w_shard = sharding.pack_weight_shard(torch.from_numpy(w), world, rank)
        assert w_shard.is_contiguous() and tuple(w_shard.shape) == (k, n // world)
        cols = sharding.column_range(n, world, rank)
        assert np.array_equal(w_shard.numpy(), w[:, cols])
        # this rank's block, silu(X @ W_r), through the CPU restatement of the op
        y_shard = torch.from_numpy(O.gemm(O.F32, x, np.ascontiguousarray(w_shard.numpy()), act=O.ACT_SILU, threads=1))
        full = sharding.all_gather_columns(y_shard)
        assert tuple(full.shape) == (m, n)
        want = O.gemm(O.F32, x, w, act=O.ACT_SILU, threads=1)
        assert np.array_equal(full.numpy(), want), "sharded result differs from the unsharded one"
        # the max-over-ranks timing reduction the benchmark uses
        t = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        dist.barrier()
        Path(out_dir, f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_column_sharded_gemm_over_gloo(world, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert sorted(p.name for p in tmp_path.iterdir()) == [f"ok{r}" for r in range(world)]


def test_partition_rules():
    sys.path.insert(0, str(ROOT))
    from numr_b200 import sharding
    assert sharding.column_range(14336, 8, 0) == slice(0, 1792)
    assert sharding.column_range(14336, 8, 7) == slice(12544, 14336)
    assert sharding.column_range(14336, 1, 0) == slice(0, 14336)
    with pytest.raises(ValueError):
        sharding.column_range(14336, 3, 0)
    with pytest.raises(ValueError):
        sharding.column_range(14336, 8, 8)
    blocks = [torch.full((2, 3), float(r)) for r in range(4)]
    full = sharding.unshard_columns(blocks)
    assert tuple(full.shape) == (2, 12) and full[0].tolist() == [0.0] * 3 + [1.0] * 3 + [2.0] * 3 + [3.0] * 3
