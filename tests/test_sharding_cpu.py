"""The multi-GPU partitioning logic on CPU: pure partition arithmetic, and two gloo ranks that shard a
batched contraction by batch index (no collective) and a big GEMM by N-column slabs (+ all-gather),
with the CPU oracle standing in for the contraction (test infrastructure; the product default is the
CUDA kernels)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_batch_range_covers_everything_once():
    from nova_compiler_b200.sharding import batch_range
    for batch in (0, 1, 5, 32, 255, 256, 257):
        for world in (1, 2, 3, 4, 8):
            owned = []
            for r in range(world):
                s, c = batch_range(batch, world, r)
                owned += list(range(s, s + c))
            assert owned == list(range(batch))
            sizes = [batch_range(batch, world, r)[1] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        batch_range(4, 2, 2)


def test_column_slab_alignment_and_coverage():
    from nova_compiler_b200.sharding import column_slab
    for n in (0, 1, 63, 64, 1000, 11007, 16384):
        for world in (1, 2, 4, 8):
            cols = []
            for r in range(world):
                s, c = column_slab(n, world, r)
                assert s % 64 == 0 or c == 0
                cols += list(range(s, s + c))
            assert cols == list(range(n))
    assert column_slab(16384, 8, 3) == (6144, 2048)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nova_compiler_b200 import sharding
    from oracle import oracle as O

    def cpu_matmul(a, b, **kw):  # the oracle as the contraction on CPU ranks
        return torch.from_numpy(O.gemm(a.contiguous().numpy(), b.contiguous().numpy()))

    g = torch.Generator().manual_seed(1234)  # same data on both ranks
    a = torch.rand(5, 24, 40, generator=g) * 2 - 1
    b = torch.rand(5, 40, 16, generator=g) * 2 - 1
    c, (start, count) = sharding.sharded_batch_matmul(a, b, rank, world, cpu_matmul)
    full = cpu_matmul(a, b)
    ok = torch.equal(c, full[start:start + count]) and count in (2, 3)

    A = torch.rand(48, 72, generator=g) * 2 - 1
    B = torch.rand(72, 200, generator=g) * 2 - 1   # ragged N: slabs of 128 and 72 columns
    slab, (s0, n0) = sharding.slab_matmul(A, B, rank, world, cpu_matmul)
    whole = cpu_matmul(A, B)
    ok = ok and torch.equal(slab, whole[:, s0:s0 + n0])
    gathered = sharding.gather_slabs(slab, B.shape[1])
    ok = ok and torch.equal(gathered, whole)
    with open(os.path.join(tmp, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "FAILED")
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
