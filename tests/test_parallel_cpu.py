"""N > 1 host logic on CPU ranks: gloo, world_size 2 and 3, one process per rank (as one process per GPU).

Covers what `bench.py --gpus N` and the column-split MatMul rely on: request sharding, max-over-ranks timing,
column ranges that keep every shard a multiple of 128, and the gather order of `ColumnParallelMatMul` (compute
and permute steps replaced by torch CPU ops; the CUDA kernels behind them have their own GPU tests).
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rmlk_b200.parallel import ColumnParallelMatMul, column_shards, max_over_ranks, shard_range  # noqa: E402


def test_shard_range_is_a_partition():
    for total in [0, 1, 7, 64, 65, 1000]:
        for world in [1, 2, 3, 8]:
            parts = [shard_range(total, world, r) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == total
            for (a0, a1), (b0, b1) in zip(parts, parts[1:]):
                assert a1 == b0 and a1 >= a0
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1


def test_column_shards_keep_multiples_of_128():
    for n, world in [(14336, 2), (14336, 4), (14336, 8), (4096, 8), (128256, 8), (8192, 3), (1000, 2), (128, 4)]:
        sh = column_shards(n, world)
        assert sh[0][0] == 0 and sh[-1][1] == n and len(sh) == world
        for (a0, a1), (b0, b1) in zip(sh, sh[1:]):
            assert a1 == b0
        for a, b in sh[:-1]:
            assert (b - a) % 128 == 0
        if n % (128 * world) == 0:
            assert len({b - a for a, b in sh}) == 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        g = torch.Generator().manual_seed(7)  # same weights and activations on every rank
        k, m = 48, 5
        w = torch.randn(k, n, generator=g)
        x = torch.randn(m, k, generator=g)
        tp = ColumnParallelMatMul.from_full(w, multiple=128 if n % 128 == 0 else 8,
                                            matmul=lambda a, b, out=None: a @ b, permute=lambda t: t.permute(1, 0, 2).contiguous())
        y = tp(x)
        a, b = tp.shards[rank]
        ok = torch.allclose(y, x @ w, atol=1e-5) and torch.equal(tp.local(x), x @ w[:, a:b]) and y.shape == (m, n)
        # request sharding + max-over-ranks timing as bench.py does it
        lo, hi = shard_range(64 * world + 1, world, rank)
        slow = max_over_ranks(10.0 + rank)
        counts = torch.tensor([hi - lo], dtype=torch.int64)
        dist.all_reduce(counts)
        ok = ok and slow == 10.0 + world - 1 and int(counts.item()) == 64 * world + 1
        q.put((rank, bool(ok)))
        dist.destroy_process_group()
    except Exception as e:  # surface the failure to the parent instead of hanging it
        q.put((rank, repr(e)))


@pytest.mark.parametrize("world,n", [(2, 512), (2, 200), (3, 1024), (2, 14336)])
def test_column_parallel_matmul_and_sharding_gloo(world, n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(r, True) for r in range(world)], results


def test_single_process_degenerates_to_local_matmul():
    w = torch.randn(16, 256)
    x = torch.randn(3, 16)
    tp = ColumnParallelMatMul(w, [(0, 256)], matmul=lambda a, b, out=None: a @ b, permute=lambda t: t)
    assert torch.equal(tp(x), x @ w)
    assert np.isclose(max_over_ranks(3.5), 3.5)
