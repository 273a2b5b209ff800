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


# ------------------------------------------------------------------------------------------------
# Column-split MatMul with peer stores: bookkeeping on CPU ranks
# ------------------------------------------------------------------------------------------------
class _SharedBuffers:
    """Stand-in for rmlk_b200.parallel.PeerBuffers on CPU ranks: every rank's buffer is a shared-memory tensor that all
    ranks hold (handed to the workers by the parent)."""

    def __init__(self, tensors, rank):
        self.tensors = tensors
        self.local = tensors[rank]
        self.nbytes = tensors[rank].numel()
        self.world, self.rank = len(tensors), rank
        self.ptrs = list(range(len(tensors)))   # "addresses": indices into `tensors`


def _host_tp_class():
    from rmlk_b200.parallel import PeerStoreColumnParallelMatMul

    class HostTp(PeerStoreColumnParallelMatMul):
        """The two device steps restated on the host: the block of columns goes into every rank's buffer, then word `rank`
        of every flag array is set to the epoch; the wait polls the local flag array with a bound."""
        wait_seconds = 20.0

        def _load_library(self):
            return None

        def _store_block(self, x, buf):
            a, b = self.shards[self.rank]
            block = x @ self.w
            for r in range(self.world):
                out = self.buffers.tensors[r][buf * self.out_bytes: buf * self.out_bytes + self.m_max * self.n * 4].view(torch.float32).view(self.m_max, self.n)
                out[: x.shape[0], a:b] = block
            for r in range(self.world):
                self.buffers.tensors[r][self.flag_off:self.flag_off + 4 * self.world].view(torch.int32)[self.rank] = self.epoch

        def _wait_all(self):
            import time
            flags = self.buffers.local[self.flag_off:self.flag_off + 4 * self.world].view(torch.int32)
            t0 = time.time()
            while time.time() - t0 < self.wait_seconds:
                if bool((flags >= self.epoch).all()):
                    return
                time.sleep(0.001)
            self._status[0] = 5   # RMLK_ERR_TIMEOUT, as the device wait reports it

    return HostTp


def _tp_worker(rank, world, port, n, tensors, absent_rank, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        HostTp = _host_tp_class()
        g = torch.Generator().manual_seed(11)
        k, m_max = 40, 6
        w = torch.randn(k, n, generator=g)
        shards = column_shards(n, world, multiple=128 if n % 128 == 0 else 4)
        a, b = shards[rank]
        tp = HostTp(w[:, a:b].contiguous(), shards, m_max, buffers=_SharedBuffers(tensors, rank))
        ok = True
        if absent_rank is None:
            views = []
            for call, m in enumerate([5, 6, 1, 3]):     # alternating buffers, varying M
                x = torch.randn(m, k, generator=g)
                y = tp(x)
                ok = ok and torch.allclose(y, x @ w, atol=1e-5) and tp.status() == 0 and tp.epoch == call + 1
                views.append((y, (x @ w).clone()))
                if call >= 1:   # the previous call's result lives in the other buffer and is still intact
                    ok = ok and torch.allclose(views[call - 1][0], views[call - 1][1], atol=1e-5)
                dist.barrier()  # the stand-in has no stream order between ranks: keep them within one call of each other
        else:
            # one rank never stores its block: the others' wait runs out and reports it instead of hanging
            tp.wait_seconds = 1.0
            x = torch.randn(3, k, generator=g)
            if rank != absent_rank:
                tp(x)
                ok = tp.status() == 5
            dist.barrier()
        q.put((rank, bool(ok)))
        dist.destroy_process_group()
    except Exception as e:
        q.put((rank, repr(e)))


@pytest.mark.parametrize("world,n,absent", [(2, 512, None), (3, 768, None), (2, 200, None), (2, 512, 1), (3, 768, 0)])
def test_peer_store_column_parallel_bookkeeping_gloo(world, n, absent):
    from rmlk_b200.parallel import tp_layout
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    total = tp_layout(6, n, world)[2]
    tensors = [torch.zeros(total, dtype=torch.uint8).share_memory_() for _ in range(world)]
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, n, tensors, absent, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(r, True) for r in range(world)], results


def test_peer_store_column_parallel_rejects_wrong_sizes():
    from rmlk_b200.parallel import tp_layout
    HostTp = _host_tp_class()
    w = torch.randn(16, 256)
    bufs = _SharedBuffers([torch.zeros(tp_layout(4, 256, 1)[2], dtype=torch.uint8)], 0)
    tp = HostTp(w, [(0, 256)], 4, buffers=bufs)
    assert torch.allclose(tp(torch.ones(2, 16)), torch.ones(2, 16) @ w)
    with pytest.raises(ValueError):
        tp(torch.ones(5, 16))                                   # more rows than the buffers were sized for
    with pytest.raises(ValueError):
        tp(torch.ones(2, 17))                                   # wrong K
    with pytest.raises(ValueError):
        HostTp(w[:, :128], [(0, 256)], 4, buffers=bufs)         # shard width does not match the column range
    with pytest.raises(ValueError):
        HostTp(w, [(0, 256)], 4, buffers=_SharedBuffers([torch.zeros(64, dtype=torch.uint8)], 0))   # buffers too small
    with pytest.raises(ValueError):
        tp_layout(4, 255, 1)
