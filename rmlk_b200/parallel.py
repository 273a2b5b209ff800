"""Multi-GPU plumbing of the operator path: one process per GPU, torch.distributed underneath.

Two ways the path spreads over GPUs (the reference itself is single-GPU: one `CudaContext::new(0)`,
runtime/src/core/instance.rs:199-205):

* request sharding - independent requests, weights replicated, no data-path collective.  `shard_range` gives a
  rank its contiguous share; `max_over_ranks` turns per-rank device times into the job's time.
* column-split MatMul - for weights too large or too slow for one GPU, W[K, N] is split by columns, every rank
  multiplies the same activations with its shard and the [M, N / world] results are gathered
  (`ColumnParallelMatMul`).  The gather is the path's one real exchange step; it runs as one NCCL all-gather
  followed by one permuting copy, both on the launching stream.

The compute and copy steps are injected as callables so that the sharding and gathering logic can be exercised
with gloo on CPU ranks; on GPUs they are the library's MatMul and transpose kernels.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split of `total` units: the first `total % world` ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world / rank")
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def column_shards(n: int, world: int, multiple: int = 128) -> List[Tuple[int, int]]:
    """Column ranges of an [K, n] weight for `world` ranks.  Shard widths are multiples of `multiple` (the
    tensor-core MatMul wants N % 128 == 0) except that the last rank also takes the remainder."""
    if n <= 0 or world <= 0:
        raise ValueError("bad n / world")
    blocks = n // multiple
    out, start = [], 0
    for r in range(world):
        b0, b1 = shard_range(blocks, world, r)
        stop = start + (b1 - b0) * multiple
        if r == world - 1:
            stop = n
        out.append((start, stop))
        start = stop
    return out


def max_over_ranks(value: float, device: Optional[torch.device] = None, group=None) -> float:
    """A multi-GPU step is as slow as its slowest rank."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class ColumnParallelMatMul:
    """y[M, N] = x[M, K] @ W[K, N] with W split by columns over the ranks of `group`.

    `matmul(x, w_shard) -> [M, n_r]` and `permute(t[world, M, n_max]) -> [M, world, n_max]` default to the
    library's CUDA kernels.  Shards may differ in width (N not divisible); narrower ones are padded to the
    widest for the gather and trimmed afterwards.
    """

    def __init__(self, w_shard: torch.Tensor, shards: Sequence[Tuple[int, int]], group=None,
                 matmul: Optional[Callable] = None, permute: Optional[Callable] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if len(shards) != self.world:
            raise ValueError("one column range per rank")
        self.shards = list(shards)
        self.n = self.shards[-1][1]
        self.widths = [b - a for a, b in self.shards]
        self.n_max = max(self.widths)
        if w_shard.shape[1] != self.widths[self.rank]:
            raise ValueError(f"rank {self.rank}: weight shard has {w_shard.shape[1]} columns, expected {self.widths[self.rank]}")
        self.w = w_shard
        self._scratch = {}
        if matmul is None or permute is None:
            from . import kernels as K

            def lib_matmul(x, w, out=None):
                # split-K scratch, sized once per M and kept: a shard is narrow, so K usually has to be split
                m = x.shape[0]
                if m not in self._scratch:
                    need = K.matmul_workspace_bytes(1, m, w.shape[1], w.shape[0])
                    self._scratch[m] = torch.empty(max(need // 4, 1), dtype=torch.float32, device=x.device) if need else None
                return K.matmul(x, w, out=out, workspace=self._scratch[m])

            matmul = matmul or lib_matmul
            permute = permute or (lambda t: K.transpose(t, [1, 0, 2]))
        self._matmul, self._permute = matmul, permute

    @classmethod
    def from_full(cls, w_full: torch.Tensor, group=None, multiple: int = 128, **kw) -> "ColumnParallelMatMul":
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        shards = column_shards(w_full.shape[1], world, multiple)
        a, b = shards[rank]
        return cls(w_full[:, a:b].contiguous(), shards, group, **kw)

    def local(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's [M, n_r] slice of the product (no communication)."""
        return self._matmul(x, self.w)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        mine = self.local(x)
        if self.world == 1:
            return mine
        even = all(w == self.n_max for w in self.widths)
        if not even:
            pad = torch.zeros(m, self.n_max, dtype=mine.dtype, device=mine.device)
            pad[:, : mine.shape[1]] = mine
            mine = pad
        gathered = torch.empty(self.world * m, self.n_max, dtype=mine.dtype, device=mine.device)  # rank-major rows
        dist.all_gather_into_tensor(gathered, mine.contiguous(), group=self.group)
        y = self._permute(gathered.view(self.world, m, self.n_max)).reshape(m, self.world * self.n_max)
        if even:
            return y
        cols = torch.cat([torch.arange(r * self.n_max, r * self.n_max + w, device=y.device) for r, w in enumerate(self.widths)])
        return y.index_select(1, cols)
