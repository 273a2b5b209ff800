"""Multi-GPU plumbing of the operator path: one process per GPU, torch.distributed underneath.

Two ways the path spreads over GPUs (the reference itself is single-GPU: one `CudaContext::new(0)`,
runtime/src/core/instance.rs:199-205):

* request sharding - independent requests, weights replicated, no data-path collective.  `shard_range` gives a
  rank its contiguous share; `max_over_ranks` turns per-rank device times into the job's time.
* column-split MatMul - for weights too large or too slow for one GPU, W[K, N] is split by columns, every rank
  multiplies the same activations with its shard and every rank ends up with the whole [M, N] product.  Two forms of
  that one real exchange step: `PeerStoreColumnParallelMatMul` has the MatMul kernel's epilogue store each rank's block
  of columns straight into every rank's output buffer over NVLink (rmlk_b200_matmul_tp: peer stores + flags, no
  collective call); `ColumnParallelMatMul` runs the shard MatMul, one NCCL all-gather and one permuting copy - the
  baseline the first is measured against.

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


class PeerBuffers:
    """Device buffers of every rank of `group`, reachable from this process: what rmlk_b200_matmul_tp stores into.

    Allocation and the exchange of addresses go through torch's symmetric memory (one allocation of the same size on
    every rank, mapped into every process of the group).  `ptrs[r]` is rank r's buffer as seen from this process.
    No multicast object is bound: the data path uses plain peer stores only."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.nbytes = (nbytes + 255) // 256 * 256
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.local, group=group)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world:
            raise RuntimeError("symmetric memory returned a pointer table of the wrong size")
        self.local.zero_()


def tp_layout(m_max: int, n_total: int, world: int):
    """Byte layout of one rank's peer-visible buffer for PeerStoreColumnParallelMatMul: two output buffers
    [m_max, n_total] fp32 (even / odd calls) followed by the flag array (`world` 32-bit words, padded to 256 bytes).
    Returns (bytes of one output buffer, offset of the flags, total bytes)."""
    if m_max <= 0 or n_total <= 0 or n_total % 4 or not 1 <= world <= 8:
        raise ValueError("tp_layout: m_max, n_total must be positive, n_total a multiple of 4, world in 1..8")
    out_bytes = (m_max * n_total * 4 + 255) // 256 * 256
    return out_bytes, 2 * out_bytes, 2 * out_bytes + 256


class PeerStoreColumnParallelMatMul:
    """y[M, N] = x[M, K] @ W[K, N], W split by columns over the ranks of `group`; the rank that computes a block of
    columns writes it into every rank's output from the MatMul kernel itself (include/rmlk_b200.h: rmlk_b200_matmul_tp,
    rmlk_b200_tp_wait).  x must hold the same values on every rank.  The returned tensor is a view of one of two
    alternating output buffers: it stays valid until the call after next."""

    def __init__(self, w_shard: torch.Tensor, shards: Sequence[Tuple[int, int]], m_max: int, group=None, buffers=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if len(shards) != self.world:
            raise ValueError("one column range per rank")
        self.shards = list(shards)
        self.n = self.shards[-1][1]
        a, b = self.shards[self.rank]
        if w_shard.shape[1] != b - a:
            raise ValueError(f"rank {self.rank}: weight shard has {w_shard.shape[1]} columns, expected {b - a}")
        if any(lo % 4 or hi % 4 for lo, hi in self.shards):
            raise ValueError("shard boundaries must be multiples of 4 columns")
        self.w = w_shard.contiguous()
        self.k = w_shard.shape[0]
        self.m_max = m_max
        self.out_bytes, self.flag_off, total = tp_layout(m_max, self.n, self.world)
        self.buffers = buffers if buffers is not None else PeerBuffers(total, w_shard.device, group)
        if self.buffers.nbytes < total:
            raise ValueError("peer buffers are smaller than tp_layout() asks for")
        self.epoch = 0
        self._ws = None
        from . import dtypes as dt
        self._f32 = dt.F32
        self._lib = self._load_library()
        self._status = torch.zeros(1, dtype=torch.int32, device=w_shard.device)
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group)   # every rank's flags are zero before anybody signals

    def _load_library(self):
        from ._lib import lib
        return lib()

    def _peers(self, buf: int):
        import ctypes

        class Peers(ctypes.Structure):
            _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("out", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8)]

        p = Peers()
        p.world, p.rank = self.world, self.rank
        for r in range(self.world):
            p.out[r] = self.buffers.ptrs[r] + buf * self.out_bytes
            p.flags[r] = self.buffers.ptrs[r] + self.flag_off
        return p

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        m = x.shape[0]
        if m > self.m_max or x.shape[1] != self.k:
            raise ValueError(f"activations {tuple(x.shape)} do not fit m_max {self.m_max} / K {self.k}")
        self.epoch += 1
        buf = self.epoch & 1
        self._store_block(x.contiguous(), buf)   # this rank's columns into every rank's buffer `buf`, then the flags
        self._wait_all()                         # until every rank's flag in the local array has reached the epoch
        return self.buffers.local[buf * self.out_bytes: buf * self.out_bytes + m * self.n * 4].view(torch.float32).view(m, self.n)

    # The two device steps, as calls into the library; a host stand-in overrides them to exercise the bookkeeping on CPU ranks.
    def _store_block(self, x: torch.Tensor, buf: int):
        import ctypes
        m = x.shape[0]
        a, b = self.shards[self.rank]
        need = int(self._lib.rmlk_b200_matmul_tp_workspace_bytes(self._f32, ctypes.c_int64(m), ctypes.c_int64(b - a), ctypes.c_int64(self.k)))
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
        peers = self._peers(buf)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = self._lib.rmlk_b200_matmul_tp(stream, self._f32, ctypes.c_int64(m), ctypes.c_int64(b - a), ctypes.c_int64(self.k),
                                           ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(self.w.data_ptr()), ctypes.c_int64(self.n), ctypes.c_int64(a),
                                           ctypes.byref(peers), ctypes.c_uint(self.epoch), ctypes.c_void_p(self._ws.data_ptr()),
                                           ctypes.c_size_t(self._ws.numel()), ctypes.c_void_p(self._status.data_ptr()))
        if rc != 0:
            from ._lib import last_error
            raise RuntimeError(f"rmlk_b200_matmul_tp failed ({rc}): {last_error()}")

    def _wait_all(self):
        import ctypes
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = self._lib.rmlk_b200_tp_wait(stream, ctypes.c_void_p(self.buffers.ptrs[self.rank] + self.flag_off), self.world, ctypes.c_uint(self.epoch),
                                         ctypes.c_void_p(self._status.data_ptr()))
        if rc != 0:
            from ._lib import last_error
            raise RuntimeError(f"rmlk_b200_tp_wait failed ({rc}): {last_error()}")

    def status(self) -> int:
        """Device status word (synchronises): 0, or RMLK_ERR_TIMEOUT (5) if a rank never arrived within the wait's bound."""
        return int(self._status.item())
