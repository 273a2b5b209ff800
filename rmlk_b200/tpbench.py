"""Column-split MatMul across GPUs: the Llama-8B-shaped FFN MatMuls at decode-sized M.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m rmlk_b200.tpbench [--iters 30]

Shapes: [M, 4096] x [4096, 14336] and [M, 14336] x [14336, 4096] for M in {1, 8, 64, 4096}, fp32, W ~ N(0, 0.02).
Every rank holds the full W too, so the same run times the one-GPU MatMul beside the N-GPU ones:

  full_us    the whole MatMul on one GPU
  local_us   this library's MatMul on the rank's column shard only (no communication)
  peer_us    rmlk_b200_matmul_tp + rmlk_b200_tp_wait: the shard's MatMul stores its columns into every rank's output
             over NVLink from its own epilogue, flags, bounded wait (PeerStoreColumnParallelMatMul)
  nccl_us    shard MatMul + NCCL all-gather of the [M, N / world] slices + permuting copy to [M, N] (ColumnParallelMatMul)

Every result is checked against float64 (max error relative to the largest element <= 1e-4, asserted).

Times are CUDA-event device times on the launching stream, maximum over ranks.  Weights rotate over a ring
larger than L2.  One JSON line per shape on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import kernels as K
from .parallel import ColumnParallelMatMul, PeerBuffers, PeerStoreColumnParallelMatMul, column_shards, max_over_ranks, tp_layout

L2_BYTES = 126 << 20


def timed(fn, iters, warm=5):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return max_over_ranks(e0.elapsed_time(e1) / iters, torch.device("cuda")) * 1e3


def sweep(world, rank, iters, ms=(1, 8, 64, 4096), shapes=((4096, 14336), (14336, 4096)), emit=None):
    """Runs the sweep on the current device; returns the rows (rank 0) and prints / collects them through `emit`."""
    dev = "cuda"
    rows = []
    m_max = max(ms)
    for (k, n) in shapes:
        ring_n = max(2, (2 * L2_BYTES) // (4 * k * n) + 1)
        g = torch.Generator(device=dev).manual_seed(1)          # same weights on every rank
        ws = [torch.randn(k, n, device=dev, generator=g) * 0.02 for _ in range(ring_n)]
        shards = column_shards(n, world)
        a, b = shards[rank]
        shard_ws = [w[:, a:b].contiguous() for w in ws]
        tps = [ColumnParallelMatMul(sw, shards) for sw in shard_ws]
        peer = None
        if world > 1:
            bufs = PeerBuffers(tp_layout(m_max, n, world)[2], torch.device(dev))
            peer = PeerStoreColumnParallelMatMul(shard_ws[0], shards, m_max, buffers=bufs)
        for m in ms:
            x = torch.randn(m, k, device=dev, generator=g)
            full_out = torch.empty(m, n, device=dev)
            wsb = K.matmul_workspace_bytes(1, m, n, k)
            scratch = torch.empty(max(wsb // 4, 1), device=dev) if wsb else None
            it = iters if m <= 64 else max(3, iters // 6)
            full_us = timed(lambda i: K.matmul(x, ws[i % ring_n], out=full_out, workspace=scratch), it)
            local_us = timed(lambda i: tps[i % ring_n].local(x), it)
            nccl_us = timed(lambda i: tps[i % ring_n](x), it)
            ref = x.double() @ ws[0].double()
            scale = float(ref.abs().max())
            err = float((tps[0](x).double() - ref).abs().max()) / scale
            row = {"shape": [m, k, n], "n_gpus": world, "full_us": full_us, "local_us": local_us, "nccl_us": nccl_us,
                   "nccl_speedup_vs_one_gpu": full_us / nccl_us, "max_rel_err_nccl": err}
            assert err <= 1e-4, row
            if peer is not None:
                def run_peer(i):
                    peer.w = shard_ws[i % ring_n]
                    peer(x)
                peer_us = timed(run_peer, it)
                peer.w = shard_ws[0]
                y = peer(x).clone()
                perr = float((y.double() - ref).abs().max()) / scale
                st = peer.status()
                row.update(peer_us=peer_us, peer_speedup_vs_one_gpu=full_us / peer_us, max_rel_err_peer=perr, peer_status=st,
                           weight_GBps_peer_aggregate=4 * k * n / peer_us / 1e3)
                assert st == 0 and perr <= 1e-4, row
            row["weight_GBps_one_gpu"] = 4 * k * n / full_us / 1e3
            if rank == 0:
                rows.append(row)
                if emit:
                    emit(row)
        del ws, tps, shard_ws, peer
        torch.cuda.empty_cache()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=30)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    sweep(world, rank, args.iters, emit=lambda row: print(json.dumps(row), flush=True))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
