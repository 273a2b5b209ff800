"""Column-split MatMul across GPUs: the Llama-8B-shaped FFN MatMuls at decode-sized M.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m rmlk_b200.tpbench [--iters 30]

Shapes: [M, 4096] x [4096, 14336] and [M, 14336] x [14336, 4096] for M in {1, 8, 64}, fp32, W ~ N(0, 0.02).
Every rank holds the full W too, so the same run times the one-GPU MatMul beside the N-GPU one:

  local_us   this library's MatMul on the rank's column shard only (no communication)
  tp_us      shard MatMul + NCCL all-gather of the [M, N / world] slices + permuting copy to [M, N]
  full_us    the whole MatMul on one GPU

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
from .parallel import ColumnParallelMatMul, column_shards, max_over_ranks

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
    dev = "cuda"
    for (k, n) in [(4096, 14336), (14336, 4096)]:
        ring_n = max(2, (2 * L2_BYTES) // (4 * k * n) + 1)
        g = torch.Generator(device=dev).manual_seed(1)          # same weights on every rank
        ws = [torch.randn(k, n, device=dev, generator=g) * 0.02 for _ in range(ring_n)]
        shards = column_shards(n, world)
        a, b = shards[rank]
        tps = [ColumnParallelMatMul(w[:, a:b].contiguous(), shards) for w in ws]
        for m in (1, 8, 64):
            x = torch.randn(m, k, device=dev, generator=g)
            full_out = torch.empty(m, n, device=dev)
            wsb = K.matmul_workspace_bytes(1, m, n, k)
            scratch = torch.empty(max(wsb // 4, 1), device=dev) if wsb else None
            full_us = timed(lambda i: K.matmul(x, ws[i % ring_n], out=full_out, workspace=scratch), args.iters)
            local_us = timed(lambda i: tps[i % ring_n].local(x), args.iters)
            tp_us = timed(lambda i: tps[i % ring_n](x), args.iters)
            y = tps[0](x)
            ref = x.double() @ ws[0].double()
            err = float((y.double() - ref).abs().max() / ref.abs().max())
            if rank == 0:
                wbytes = 4 * k * n
                print(json.dumps({"shape": [m, k, n], "n_gpus": world, "full_us": full_us, "local_us": local_us, "tp_us": tp_us,
                                  "speedup_vs_one_gpu": full_us / tp_us, "weight_GBps_one_gpu": wbytes / full_us / 1e3,
                                  "weight_GBps_tp_aggregate": wbytes / tp_us / 1e3, "max_rel_err": err}), flush=True)
        del ws, tps
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
