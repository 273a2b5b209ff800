"""GPU: the column-split MatMul with peer stores (rmlk_b200_matmul_tp / rmlk_b200_tp_wait) through the C ABI.

On one GPU the "peers" are the rank's own buffers (world 1) or two buffers of the same device standing for two ranks
(the stores and flags take the same code path; only the addresses differ).  The bounded wait is exercised with a flag
that nothing sets: it must give up with RMLK_ERR_TIMEOUT in the status word and leave the context usable.  With two or
more GPUs in the box the real thing runs as one process per GPU (rmlk_b200.tpbench, which asserts its own error bound)."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OneDeviceBuffers:
    """Stand-in for rmlk_b200.parallel.PeerBuffers: `world` buffers on this device, rank 0's view of them."""

    def __init__(self, nbytes, world=1):
        self.tensors = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        self.local = self.tensors[0]
        self.nbytes = nbytes
        self.world, self.rank = world, 0
        self.ptrs = [t.data_ptr() for t in self.tensors]


@pytest.mark.parametrize("shape", [(64, 512, 1024), (64, 8192, 256), (4096, 256, 512), (3, 77, 200), (1, 2048, 8192), (17, 96, 384)])
def test_matmul_tp_world_1_equals_matmul(cuda, shape):
    from rmlk_b200 import kernels as K
    from rmlk_b200.parallel import PeerStoreColumnParallelMatMul, tp_layout
    m, k, n = shape
    g = torch.Generator(device="cuda").manual_seed(m + k + n)
    w = torch.randn(k, n, device="cuda", generator=g) * 0.05
    tp = PeerStoreColumnParallelMatMul(w, [(0, n)], m, buffers=OneDeviceBuffers(tp_layout(m, n, 1)[2]))
    for call in range(3):                        # alternating output buffers, growing epochs
        x = torch.randn(m, k, device="cuda", generator=g)
        y = tp(x)
        want = x.double() @ w.double()
        assert tp.status() == 0
        assert float((y.double() - want).abs().max()) <= 1e-4 * float(want.abs().max()), (shape, call)
        assert torch.allclose(y, K.matmul(x, w), rtol=0, atol=2e-5 * float(want.abs().max()))


def test_matmul_tp_two_blocks_of_columns_on_one_device(cuda):
    """Two 'ranks' on one device, run one after the other on one stream: each stores its block of columns into both output
    buffers and raises its flag in both flag arrays; after both, either buffer holds the whole product and the wait passes."""
    from rmlk_b200 import dtypes as dt
    from rmlk_b200._lib import last_error, lib
    from rmlk_b200.parallel import tp_layout
    m, k, n = 64, 1024, 2048
    out_bytes, flag_off, total = tp_layout(m, n, 2)
    bufs = [torch.zeros(total, dtype=torch.uint8, device="cuda") for _ in range(2)]
    x = torch.randn(m, k, device="cuda")
    w = torch.randn(k, n, device="cuda") * 0.05
    shards = [(0, 1024), (1024, 2048)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    L = lib()

    class Peers(ctypes.Structure):
        _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("out", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8)]

    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for rank, (a, b) in enumerate(shards):
        p = Peers()
        p.world, p.rank = 2, rank
        for r in range(2):
            p.out[r] = bufs[r].data_ptr()
            p.flags[r] = bufs[r].data_ptr() + flag_off
        ws_bytes = int(L.rmlk_b200_matmul_tp_workspace_bytes(dt.F32, ctypes.c_int64(m), ctypes.c_int64(b - a), ctypes.c_int64(k)))
        ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")
        shard = w[:, a:b].contiguous()
        rc = L.rmlk_b200_matmul_tp(stream, dt.F32, ctypes.c_int64(m), ctypes.c_int64(b - a), ctypes.c_int64(k), ctypes.c_void_p(x.data_ptr()),
                                   ctypes.c_void_p(shard.data_ptr()), ctypes.c_int64(n), ctypes.c_int64(a), ctypes.byref(p), ctypes.c_uint(1),
                                   ctypes.c_void_p(ws.data_ptr()), ctypes.c_size_t(ws.numel()), ctypes.c_void_p(status.data_ptr()))
        assert rc == 0, last_error()
    want = x.double() @ w.double()
    for r in range(2):
        rc = L.rmlk_b200_tp_wait(stream, ctypes.c_void_p(bufs[r].data_ptr() + flag_off), 2, ctypes.c_uint(1), ctypes.c_void_p(status.data_ptr()))
        assert rc == 0, last_error()
        y = bufs[r][: m * n * 4].view(torch.float32).view(m, n)
        assert float((y.double() - want).abs().max()) <= 1e-4 * float(want.abs().max()), r
        assert bufs[r][flag_off: flag_off + 8].view(torch.int32).tolist() == [1, 1]
    assert int(status.item()) == 0
    # bad arguments are refused before anything is launched
    p.world = 9
    assert L.rmlk_b200_matmul_tp(stream, dt.F32, ctypes.c_int64(m), ctypes.c_int64(1024), ctypes.c_int64(k), ctypes.c_void_p(x.data_ptr()),
                                 ctypes.c_void_p(w.data_ptr()), ctypes.c_int64(n), ctypes.c_int64(0), ctypes.byref(p), ctypes.c_uint(2), None,
                                 ctypes.c_size_t(0), None) == 1
    p.world = 2
    assert L.rmlk_b200_matmul_tp(stream, dt.F32, ctypes.c_int64(m), ctypes.c_int64(1024), ctypes.c_int64(k), ctypes.c_void_p(x.data_ptr()),
                                 ctypes.c_void_p(w.data_ptr()), ctypes.c_int64(n), ctypes.c_int64(1536), ctypes.byref(p), ctypes.c_uint(2), None,
                                 ctypes.c_size_t(0), None) == 1           # the block would end past the last column


def test_tp_wait_gives_up_when_a_rank_never_arrives(cuda):
    """A flag that nothing sets: the wait is bounded (a second or two), stores RMLK_ERR_TIMEOUT in the status word and the
    stream - and the context - carry on."""
    from rmlk_b200._lib import last_error, lib
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags[0] = 7                                   # "rank 0" arrived at epoch 7, "rank 1" never does
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib().rmlk_b200_tp_wait(stream, ctypes.c_void_p(flags.data_ptr()), 2, ctypes.c_uint(7), ctypes.c_void_p(status.data_ptr()))
    assert rc == 0, last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 5                 # RMLK_ERR_TIMEOUT
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0   # the context still works
    # an epoch already passed is not waited for
    status.zero_()
    flags[1] = 9
    rc = lib().rmlk_b200_tp_wait(stream, ctypes.c_void_p(flags.data_ptr()), 2, ctypes.c_uint(7), ctypes.c_void_p(status.data_ptr()))
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0


def test_column_split_matmul_across_gpus(cuda):
    """One process per GPU (2 of the box's GPUs): peer stores over NVLink against NCCL all-gather and one GPU, every result
    checked against float64 inside the sweep."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29577", "-m", "rmlk_b200.tpbench", "--iters", "3"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(rows) == 8 and all('"peer_status": 0' in l for l in rows)
