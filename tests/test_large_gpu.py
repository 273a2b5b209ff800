"""Indexing / layout ops at the large end of the sweep: 4 GB tensors (2^30 fp32 elements, 2^29 int64 elements), so that
element offsets pass 2^31 bytes and byte offsets pass 2^32 - the range where the reference's kernels, which index with
32-bit `unsigned int` (cuda/src/ptx/headers/binary_op_macros.cuh:26-29), wrap.  Bit-exact against torch's own indexing
on the same device (an independent implementation used as the checker) and through round trips.  Values are uniform,
indices uniform in range, as in the sweep's description.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

K = None


@pytest.fixture(scope="module", autouse=True)
def _k(cuda):
    global K
    from rmlk_b200 import kernels
    K = kernels
    yield kernels
    torch.cuda.empty_cache()


def uniform(shape, dtype, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    if dtype == torch.float32:
        return torch.rand(shape, device="cuda", generator=g) * 8 - 4
    return torch.randint(-(1 << 40), 1 << 40, shape, device="cuda", dtype=dtype, generator=g)


@pytest.mark.parametrize("dtype,rows", [(torch.float32, 1 << 19), (torch.int64, 1 << 18)])
def test_gather_rows_of_a_4gb_table(dtype, rows):
    data = uniform((rows, 2048), dtype, 1)                       # 4 GB
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    idx = torch.randint(0, rows, (rows // 2,), device="cuda", generator=g)
    idx[0], idx[1] = rows - 1, 0                                 # both ends of the table
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = K.gather(data, idx, 0, status)
    assert int(status.item()) == 0
    assert torch.equal(got, data.index_select(0, idx))
    # negative indices address the same rows
    got_neg = K.gather(data, idx - rows, 0, status)
    assert int(status.item()) == 0 and torch.equal(got_neg, got)


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (1024, 1024, 1024)), (torch.int64, (512, 1024, 1024))])
def test_strided_and_reversed_slices_of_4gb(dtype, shape):
    x = uniform(shape, dtype, 3)
    big = 1 << 62
    for axis in (0, 1, 2):
        got = K.slice_(x, [1], [big], [axis], [2])
        want = x[tuple(slice(1, None, 2) if d == axis else slice(None) for d in range(3))]
        assert torch.equal(got, want.contiguous()), ("step 2", axis)
        del got, want
    for axis in (0, 2):
        got = K.slice_(x, [-1], [-big], [axis], [-1])
        assert torch.equal(got, x.flip(axis)), ("step -1", axis)
        # reversing twice gives the tensor back
        assert torch.equal(K.slice_(got, [-1], [-big], [axis], [-1]), x)
        del got


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (64, 16, 4096, 256)), (torch.int64, (64, 8, 4096, 256))])
def test_4d_transposes_of_4gb(dtype, shape):
    x = uniform(shape, dtype, 4)
    for perm in ([0, 2, 1, 3], [0, 1, 3, 2], [3, 2, 1, 0], [1, 0, 3, 2], [2, 3, 0, 1]):
        got = K.transpose(x, perm)
        assert torch.equal(got, x.permute(perm).contiguous()), perm
        inv = [perm.index(i) for i in range(4)]
        assert torch.equal(K.transpose(got, inv), x), perm
        del got


def test_concat_into_a_4gb_tensor():
    a = uniform((64, 8, 4096, 128), torch.float32, 5)            # 1 GB
    b = uniform((64, 8, 12288, 128), torch.float32, 6)           # 3 GB
    got = K.concat([a, b], 2)                                    # the KV-append axis; output 4 GB
    assert torch.equal(got, torch.cat([a, b], 2))
    del got
    c = uniform((64, 8, 4096, 384), torch.float32, 7)            # 3 GB
    got = K.concat([a, c], 3)                                    # innermost axis
    assert torch.equal(got, torch.cat([a, c], 3))
    del got, b, c
    a0 = uniform((1 << 28,), torch.int64, 8)                     # 2 GB each, axis 0, int64
    got = K.concat([a0, a0.flip(0)], 0)
    assert torch.equal(got[:1 << 28], a0) and torch.equal(got[1 << 28:], a0.flip(0))


def test_expand_to_4gb():
    x = uniform((128, 8, 1, 4096, 64), torch.float32, 9)         # 1 GB: the grouped-query repeat, 1 -> 4 on a middle axis
    got = K.expand(x, (128, 8, 4, 4096, 64))                     # 4 GB
    assert torch.equal(got, x.expand(128, 8, 4, 4096, 64).contiguous())
    del got
    y = uniform((1 << 27, 1), torch.int64, 10)
    got = K.expand(y, (1 << 27, 4))                              # 4 GB of int64, innermost broadcast
    assert torch.equal(got, y.expand(1 << 27, 4).contiguous())


@pytest.mark.parametrize("dtype,rows", [(torch.float32, 1 << 19), (torch.int64, 1 << 18)])
def test_scatter_nd_rows_of_a_4gb_tensor(dtype, rows):
    data = uniform((rows, 2048), dtype, 11)                      # 4 GB
    n = rows // 4
    idx = torch.randperm(rows, device="cuda")[:n].contiguous()   # unique row numbers
    idx[0] = rows - 1
    idx = torch.unique(idx)
    upd = uniform((idx.numel(), 2048), dtype, 12)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = K.scatter_nd(data, idx.view(-1, 1), upd, "none", status)
    assert int(status.item()) == 0
    want = data.clone()
    want.index_copy_(0, idx, upd)
    assert torch.equal(got, want)
    if dtype == torch.int64:                                     # integer add is order independent and exact
        got = K.scatter_nd(data, idx.view(-1, 1), upd, "add", status)
        want = data.clone()
        want.index_add_(0, idx, upd)
        assert torch.equal(got, want)
