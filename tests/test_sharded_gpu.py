"""The sharded search on one GPU (world size 1) through `bitsknn_sharded_*`: `select`, `knn` and the
submit form `submit_select` / `drain` must agree with the plain calls.  The multi-rank exchange is
covered by test_sharded_multi_gpu.py (two or more GPUs), the gloo test of the host logic on CPU and
the checks inside `bench.py --gpus N`."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_search_equals_plain_calls(bk, cuda):
    import __graft_entry__ as entry
    from importlib import import_module
    sharded = import_module(entry.PKG_NAME + ".sharded")
    gen = torch.Generator(device="cuda").manual_seed(8)
    matrix = torch.rand((37, 50000), generator=gen, device="cuda")
    k = 48
    want_d, want_i = bk.select(matrix, k)
    search = sharded.ShardedSearch(bk, 0, 1)
    got_d, got_i = search.select(matrix, k, 0)
    assert torch.equal(got_d, want_d) and torch.equal(got_i, want_i)
    # submit form: three searches; a submit hands back the previous search's output, drain the last
    done = []
    for step in range(3):
        done.append(search.submit_select(torch.roll(matrix, step, dims=0).contiguous(), k, 0))
    done.append(search.drain())
    assert done[0] is None and search.drain() is None
    for step in range(3):
        exp_d, exp_i = bk.select(torch.roll(matrix, step, dims=0).contiguous(), k)
        assert torch.equal(done[step + 1][0], exp_d) and torch.equal(done[step + 1][1], exp_i)
    # shard offset = global labels
    off_d, off_i = search.select(matrix, k, 1000)
    assert torch.equal(off_d, want_d) and torch.equal(off_i, want_i + 1000)
    points = torch.rand((20000, 8), generator=gen, device="cuda")
    queries = torch.rand((65, 8), generator=gen, device="cuda")
    kd, ki = search.knn(points, queries, 16, 500)
    fd, fi = bk.fused(points, queries, 16, index_base=500)
    torch.cuda.synchronize()
    bk.device_status()
    assert torch.equal(kd, fd) and torch.equal(ki, fi)
    search.close()


def test_argument_checks_of_the_sharded_entry_points(bk, cuda):
    import ctypes
    lib = bk.lib()
    handle = ctypes.c_void_p()
    assert lib.bitsknn_sharded_create(ctypes.byref(handle), None, 2, 2) == bk.ERR_INVALID_ARGUMENT   # rank >= world
    assert lib.bitsknn_sharded_create(ctypes.byref(handle), None, 0, 2) == bk.ERR_INVALID_ARGUMENT   # no id
    assert lib.bitsknn_sharded_init(ctypes.byref(handle), None, 0, 2) == bk.ERR_INVALID_ARGUMENT     # no communicator
    h = bk.sharded_create(None, 0, 1)
    assert bk.sharded_workspace_bytes(h, 100, 10) == 0
    bk.sharded_destroy(h)
