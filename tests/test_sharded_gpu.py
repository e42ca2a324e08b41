"""The sharded-search host layer on one GPU (world size 1): `select`, `knn` and the stream form
`submit_select` / `drain` go through the CUDA kernels and must agree with the plain calls.  The
multi-rank exchange itself is covered by the gloo test on CPU and by `bench.py --gpus N`."""
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
    # stream form: three searches, results identical to the plain call
    for step in range(3):
        done = search.submit_select(torch.roll(matrix, step, dims=0).contiguous(), k, 0)
        exp_d, exp_i = bk.select(torch.roll(matrix, step, dims=0).contiguous(), k)
        assert torch.equal(done[0], exp_d) and torch.equal(done[1], exp_i)
    assert search.drain() is None
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
