"""Candidate-list merge (`bitsknn_merge`, `bitsknn_merge_lists`) and exact re-ranking
(`bitsknn_refine`) against the oracle, bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

PAD = np.int32(0x7fffffff)


def sorted_lists(rng, lists, q, k, values, pad_from=None):
    """(lists, q, k) candidate lists, each ascending in the (distance, index) order; entries from
    `pad_from` on are padding pairs (+inf, INT32_MAX)."""
    cd = rng.integers(0, values, size=(lists, q, k)).astype(np.float32)
    ci = rng.permutation(lists * q * k).astype(np.int32).reshape(lists, q, k)
    if pad_from is not None:
        cd[:, :, pad_from:] = np.inf
        ci[:, :, pad_from:] = PAD
    order = np.lexsort((ci, cd), axis=2)
    return np.take_along_axis(cd, order, 2), np.take_along_axis(ci, order, 2)


@pytest.mark.parametrize("lists,k", [(1, 5), (2, 128), (8, 128), (8, 256), (8, 2048), (3, 300), (64, 1000), (5, 32),
                                     (16, 17), (7, 512), (2, 1024), (33, 64)])
def test_sorted_lists_merge_like_unsorted_ones(bk, oracle, cuda, lists, k):
    rng = np.random.default_rng(lists * 1000 + k)
    q = 11
    cd, ci = sorted_lists(rng, lists, q, k, values=3000)
    want_d, want_i = oracle.merge(cd, ci)
    dev_d, dev_i = torch.from_numpy(cd).cuda(), torch.from_numpy(ci).cuda()
    for promise in (True, False):
        got_d, got_i = bk.merge(dev_d, dev_i, sorted_lists=promise)
        torch.cuda.synchronize()
        assert np.array_equal(got_d.cpu().numpy(), want_d), promise
        assert np.array_equal(got_i.cpu().numpy(), want_i), promise


@pytest.mark.parametrize("lists,k,pad_from", [(4, 100, 60), (8, 256, 1), (3, 2048, 2000), (2, 32, 0)])
def test_sorted_lists_with_padding(bk, oracle, cuda, lists, k, pad_from):
    rng = np.random.default_rng(k + pad_from)
    cd, ci = sorted_lists(rng, lists, 7, k, values=50, pad_from=pad_from)
    want_d, want_i = oracle.merge(cd, ci)
    got_d, got_i = bk.merge(torch.from_numpy(cd).cuda(), torch.from_numpy(ci).cuda(), sorted_lists=True)
    torch.cuda.synchronize()
    # padding that reaches the output is reported as (+inf, position), like a short row
    pad = want_i == PAD
    want_i = np.where(pad, np.arange(k, dtype=np.int32)[None, :], want_i)
    assert np.array_equal(got_d.cpu().numpy(), want_d) and np.array_equal(got_i.cpu().numpy(), want_i)


@pytest.mark.parametrize("k", [48, 256])
def test_column_shards_packed_like_the_sharded_search(bk, oracle, cuda, k):
    """Three column shards of one matrix, selected with their label offsets into one packed
    float32 buffer [shard][2][q][k] (plane 1 = the labels' bit patterns), then merged with the
    strides of that layout: equals the selection over the whole matrix.  Small integer values make
    ties across shards frequent."""
    rng = np.random.default_rng(k)
    q, n = 19, 30011
    dist = rng.integers(0, 400, size=(q, n)).astype(np.float32)
    full = torch.from_numpy(dist).cuda()
    bounds = [0, 10004, 20011, n]
    packed = torch.empty((3, 2, q, k), dtype=torch.float32, device="cuda")
    for s in range(3):
        b, e = bounds[s], bounds[s + 1]
        offsets = torch.full((q,), b, dtype=torch.int32, device="cuda")
        shard = full[:, b:e].contiguous()
        bk.select(shard, k, label_offsets=offsets, out=(packed[s, 0], packed.view(torch.int32)[s, 1]))
    got_d, got_i = bk.merge_strided(packed[:, 0], packed.view(torch.int32)[:, 1], list_stride=2 * q * k,
                                    query_stride=k, q=q, lists=3, k=k, sorted_lists=True)
    torch.cuda.synchronize()
    bk.device_status()
    want_d, want_i = oracle.select(dist, k)
    assert np.array_equal(got_d.cpu().numpy(), want_d) and np.array_equal(got_i.cpu().numpy(), want_i)
    one_d, one_i = bk.select(full, k)
    assert torch.equal(one_d, got_d) and torch.equal(one_i, got_i)


@pytest.mark.parametrize("n,q,dim,cands,k,base", [(5000, 33, 16, 64, 32, 0), (3000, 5, 7, 300, 100, 1000),
                                                 (20000, 64, 64, 160, 128, 0), (999, 3, 1, 999, 256, 7),
                                                 (4096, 9, 130, 2500, 2048, 0)])
def test_refine_reports_the_exact_chain(bk, oracle, cuda, n, q, dim, cands, k, base):
    rng = np.random.default_rng(n + dim)
    points = rng.random((n, dim), dtype=np.float32)
    queries = rng.random((q, dim), dtype=np.float32)
    cand = np.stack([rng.permutation(n)[:cands] for _ in range(q)]).astype(np.int32)
    exact = oracle.l2(points, queries)                       # sum of fmaf(y - x, y - x, acc), in order
    cand_d = np.take_along_axis(exact, cand.astype(np.int64), 1)
    want_d, want_i = oracle.select(np.ascontiguousarray(cand_d), k, labels=np.ascontiguousarray(cand + base))
    got_d, got_i = bk.refine(torch.from_numpy(points).cuda(), torch.from_numpy(queries).cuda(),
                             torch.from_numpy(cand + base).cuda(), k, index_base=base)
    torch.cuda.synchronize()
    assert np.array_equal(got_d.cpu().numpy().view(np.uint32), want_d.view(np.uint32))
    assert np.array_equal(got_i.cpu().numpy(), want_i)


def test_refine_skips_entries_outside_the_shard(bk, oracle, cuda):
    points = torch.rand((100, 8), device="cuda")
    queries = torch.rand((4, 8), device="cuda")
    cand = torch.tensor([[5, 0x7fffffff, 250, 7, -3, 99, 1, 2]] * 4, dtype=torch.int32, device="cuda")
    d, i = bk.refine(points, queries, cand, 5)
    torch.cuda.synchronize()
    assert sorted(i[0].tolist()) == [1, 2, 5, 7, 99]
    assert bool((d[:, 1:] >= d[:, :-1]).all())
