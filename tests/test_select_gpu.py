"""Parity of the CUDA `bits` selection (through the C ABI) with the CPU oracle: bit-exact
distances AND indices, ties to the lowest index.  Shapes include the reference's own test
cases (tests/topk/bits_knn_test.cpp:7-63: k=128,n=128,q=1 and k=256,n=1024,q=1, dim 10)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run_select(bk, oracle, dist, k, **kw):
    d = torch.from_numpy(dist).cuda()
    labels = kw.get("labels")
    offsets = kw.get("label_offsets")
    got_d, got_i = bk.select(d, k, labels=None if labels is None else torch.from_numpy(labels).cuda(),
                             label_offsets=None if offsets is None else torch.from_numpy(offsets).cuda())
    torch.cuda.synchronize()
    bk.device_status()
    want_d, want_i = oracle.select(dist, k, labels=labels, label_offsets=offsets)
    gd, gi = got_d.cpu().numpy(), got_i.cpu().numpy()
    assert np.array_equal(gd.view(np.uint32), want_d.view(np.uint32)), "distances differ"
    assert np.array_equal(gi, want_i), "indices differ"


@pytest.mark.parametrize("k,n,q,dim", [(128, 128, 1, 10), (256, 1024, 1, 10), (32, 1024, 32, 8), (32, 997, 43, 37),
                                        (16, 25, 7, 9)])
def test_reference_test_shapes(bk, oracle, cuda, k, n, q, dim):
    points, queries = oracle.generate("uniform", 42, n, q, dim)
    run_select(bk, oracle, oracle.l2(points, queries), k)


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 7, 127, 128, 129, 255, 256, 257, 1023, 1025, 4095, 4096, 4097, 4099,
                               16385, 50001, 262144 + 3])
@pytest.mark.parametrize("k", [1, 32, 256])
def test_row_lengths(bk, oracle, cuda, n, k):
    rng = np.random.default_rng(n * 131 + k)
    dist = rng.random((5, n), dtype=np.float32)
    run_select(bk, oracle, dist, k)


@pytest.mark.parametrize("k", [1, 2, 7, 16, 31, 33, 64, 100, 128, 255, 256, 257, 300, 512, 513, 1000, 1024, 1025, 2000,
                               2048])
def test_every_list_size(bk, oracle, cuda, k):
    rng = np.random.default_rng(k)
    dist = rng.random((9, 40000), dtype=np.float32)
    run_select(bk, oracle, dist, k)


@pytest.mark.parametrize("k", [8, 256, 2048])
@pytest.mark.parametrize("values", [3, 50, 4000])
def test_heavy_ties_take_lowest_index(bk, oracle, cuda, k, values):
    rng = np.random.default_rng(values + k)
    dist = rng.integers(0, values, size=(6, 30011)).astype(np.float32)
    run_select(bk, oracle, dist, k)


@pytest.mark.parametrize("k", [32, 256, 1024])
@pytest.mark.parametrize("order", ["descending", "ascending", "constant"])
def test_adversarial_orders(bk, oracle, cuda, k, order):
    rng = np.random.default_rng(7)
    n = 70000
    base = np.sort(rng.random((4, n), dtype=np.float32), axis=1)
    if order == "descending":
        dist = np.ascontiguousarray(base[:, ::-1])      # every element enters the buffer
    elif order == "ascending":
        dist = base
    else:
        dist = np.full((4, n), 0.25, dtype=np.float32)
    run_select(bk, oracle, dist, k)


def test_reference_descending_preprocessor(bk, oracle, cuda):
    # `-p descending -d 1`: sorted coordinates, zero queries -> rows of x^2 in decreasing order
    points, queries = oracle.generate("uniform", 24, 100000, 3, 1)
    oracle.preprocess(points, queries, "descending")
    run_select(bk, oracle, oracle.l2(points, queries), 64)


def test_special_values(bk, oracle, cuda):
    rng = np.random.default_rng(3)
    dist = rng.random((4, 5000), dtype=np.float32)
    dist[0, ::3] = np.inf
    dist[1, :] = np.inf
    dist[1, 17] = 1.0
    dist[2, 100:200] = -0.0
    dist[2, 300:400] = 0.0
    dist[3, ::2] = -dist[3, ::2]                          # partial distances can be negative
    dist[3, 4999] = -np.inf
    run_select(bk, oracle, dist, 64)
    run_select(bk, oracle, dist, 2048)


@pytest.mark.parametrize("k", [1024, 2048])
def test_long_lists_with_runs_of_equal_distances(bk, oracle, cuda, k):
    # lists of 1024 pairs and more are folded by selection on (distance, label) keys: rows in which
    # the k-th pair sits inside a long run of equal distances, at the top of the key range (+inf),
    # at its bottom (-inf) and in the middle, and repeated (distance, label) pairs
    rng = np.random.default_rng(k)
    n = 20000
    dist = np.full((6, n), np.inf, dtype=np.float32)
    dist[0, 17] = 1.0
    dist[1, :] = -np.inf
    dist[1, 5::7] = rng.random(len(dist[1, 5::7]), dtype=np.float32)
    dist[2, :] = 0.5
    dist[2, ::50] = rng.random(len(dist[2, ::50]), dtype=np.float32)
    dist[3, :] = rng.integers(0, 3, size=n).astype(np.float32)
    dist[4, :] = np.float32(3.0e38)
    dist[4, 1::2] = -np.float32(3.0e38)
    dist[5, :] = rng.random(n, dtype=np.float32)
    run_select(bk, oracle, dist, k)
    labels = rng.integers(0, 40, size=(6, n)).astype(np.int32)   # many identical pairs
    run_select(bk, oracle, dist, k, labels=labels)


@pytest.mark.parametrize("seed", range(24))
def test_long_lists_random_shapes(bk, oracle, cuda, seed):
    # k above 512 (lists folded by selection), row lengths around the stage and buffer sizes, value
    # patterns that make stages sparse, dense, tied or partly infinite; whole rows and split rows
    rng = np.random.default_rng(1000 + seed)
    k = int(rng.choice([513, 777, 1000, 1024, 1025, 1500, 2000, 2048]))
    n = int(rng.choice([k, k + 1, 3000, 4097, 16384, 16385, 50000, 131072 + 5, 300001]))
    q = int(rng.integers(1, 5))
    kind = seed % 5
    if kind == 0:
        dist = rng.random((q, n), dtype=np.float32)
    elif kind == 1:
        dist = np.sort(rng.random((q, n), dtype=np.float32), axis=1)[:, ::-1].copy()
    elif kind == 2:
        dist = rng.integers(0, 7, size=(q, n)).astype(np.float32)
    elif kind == 3:
        dist = np.sort(rng.random((q, n), dtype=np.float32), axis=1)
    else:
        dist = (rng.standard_normal((q, n)) * 1e3).astype(np.float32)
        dist[:, ::11] = np.inf
    run_select(bk, oracle, dist, k)
    if n > 20000:
        d = torch.from_numpy(dist).cuda()
        got_d, got_i = bk.select_split(d, k, splits=int(rng.choice([2, 5])))
        torch.cuda.synchronize()
        bk.device_status()
        want_d, want_i = oracle.select(dist, k)
        assert np.array_equal(got_d.cpu().numpy().view(np.uint32), want_d.view(np.uint32)), "distances differ (split rows)"
        assert np.array_equal(got_i.cpu().numpy(), want_i), "indices differ (split rows)"


@pytest.mark.parametrize("n,k", [(3, 16), (100, 256), (1, 1), (255, 2048)])
def test_rows_shorter_than_k_are_padded(bk, oracle, cuda, n, k):
    rng = np.random.default_rng(n)
    run_select(bk, oracle, rng.random((3, n), dtype=np.float32), k)


@pytest.mark.parametrize("pad", [1, 2, 3, 5])
def test_unaligned_leading_dimension(bk, oracle, cuda, pad):
    # rows that do not start on a 16-byte boundary: scalar head + bulk middle + scalar tail
    rng = np.random.default_rng(pad)
    n = 20000
    full = rng.random((7, n + pad), dtype=np.float32)
    d = torch.from_numpy(full).cuda()
    view = d[:, 1:1 + n - 1] if pad > 1 else d[:, :n]
    got_d, got_i = bk.select(view, 48)
    torch.cuda.synchronize()
    sub = np.ascontiguousarray(full[:, 1:1 + n - 1] if pad > 1 else full[:, :n])
    want_d, want_i = oracle.select(sub, 48)
    assert np.array_equal(got_d.cpu().numpy(), want_d) and np.array_equal(got_i.cpu().numpy(), want_i)


def test_explicit_labels_and_offsets(bk, oracle, cuda):
    rng = np.random.default_rng(11)
    dist = rng.integers(0, 100, size=(6, 9000)).astype(np.float32)
    labels = np.stack([rng.permutation(9000) for _ in range(6)]).astype(np.int32) + 5
    run_select(bk, oracle, dist, 100, labels=labels)
    offsets = (np.arange(6, dtype=np.int32) * 9000)
    run_select(bk, oracle, dist, 100, label_offsets=offsets)


@pytest.mark.parametrize("stage_bytes,stages,merge_at", [(4096, 2, 100), (8192, 8, 50), (32768, 3, 100), (65536, 2, 10)])
def test_launch_shapes_do_not_change_results(bk, oracle, cuda, stage_bytes, stages, merge_at):
    old = {key: bk.get_tuning(key) for key in ("select.stage_bytes", "select.stages", "select.merge_at")}
    try:
        bk.set_tuning("select.stage_bytes", stage_bytes)
        bk.set_tuning("select.stages", stages)
        bk.set_tuning("select.merge_at", merge_at)
        rng = np.random.default_rng(stage_bytes)
        for k in (16, 256, 700):
            run_select(bk, oracle, rng.random((6, 150001), dtype=np.float32), k)
            run_select(bk, oracle, rng.integers(0, 9, size=(3, 33333)).astype(np.float32), k)
    finally:
        for key, value in old.items():
            bk.set_tuning(key, value)


@pytest.mark.parametrize("threads,ipt", [(256, 1), (256, 2), (256, 4), (512, 1), (512, 2), (512, 4), (1024, 1), (1024, 2)])
def test_block_shapes_do_not_change_results(bk, oracle, cuda, threads, ipt):
    # every (block size, pairs per thread) the tuning table may pick, on random, tie-heavy and
    # descending rows (the last keep every stage dense)
    old = {key: bk.get_tuning(key) for key in ("select.threads", "select.ipt")}
    try:
        bk.set_tuning("select.threads", threads)
        bk.set_tuning("select.ipt", ipt)
        rng = np.random.default_rng(threads + ipt)
        for k in {min(threads * ipt, 2048), max(1, threads * ipt // 2 - 3), 17}:
            run_select(bk, oracle, rng.random((5, 200001), dtype=np.float32), k)
            run_select(bk, oracle, rng.integers(0, 9, size=(3, 70000)).astype(np.float32), k)
            run_select(bk, oracle, np.sort(rng.random((3, 150000), dtype=np.float32), axis=1)[:, ::-1].copy(), k)
    finally:
        for key, value in old.items():
            bk.set_tuning(key, value)


@pytest.mark.parametrize("variant", ["no_buffer", "shared_list"])
def test_ablation_variants_give_the_same_result(bk, oracle, cuda, variant):
    # no_buffer: every value is sorted and merged (partial-bitonic-regs); shared_list: filtered
    # buffer, list and networks in shared memory (partial-bitonic-buffered-static)
    which = bk.ABLATION_NO_BUFFER if variant == "no_buffer" else bk.ABLATION_SHARED_LIST
    rng = np.random.default_rng(12)
    for k in (1, 16, 100, 256, 600, 2048):
        for dist in (rng.random((5, 30001), dtype=np.float32), rng.integers(0, 40, size=(3, 9000)).astype(np.float32),
                     np.sort(rng.random((2, 5000), dtype=np.float32), axis=1)[:, ::-1].copy()):
            got_d, got_i = bk.select_ablation(torch.from_numpy(dist).cuda(), k, which)
            torch.cuda.synchronize()
            bk.device_status()
            want_d, want_i = oracle.select(dist, k)
            assert np.array_equal(got_d.cpu().numpy().view(np.uint32), want_d.view(np.uint32)), (variant, k)
            assert np.array_equal(got_i.cpu().numpy(), want_i), (variant, k)


def test_expired_device_wait_is_reported_and_the_context_survives(bk, oracle, cuda):
    # a bounded wait that nothing satisfies: the kernel gives up, sets the status word, returns
    bk.device_status()
    bk.selftest_bounded_wait()
    with pytest.raises(bk.BitsKnnError) as err:
        bk.device_status()
    assert err.value.status == bk.ERR_DEVICE_TIMEOUT
    bk.device_status()                                   # reported once, then cleared
    rng = np.random.default_rng(1)
    run_select(bk, oracle, rng.random((4, 5000), dtype=np.float32), 16)   # the context is still fine


def test_config_c1_full_parity(bk, oracle, cuda):
    # q=1024 x n=32768 Uniform[0,1) (numpy Philox stand-in for the seeded matrix), k=32
    rng = np.random.default_rng(42)
    run_select(bk, oracle, rng.random((1024, 32768), dtype=np.float32), 32)


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 16, 0])
@pytest.mark.parametrize("k", [10, 256, 1024])
def test_split_rows_then_merge(bk, oracle, cuda, splits, k):
    rng = np.random.default_rng(splits * 7 + k)
    dist = rng.integers(0, 5000, size=(5, 100003)).astype(np.float32)
    got_d, got_i = bk.select_split(torch.from_numpy(dist).cuda(), k, splits=splits)
    torch.cuda.synchronize()
    bk.device_status()
    want_d, want_i = oracle.select(dist, k)
    assert np.array_equal(got_d.cpu().numpy(), want_d) and np.array_equal(got_i.cpu().numpy(), want_i)


@pytest.mark.parametrize("lists,k", [(1, 5), (2, 128), (8, 128), (8, 2048), (3, 300), (64, 1000)])
def test_merge_of_candidate_lists(bk, oracle, cuda, lists, k):
    rng = np.random.default_rng(lists * 1000 + k)
    q = 11
    cd = np.sort(rng.integers(0, 3000, size=(lists, q, k)).astype(np.float32), axis=2)
    ci = rng.permutation(lists * q * k).astype(np.int32).reshape(lists, q, k)
    got_d, got_i = bk.merge(torch.from_numpy(cd).cuda(), torch.from_numpy(ci).cuda())
    torch.cuda.synchronize()
    want_d, want_i = oracle.merge(cd, ci)
    assert np.array_equal(got_d.cpu().numpy(), want_d) and np.array_equal(got_i.cpu().numpy(), want_i)


def test_published_checksum_on_gpu(bk, oracle, cuda):
    # the reference's published run: seed 24, n=2^20, q=1024 (query 0 suffices), dim 1, k=32
    points, queries = oracle.generate("uniform", 24, 1 << 20, 1, 1)
    dist = torch.from_numpy(oracle.l2(points, queries)).cuda()
    _, idx = bk.select(dist, 32)
    assert oracle.checksum(idx[0].cpu().numpy()) == 16556617


def test_full_size_properties(bk, cuda):
    """Configuration C2 size (q=1024, n=2^20, 4 GiB): properties that need no CPU oracle."""
    q, n = 1024, 1 << 20
    gen = torch.Generator(device="cuda").manual_seed(42)
    dist = torch.rand((q, n), generator=gen, device="cuda", dtype=torch.float32)
    for k in (16, 256, 2048):
        d, i = bk.select(dist, k)
        torch.cuda.synchronize()
        bk.device_status()
        # (1) ascending, (2) every reported pair is an element of its row
        assert bool((d[:, 1:] >= d[:, :-1]).all())
        assert bool((torch.gather(dist, 1, i.long()) == d).all())
        # (3) exactly the k smallest: the library's top-k values are a second opinion
        ref = torch.topk(dist, k, dim=1, largest=False, sorted=True).values
        assert bool((ref == d).all())
        # (4) ties inside the result are in increasing index order, indices are distinct
        same = d[:, 1:] == d[:, :-1]
        assert bool((i[:, 1:][same] > i[:, :-1][same]).all())
        assert all(len(torch.unique(i[r])) == k for r in range(0, q, 97))
        # (5) idempotence: selecting from the selected pairs returns them unchanged
        d2, i2 = bk.select(d, k, labels=i)
        assert bool((d2 == d).all()) and bool((i2 == i).all())
        # (6) tie cut by the k boundary holds the lowest indices
        kth = d[:, -1:]
        n_less = (dist < kth).sum(1)
        boundary = (dist == kth)
        want_last = torch.where(boundary, torch.arange(n, device="cuda").expand(q, n),
                                torch.full((1,), n, device="cuda")).sort(1).values
        take = (k - n_less)
        rows = torch.arange(q, device="cuda")
        assert bool((want_last[rows, take - 1] == i[:, -1]).all())
    del dist
    torch.cuda.empty_cache()
