"""Parity of `bits-fused` (through the C ABI) with the CPU oracle: bit-exact partial distances
(|x|^2 - 2 x.y, no query norm -- what the reference's fused kernel reports) and indices with
ties to the lowest index.  First four shapes are the reference's own fused tests
(tests/topk/fused_cache_kernel_test.cu:12-82)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1], ids=["rows8", "tiled"], autouse=True)
def fused_variant(request, bk):
    """Every test runs with both FP32 kernels: 8 queries per block, and 128 x 128 tiles."""
    old = bk.get_tuning("fused.variant")
    bk.set_tuning("fused.variant", request.param)
    yield request.param
    bk.set_tuning("fused.variant", old)


def run_fused(bk, oracle, points, queries, k, partial=True, index_base=0):
    got_d, got_i = bk.fused(torch.from_numpy(points).cuda(), torch.from_numpy(queries).cuda(), k,
                            mode=bk.L2_PARTIAL if partial else bk.L2_EXACT, index_base=index_base)
    torch.cuda.synchronize()
    want_d, want_i = oracle.knn(points, queries, k, partial=partial, index_base=index_base)
    assert np.array_equal(got_d.cpu().numpy().view(np.uint32), want_d.view(np.uint32)), "distances differ"
    assert np.array_equal(got_i.cpu().numpy(), want_i), "indices differ"


@pytest.mark.parametrize("dim,n,q,k", [(8, 1024, 32, 32), (16, 1024, 1, 32), (37, 997, 43, 32), (9, 25, 7, 16)])
def test_reference_test_shapes(bk, oracle, cuda, dim, n, q, k):
    points, queries = oracle.generate("uniform", 42, n, q, dim)
    run_fused(bk, oracle, points, queries, k)


@pytest.mark.parametrize("k", [1, 4, 16, 31, 32, 33, 64, 100, 128, 200, 256])
@pytest.mark.parametrize("dim", [1, 3, 4, 8, 16])
def test_k_and_dim_grid(bk, oracle, cuda, k, dim):
    points, queries = oracle.generate("uniform", 42, 5000 + k, 19, dim)
    run_fused(bk, oracle, points, queries, k)


@pytest.mark.parametrize("dim", [2, 5, 32, 64, 65, 128])
@pytest.mark.parametrize("partial", [True, False])
def test_larger_dims_both_forms(bk, oracle, cuda, dim, partial):
    points, queries = oracle.generate("normal", 9, 3333, 21, dim)
    run_fused(bk, oracle, points, queries, 32, partial=partial)


def test_many_tiles_and_index_base(bk, oracle, cuda):
    points, queries = oracle.generate("uniform", 42, 100000, 24, 16)
    run_fused(bk, oracle, points, queries, 128, index_base=1 << 20)


def test_few_queries_long_database(bk, oracle, cuda):
    # the tiled kernel cuts the database into parts when the query tiles cannot fill the SMs
    points, queries = oracle.generate("uniform", 11, 300000, 5, 16)
    run_fused(bk, oracle, points, queries, 64)
    run_fused(bk, oracle, points, queries, 7, partial=False, index_base=12345)


def test_ties_take_lowest_index(bk, oracle, cuda):
    rng = np.random.default_rng(5)
    points = rng.integers(0, 4, size=(20000, 4)).astype(np.float32)   # many identical points
    queries = rng.integers(0, 4, size=(17, 4)).astype(np.float32)
    for k in (8, 64, 256):
        run_fused(bk, oracle, points, queries, k)
        run_fused(bk, oracle, points, queries, k, partial=False)


def test_sorted_database_is_the_adversarial_order(bk, oracle, cuda):
    # points sorted by decreasing distance to the origin, queries at the origin: every point
    # is a new best candidate for every query
    points, queries = oracle.generate("uniform", 24, 30000, 9, 1)
    oracle.preprocess(points, queries, "descending")
    run_fused(bk, oracle, points, queries, 32)


def test_fewer_points_than_k(bk, oracle, cuda):
    points, queries = oracle.generate("uniform", 3, 10, 5, 6)
    run_fused(bk, oracle, points, queries, 64)


def test_fused_equals_distance_matrix_plus_selection_at_scale(bk, cuda):
    """n = 2^20 points, dim 16: the fused result for 512 queries equals the unfused pipeline
    (partial distance matrix, then the bits selection) bit for bit."""
    gen = torch.Generator(device="cuda").manual_seed(42)
    points = torch.rand((1 << 20, 16), generator=gen, device="cuda")
    queries = torch.rand((512, 16), generator=gen, device="cuda")
    for k in (16, 128):
        d, i = bk.fused(points, queries, k)
        dist = bk.l2(points, queries, mode=bk.L2_PARTIAL)
        d2, i2 = bk.select(dist, k)
        torch.cuda.synchronize()
        assert bool((d == d2).all()) and bool((i == i2).all())


def test_argument_errors(bk, cuda):
    x = torch.zeros((64, 4), device="cuda")
    with pytest.raises(bk.BitsKnnError) as err:
        bk.fused(x, x, 512)
    assert err.value.status == bk.ERR_UNSUPPORTED_K and "Unsupported k value: 512" in err.value.message
    with pytest.raises(bk.BitsKnnError) as err:
        bk.fused(x, x, 8, mode=42)
    assert err.value.status == bk.ERR_UNSUPPORTED_MODE
