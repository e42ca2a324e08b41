"""Tensor-core modes at the sizes the benchmark quotes: n = 2^20 points (uniform and clustered
coordinates) and one shard of the largest configuration (n = 2^24, dim 64, k = 128).

Tolerances (the ones stated for these modes): recall@k >= 0.999 over the compared queries and
relative error of the k-th distance <= 1e-3 for every compared query, both against the FP32 path
(`bitsknn_fused` in BITSKNN_L2_EXACT mode: sum of (x - y)^2 as one FMA chain per pair).
Both tensor-core pipelines end with the exact re-ranking of their candidates, so a reported
distance is an FP32-path distance and the k-th distance differs only where the k-th neighbour does.

The tensor-core search runs over the full query set of the benchmark shape (so the block layout
-- one database range per query tile -- is the benchmarked one); the FP32 side runs over the first
`sub` queries only, which keeps it to a few hundred milliseconds.  A query's result does not depend
on the other queries, so comparing the first `sub` rows is exact.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

MIN_RECALL = 0.999
MAX_KTH_REL = 1e-3


def make_data(kind, n, q, dim, seed):
    """Uniform[0,1) coordinates, or 256 Gaussian clusters (sigma 0.05) around uniform centres."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    if kind == "uniform":
        return (torch.rand((n, dim), generator=gen, device="cuda"),
                torch.rand((q, dim), generator=gen, device="cuda"))
    centres = torch.rand((256, dim), generator=gen, device="cuda")

    def draw(count):
        out = torch.empty((count, dim), device="cuda")
        step = 1 << 22
        for b in range(0, count, step):
            e = min(count, b + step)
            pick = torch.randint(0, 256, (e - b,), generator=gen, device="cuda")
            out[b:e] = centres[pick] + 0.05 * torch.randn((e - b, dim), generator=gen, device="cuda")
        return out

    return draw(n), draw(q)


def recall_and_kth_error(i_tc, d_tc, i_ex, d_ex):
    """recall@k over all rows, and the largest relative error of the k-th distance."""
    k = i_ex.shape[1]
    a = torch.sort(i_tc, dim=1).values
    b = torch.sort(i_ex, dim=1).values
    # membership of every approximate index in the exact row (both rows sorted)
    pos = torch.searchsorted(b, a).clamp_(max=k - 1)
    hits = (torch.gather(b, 1, pos) == a).sum().item()
    recall = hits / a.numel()
    rel = ((d_tc[:, -1] - d_ex[:, -1]).abs() / d_ex[:, -1].abs().clamp_min(1e-30)).max().item()
    return recall, rel


def fused_quality(bk, points, queries, k, mode, sub):
    d_tc, i_tc = bk.fused(points, queries, k, mode=mode)
    d_ex, i_ex = bk.fused(points, queries[:sub].contiguous(), k, mode=bk.L2_EXACT)
    torch.cuda.synchronize()
    bk.device_status()
    assert bool((d_tc[:, 1:] >= d_tc[:, :-1]).all()), "distances not ascending"
    return recall_and_kth_error(i_tc[:sub], d_tc[:sub], i_ex, d_ex)


def unfused_quality(bk, points, queries, k, mode):
    # the tensor-core matrix ranks the candidates (k plus a margin), the exact re-ranking decides
    margin = max(8, k // 4)
    _, cand = bk.select(bk.l2(points, queries, mode=mode), k + margin)
    d_tc, i_tc = bk.refine(points, queries, cand, k)
    d_ex, i_ex = bk.select(bk.l2(points, queries, mode=bk.L2_EXACT), k)
    torch.cuda.synchronize()
    bk.device_status()
    return recall_and_kth_error(i_tc, d_tc, i_ex, d_ex)


@pytest.mark.parametrize("kind", ["uniform", "clustered"])
@pytest.mark.parametrize("mode_name", ["tf32", "bf16"])
@pytest.mark.parametrize("dim", [4, 16, 64])
def test_fused_tc_at_two_to_the_twenty_points(bk, cuda, kind, mode_name, dim):
    mode = bk.L2_TF32 if mode_name == "tf32" else bk.L2_BF16
    n, q, sub = 1 << 20, 1 << 14, 512
    points, queries = make_data(kind, n, q, dim, seed=dim * 7 + (1 if kind == "uniform" else 2))
    for k in (4, 32, 128):
        recall, rel = fused_quality(bk, points, queries, k, mode, sub)
        assert recall >= MIN_RECALL, (kind, mode_name, dim, k, recall)
        assert rel <= MAX_KTH_REL, (kind, mode_name, dim, k, rel)


@pytest.mark.parametrize("kind", ["uniform", "clustered"])
@pytest.mark.parametrize("mode_name", ["tf32", "bf16"])
@pytest.mark.parametrize("dim,ks", [(4, (4, 32, 128)), (16, (4, 32, 128)), (32, (64,)), (64, (4, 32, 64, 128)),
                                    (128, (64,))])
def test_distance_matrix_tc_then_bits_at_two_to_the_twenty_points(bk, cuda, kind, mode_name, dim, ks):
    """The unfused pipeline: tensor-core distance matrix, `bits` selection of k plus a margin,
    exact re-ranking of those candidates (`bitsknn_refine`)."""
    mode = bk.L2_TF32 if mode_name == "tf32" else bk.L2_BF16
    n, q = 1 << 20, 512                             # 2 GiB per matrix
    points, queries = make_data(kind, n, q, dim, seed=dim * 11 + (3 if kind == "uniform" else 4))
    for k in ks:
        recall, rel = unfused_quality(bk, points, queries, k, mode)
        assert recall >= MIN_RECALL, (kind, mode_name, dim, k, recall)
        assert rel <= MAX_KTH_REL, (kind, mode_name, dim, k, rel)


def test_fused_tc_on_one_shard_of_the_largest_configuration(bk, cuda):
    n, q, dim, k, sub = 1 << 24, 1 << 14, 64, 128, 256
    points, queries = make_data("uniform", n, q, dim, seed=1000)
    recall, rel = fused_quality(bk, points, queries, k, bk.L2_BF16, sub)
    assert recall >= MIN_RECALL, recall
    assert rel <= MAX_KTH_REL, rel
