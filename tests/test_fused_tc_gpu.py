"""`bits-fused` tensor-core modes (tcgen05 MMA into tensor memory feeding the top-k directly)
against the FP32 fused path.  Tolerances stated for these modes: recall@k >= 0.999 and
relative error of the k-th distance <= 1e-3.  Structural properties are exact: ascending
distances, valid distinct indices, reported distance consistent with the reported index."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def check_against_fp32(bk, points, queries, k, mode, index_base=0, min_recall=0.999, max_rel=1e-3):
    d_tc, i_tc = bk.fused(points, queries, k, mode=mode, index_base=index_base)
    torch.cuda.synchronize()
    bk.device_status()
    d_ex, i_ex = bk.fused(points, queries, k, mode=bk.L2_EXACT, index_base=index_base)
    n = points.shape[0]
    kk = min(k, n)
    # structure
    assert bool((d_tc[:, 1:kk] >= d_tc[:, :kk - 1]).all())
    local = (i_tc[:, :kk] - index_base).long()
    assert bool(((local >= 0) & (local < n)).all())
    srt = torch.sort(local, dim=1).values
    assert bool((srt[:, 1:] != srt[:, :-1]).all()), "duplicate indices in a result"
    # reported distance belongs to the reported index (FP32 recomputation)
    diff = queries[:, None, :] - points[local]
    true_d = (diff * diff).sum(-1)
    scale = true_d.abs().max().item() + 1.0
    assert (d_tc[:, :kk] - true_d).abs().max().item() <= 2e-3 * scale
    # quality
    a, b = i_tc[:, :kk].cpu().numpy(), i_ex[:, :kk].cpu().numpy()
    hits = sum(len(np.intersect1d(a[r], b[r])) for r in range(a.shape[0]))
    recall = hits / a.size
    rel = ((d_tc[:, kk - 1] - d_ex[:, kk - 1]).abs() / d_ex[:, kk - 1].abs().clamp_min(1e-6)).max().item()
    assert recall >= min_recall, recall
    assert rel <= max_rel, rel


@pytest.mark.parametrize("mode_name,dim", [("tf32", 4), ("tf32", 16), ("tf32", 32), ("tf32", 64), ("bf16", 8),
                                           ("bf16", 32), ("bf16", 64), ("bf16", 128), ("tf32", 100), ("bf16", 200),
                                           ("bf16", 19), ("tf32", 13)])
@pytest.mark.parametrize("k", [16, 128])
def test_quality_versus_fp32(bk, cuda, mode_name, dim, k):
    mode = bk.L2_TF32 if mode_name == "tf32" else bk.L2_BF16
    gen = torch.Generator(device="cuda").manual_seed(dim * 1000 + k)
    points = torch.rand((50000, dim), generator=gen, device="cuda")
    queries = torch.rand((300, dim), generator=gen, device="cuda")
    check_against_fp32(bk, points, queries, k, mode)


@pytest.mark.parametrize("mode_name", ["tf32", "bf16"])
def test_mma_width_does_not_change_the_result(bk, cuda, mode_name):
    # 256 points per MMA (two accumulators at once) and 128 points per MMA run the same arithmetic
    mode = bk.L2_TF32 if mode_name == "tf32" else bk.L2_BF16
    gen = torch.Generator(device="cuda").manual_seed(256)
    points = torch.rand((30001, 24), generator=gen, device="cuda")
    queries = torch.rand((200, 24), generator=gen, device="cuda")
    old = bk.get_tuning("fused.tc_mma_n")
    try:
        bk.set_tuning("fused.tc_mma_n", 128)
        d_narrow, i_narrow = bk.fused(points, queries, 40, mode=mode)
        bk.set_tuning("fused.tc_mma_n", 0)
        d_wide, i_wide = bk.fused(points, queries, 40, mode=mode)
    finally:
        bk.set_tuning("fused.tc_mma_n", old)
    torch.cuda.synchronize()
    bk.device_status()
    assert torch.equal(i_narrow, i_wide) and torch.equal(d_narrow, d_wide)
    check_against_fp32(bk, points, queries, 40, mode)


def test_plain_image_for_long_vectors(bk, cuda):
    # beyond 120 (TF32) / 240 (BF16) coordinates the hi/lo split no longer fits the resident query
    # tile and the image is the plainly rounded row: same structure, looser agreement
    gen = torch.Generator(device="cuda").manual_seed(150)
    points = torch.rand((20000, 150), generator=gen, device="cuda")
    queries = torch.rand((200, 150), generator=gen, device="cuda")
    check_against_fp32(bk, points, queries, 32, bk.L2_TF32, min_recall=0.9, max_rel=1e-2)


@pytest.mark.parametrize("n,q,k", [(1000, 1, 32), (129, 129, 64), (128, 128, 128), (5000, 257, 100), (20001, 64, 256),
                                   (40, 3, 64)])
def test_ragged_shapes(bk, cuda, n, q, k):
    gen = torch.Generator(device="cuda").manual_seed(n + q + k)
    points = torch.rand((n, 16), generator=gen, device="cuda")
    queries = torch.rand((q, 16), generator=gen, device="cuda")
    check_against_fp32(bk, points, queries, k, bk.L2_TF32, index_base=1000)


def test_few_queries_long_database_is_cut_into_parts(bk, cuda):
    # 3 queries, 2^19 points: one query tile, so the database is split over many blocks and the
    # per-part lists are merged
    gen = torch.Generator(device="cuda").manual_seed(77)
    points = torch.rand(((1 << 19) + 5, 24), generator=gen, device="cuda")
    queries = torch.rand((3, 24), generator=gen, device="cuda")
    check_against_fp32(bk, points, queries, 32, bk.L2_BF16)
    check_against_fp32(bk, points, queries, 200, bk.L2_TF32)


@pytest.mark.parametrize("mode_name", ["tf32", "bf16"])
def test_more_query_tiles_than_sms(bk, cuda, mode_name):
    # whole waves of query tiles scan the database whole, the tiles left over are cut into database
    # ranges: both kinds of blocks in one launch (a few more tiles than SMs), indices against FP32
    mode = bk.L2_TF32 if mode_name == "tf32" else bk.L2_BF16
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    q, n, dim, k = (sms + 2) * 128 - 37, 20000, 8, 16
    g = torch.Generator(device="cuda").manual_seed(5)
    points = torch.rand(n, dim, device="cuda", generator=g)
    queries = torch.rand(q, dim, device="cuda", generator=g)
    d_tc, i_tc = bk.fused(points, queries, k, mode=mode)
    d_ex, i_ex = bk.fused(points, queries, k, mode=bk.L2_EXACT)
    torch.cuda.synchronize()
    bk.device_status()
    same = (i_tc == i_ex).all(dim=1).float().mean().item()
    assert same >= 0.999, same
    assert bool((d_tc[:, 1:] >= d_tc[:, :-1]).all())


def test_many_parts_and_clustered_data(bk, cuda):
    # 2^18 points: several blocks per query tile; clustered data (256 centres, sigma 0.05)
    gen = torch.Generator(device="cuda").manual_seed(5)
    dim, n, q = 32, 1 << 18, 512
    centres = torch.rand((256, dim), generator=gen, device="cuda")
    pick = torch.randint(0, 256, (n,), generator=gen, device="cuda")
    points = centres[pick] + 0.05 * torch.randn((n, dim), generator=gen, device="cuda")
    pickq = torch.randint(0, 256, (q,), generator=gen, device="cuda")
    queries = centres[pickq] + 0.05 * torch.randn((q, dim), generator=gen, device="cuda")
    check_against_fp32(bk, points.contiguous(), queries.contiguous(), 32, bk.L2_BF16)


def test_workspace_and_dim_limits(bk, cuda):
    x = torch.rand((256, 16), device="cuda")
    # FP32: optional workspace (lists of the tiled kernel); without one the 8-query kernel runs
    d0, i0 = bk.fused(x, x, 32, mode=bk.L2_PARTIAL)
    lib = bk.lib()
    import ctypes
    d1 = torch.empty_like(d0)
    i1 = torch.empty_like(i0)
    rc = lib.bitsknn_fused(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 256, 256, 16, 32, bk.L2_PARTIAL, 0,
                           ctypes.c_void_p(d1.data_ptr()), ctypes.c_void_p(i1.data_ptr()), None, 0, None)
    torch.cuda.synchronize()
    assert rc == 0 and bool((d0 == d1).all()) and bool((i0 == i1).all())
    need = bk.fused_workspace_bytes(256, 256, 16, 32, bk.L2_TF32)
    assert need > 0
    with pytest.raises(bk.BitsKnnError) as err:
        bk.fused(x, x, 32, mode=bk.L2_TF32, workspace=torch.empty(256, dtype=torch.uint8, device="cuda"))
    assert err.value.status == bk.ERR_WORKSPACE
    big = torch.rand((64, 300), device="cuda")
    with pytest.raises(bk.BitsKnnError) as err:
        bk.fused(big, big, 8, mode=bk.L2_TF32)
    assert err.value.status == bk.ERR_UNSUPPORTED_DIM
