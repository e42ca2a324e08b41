"""Parity of the FP32 distance kernels with the CPU oracle: bit-exact (same FMA chain per
output as the reference's abstract_gemm).  Shapes follow the reference's distance tests
(tests/distance/magma_dist_test.cpp:7-96: 32x32x16, 128x1x16, dim 9, partial 1024x32x32,
23*1024 x 1 x 17)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(32, 32, 16), (128, 1, 16), (100, 7, 9), (1024, 32, 32), (23 * 1024, 1, 17), (1, 1, 1), (129, 130, 1),
          (997, 43, 37), (513, 257, 64), (300, 5, 128), (2000, 3, 200), (255, 129, 4), (4097, 2, 8)]


@pytest.mark.parametrize("n,q,dim", SHAPES)
@pytest.mark.parametrize("partial", [False, True])
def test_distance_matrix_bit_exact(bk, oracle, cuda, n, q, dim, partial):
    points, queries = oracle.generate("uniform", 42, n, q, dim)
    want = oracle.l2(points, queries, partial=partial)
    got = bk.l2(torch.from_numpy(points).cuda(), torch.from_numpy(queries).cuda(),
                mode=bk.L2_PARTIAL if partial else bk.L2_EXACT)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_normal_data_and_padded_output(bk, oracle, cuda):
    points, queries = oracle.generate("normal", 7, 777, 33, 19, 0.5, 2.0)
    want = oracle.l2(points, queries)
    out = torch.full((33, 777 + 5), -1.0, device="cuda")
    bk.l2(torch.from_numpy(points).cuda(), torch.from_numpy(queries).cuda(), out=out[:, :777])
    torch.cuda.synchronize()
    res = out.cpu().numpy()
    assert np.array_equal(res[:, :777], want)
    assert np.all(res[:, 777:] == -1.0)          # nothing written past n


def test_distance_then_selection_matches_reference_pipeline(bk, oracle, cuda):
    # `knn -a bits`: magma-dist (full L2) followed by the bits selection
    points, queries = oracle.generate("uniform", 42, 20000, 64, 10)
    dist = bk.l2(torch.from_numpy(points).cuda(), torch.from_numpy(queries).cuda())
    d, i = bk.select(dist, 64)
    want_d, want_i = oracle.knn(points, queries, 64, partial=False)
    assert np.array_equal(d.cpu().numpy(), want_d) and np.array_equal(i.cpu().numpy(), want_i)


def test_unsupported_modes_report_errors(bk, cuda):
    x = torch.zeros((8, 4), device="cuda")
    with pytest.raises(bk.BitsKnnError) as err:
        bk.l2(x, x, mode=17)
    assert err.value.status == bk.ERR_UNSUPPORTED_MODE
