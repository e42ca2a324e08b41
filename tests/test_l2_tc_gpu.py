"""Tensor-core distance modes (tcgen05, TF32 / BF16 inputs, FP32 accumulation) against the
FP32 exact path.  Tolerances (the ones the task states for these modes): recall@k >= 0.999
and relative error of the k-th distance <= 1e-3, k = 64; plus an element-wise bound on the
matrix itself that follows from the input rounding (2^-11 per TF32 operand, 2^-8 per BF16
operand)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def exact_matrix(bk, points, queries):
    return bk.l2(points, queries, mode=bk.L2_EXACT)


@pytest.mark.parametrize("n,q,dim", [(20000, 300, 64), (4096, 128, 32), (5000, 129, 128), (3001, 77, 20), (1000, 5, 4),
                                     (128, 128, 256)])
@pytest.mark.parametrize("mode_name", ["tf32", "bf16"])
def test_matrix_close_to_fp32(bk, cuda, n, q, dim, mode_name):
    mode = bk.L2_TF32 if mode_name == "tf32" else bk.L2_BF16
    gen = torch.Generator(device="cuda").manual_seed(n + dim)
    points = torch.rand((n, dim), generator=gen, device="cuda")
    queries = torch.rand((q, dim), generator=gen, device="cuda")
    got = bk.l2(points, queries, mode=mode)
    torch.cuda.synchronize()
    bk.device_status()
    want = exact_matrix(bk, points, queries)
    # |x.y| <= dim for coordinates in [0,1); each product carries two input roundings (the
    # compensated images of small dims are far more accurate; this is the plain-mode bound)
    eps = 2.0 ** -11 if mode_name == "tf32" else 2.0 ** -8
    bound = 2.0 * (2.0 * eps) * dim * 0.6 + 1e-4
    err = (got - want).abs().max().item()
    assert err <= bound, (err, bound)


@pytest.mark.parametrize("mode_name,dim", [("tf32", 32), ("tf32", 64), ("bf16", 32), ("bf16", 64), ("bf16", 128)])
def test_knn_quality(bk, cuda, mode_name, dim):
    """recall@64 >= 0.999 and relative error of the 64th distance <= 1e-3 versus FP32."""
    mode = bk.L2_TF32 if mode_name == "tf32" else bk.L2_BF16
    gen = torch.Generator(device="cuda").manual_seed(dim)
    n, q, k = 1 << 16, 1024, 64
    points = torch.rand((n, dim), generator=gen, device="cuda")
    queries = torch.rand((q, dim), generator=gen, device="cuda")
    d_tc, i_tc = bk.select(bk.l2(points, queries, mode=mode), k)
    d_ex, i_ex = bk.select(exact_matrix(bk, points, queries), k)
    torch.cuda.synchronize()
    hits = 0
    a, b = i_tc.cpu().numpy(), i_ex.cpu().numpy()
    for r in range(q):
        hits += len(np.intersect1d(a[r], b[r]))
    recall = hits / (q * k)
    rel = ((d_tc[:, -1] - d_ex[:, -1]).abs() / d_ex[:, -1]).max().item()
    assert recall >= 0.999, recall
    assert rel <= 1e-3, rel


def test_workspace_is_checked(bk, cuda):
    x = torch.rand((256, 32), device="cuda")
    need = bk.l2_workspace_bytes(256, 256, 32, bk.L2_TF32)
    assert need > 0
    small = torch.empty(need - 256, dtype=torch.uint8, device="cuda")
    with pytest.raises(bk.BitsKnnError) as err:
        bk.l2(x, x, mode=bk.L2_TF32, workspace=small)
    assert err.value.status == bk.ERR_WORKSPACE
    with pytest.raises(bk.BitsKnnError) as err:
        bk.l2(torch.rand((8, 300), device="cuda"), torch.rand((8, 300), device="cuda"), mode=bk.L2_TF32)
    assert err.value.status == bk.ERR_UNSUPPORTED_DIM
