"""The allocation-free split-row selection gives the same result as the variant that takes a
caller workspace.  Runs last (file name), so a stop at the first failure has already run
every other test; passes alone in a fresh process as well."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_selection_matches_workspace_selection(bk, cuda):
    assert bk.STATIC_SCRATCH_BYTES == 8 << 20
    gen = torch.Generator(device="cuda").manual_seed(1234)
    # two different problems back to back: the second call finds the first call's candidates
    # in the shared array and must not be affected by them
    cases = [(64, 200003, 128, 8), (16, 65536, 2048, 4), (64, 200003, 128, 8)]
    for q, n, k, splits in cases:
        dist = torch.randint(0, 100000, (q, n), generator=gen, device="cuda").to(torch.float32)
        want_d, want_i = bk.select_split(dist, k, splits=splits)
        out = (torch.full((q, k), -1.0, device="cuda"), torch.full((q, k), -1, dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        bk.select_split_static(dist, k, splits, out=out)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before        # nothing came from torch's allocator
        bk.device_status()
        # ... nor from the driver: after that warm call (the first call on a device loads the kernels
        # and looks up the array), a second call leaves the device's free memory where it was
        free_before = torch.cuda.mem_get_info()[0]
        bk.select_split_static(dist, k, splits, out=out)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert np.array_equal(out[0].cpu().numpy().view(np.uint32), want_d.cpu().numpy().view(np.uint32))
        assert np.array_equal(out[1].cpu().numpy(), want_i.cpu().numpy())


def test_static_scratch_rejects_oversized_problems(bk, cuda):
    dist = torch.zeros((4096, 4096), device="cuda")
    out = (torch.empty((4096, 1024), device="cuda"), torch.empty((4096, 1024), dtype=torch.int32, device="cuda"))
    with pytest.raises(bk.BitsKnnError) as err:
        bk.select_split_static(dist, 1024, 2, out=out)      # 4096*2*1024 pairs = 64 MiB > 8 MiB
    assert err.value.status == bk.ERR_WORKSPACE
    assert "built-in scratch" in err.value.message
