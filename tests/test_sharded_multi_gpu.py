"""The database-sharded search on two (or more) GPUs of one box, one process per GPU: the merged
result of `bitsknn_sharded_search_select` / `_submit_select` / `_search_fused` equals, bit for bit,
the unsharded search over the whole matrix / database on one GPU.  Skipped on a single-GPU box."""
import os
import pathlib
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = pathlib.Path(__file__).resolve().parents[1]


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    import __graft_entry__ as entry
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # only carries the NCCL id of the library
    bk = entry.load_package()
    from importlib import import_module
    sharded = import_module(entry.PKG_NAME + ".sharded")
    search = sharded.ShardedSearch(bk, rank, world)
    gen = torch.Generator(device="cuda").manual_seed(77)           # the same data on every rank
    q, n, k = 41, 100003, 96
    matrix = torch.randint(0, 3000, (q, n), generator=gen, device="cuda").to(torch.float32)   # ties across shards
    points = torch.rand((50001, 24), generator=gen, device="cuda")
    queries = torch.rand((130, 24), generator=gen, device="cuda")
    ok = True
    begin, end = sharded.shard_bounds(n, world, rank)
    want = bk.select(matrix, k)
    got = search.select(matrix[:, begin:end].contiguous(), k, begin)
    torch.cuda.synchronize()
    ok = ok and torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    # submit form: five searches over rolled matrices with their own outputs
    outs = []
    for shift in range(5):
        shard = torch.roll(matrix, shift, dims=0)[:, begin:end].contiguous()
        out = (torch.empty((q, k), device="cuda"), torch.empty((q, k), dtype=torch.int32, device="cuda"))
        search.submit_select(shard, k, begin, out=out)
        outs.append(out)
    search.drain()
    torch.cuda.synchronize()
    for shift in range(5):
        ok = ok and torch.equal(outs[shift][0], torch.roll(want[0], shift, dims=0))
        ok = ok and torch.equal(outs[shift][1], torch.roll(want[1], shift, dims=0))
    # fused search of the sharded database, FP32 (bit-exact) and tensor-core (re-ranked: same result here)
    pb, pe = sharded.shard_bounds(points.shape[0], world, rank)
    for mode in (bk.L2_PARTIAL, bk.L2_EXACT, bk.L2_BF16):
        want_k = bk.fused(points, queries, 40, mode=mode)
        got_k = search.knn(points[pb:pe].contiguous(), queries, 40, pb, mode=mode)
        torch.cuda.synchronize()
        ok = ok and torch.equal(got_k[0], want_k[0]) and torch.equal(got_k[1], want_k[1])
    bk.device_status()
    search.close()
    with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_or_more_gpus_agree_with_one(tmp_path, bk, cuda):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        assert (tmp_path / f"rank{rank}.txt").read_text() == "ok"
