"""World-size-2 (and 3) CPU test of the database-sharded search: gloo ranks, the kernels
replaced by the CPU oracle, result compared with the unsharded oracle answer.  What is under
test is the host logic: shard bounds, global labels, gather layout, merge call."""
import os
import socket
import sys
import pathlib

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = pathlib.Path(__file__).resolve().parents[1]


class OracleKernels:
    """Stand-in for the CUDA access layer, on CPU tensors."""

    def __init__(self):
        from oracle import oracle
        self.oracle = oracle

    def select(self, dist, k, label_offsets=None, out=None):
        d, i = self.oracle.select(dist.numpy(), k, label_offsets=None if label_offsets is None else label_offsets.numpy())
        out[0].copy_(torch.from_numpy(d))
        out[1].copy_(torch.from_numpy(i))
        return out

    def fused(self, points, queries, k, index_base=0, out=None):
        d, i = self.oracle.knn(points.numpy(), queries.numpy(), k, partial=True, index_base=index_base)
        out[0].copy_(torch.from_numpy(d))
        out[1].copy_(torch.from_numpy(i))
        return out

    def merge_strided(self, cand_d, cand_i, list_stride, query_stride, q, lists, k, out=None):
        # strided views of the gathered buffer -> (lists, q, k) arrays for the oracle
        assert cand_d.shape == (lists, q, k) and cand_d.stride() == (list_stride, query_stride, 1)
        assert cand_i.shape == (lists, q, k) and cand_i.stride() == (list_stride, query_stride, 1)
        d, i = self.oracle.merge(np.ascontiguousarray(cand_d.numpy()), np.ascontiguousarray(cand_i.numpy()))
        return torch.from_numpy(d), torch.from_numpy(i)


def _worker(rank, world, port, n, q, k, result_dir):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    import __graft_entry__ as entry
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = entry.load_package()
    from importlib import import_module
    sharded = import_module(entry.PKG_NAME + ".sharded")
    rng = np.random.default_rng(99)
    matrix = rng.integers(0, 500, size=(q, n)).astype(np.float32)       # many ties across shards
    points = rng.random((n, 5), dtype=np.float32)
    queries = rng.random((q, 5), dtype=np.float32)
    begin, end = sharded.shard_bounds(n, world, rank)
    search = sharded.ShardedSearch(OracleKernels(), rank, world)
    sd, si = search.select(torch.from_numpy(np.ascontiguousarray(matrix[:, begin:end])), k, begin)
    kd, ki = search.knn(torch.from_numpy(points[begin:end]), torch.from_numpy(queries), k, begin)
    # a stream of three searches over shifted matrices: submit returns the previous search's result
    stream_out = []
    for step in range(3):
        shifted = np.ascontiguousarray(np.roll(matrix, step, axis=0)[:, begin:end])
        done = search.submit_select(torch.from_numpy(shifted), k, begin)
        assert (done is None) == (step == 0)
        if done is not None:
            stream_out.append((done[0].numpy().copy(), done[1].numpy().copy()))
    done = search.drain()
    stream_out.append((done[0].numpy().copy(), done[1].numpy().copy()))
    assert search.drain() is None
    np.savez(os.path.join(result_dir, f"rank{rank}.npz"), sd=sd.numpy(), si=si.numpy(), kd=kd.numpy(), ki=ki.numpy(),
             matrix=matrix, points=points, queries=queries,
             pd=np.stack([d for d, _ in stream_out]), pi=np.stack([i for _, i in stream_out]))
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_bounds_cover_the_database():
    import __graft_entry__ as entry
    entry.load_package()
    from importlib import import_module
    sharded = import_module(entry.PKG_NAME + ".sharded")
    for n in (1, 7, 8, 1000, (1 << 27)):
        for world in (1, 2, 3, 8):
            bounds = [sharded.shard_bounds(n, world, r) for r in range(world)]
            assert bounds[0][0] == 0 and bounds[-1][1] == n
            assert all(bounds[r][1] == bounds[r + 1][0] for r in range(world - 1))
            sizes = [e - b for b, e in bounds]
            assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_search_equals_unsharded(tmp_path, oracle, world):
    n, q, k = 1003, 9, 16
    mp.spawn(_worker, args=(world, _free_port(), n, q, k, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        got = np.load(tmp_path / f"rank{rank}.npz")
        want_d, want_i = oracle.select(got["matrix"], k)
        assert np.array_equal(got["sd"], want_d) and np.array_equal(got["si"], want_i)
        want_d, want_i = oracle.knn(got["points"], got["queries"], k, partial=True)
        assert np.array_equal(got["kd"], want_d) and np.array_equal(got["ki"], want_i)
        for step in range(3):
            want_d, want_i = oracle.select(np.roll(got["matrix"], step, axis=0), k)
            assert np.array_equal(got["pd"][step], want_d) and np.array_equal(got["pi"][step], want_i)
