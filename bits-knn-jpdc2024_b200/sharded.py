"""Database-sharded search over several GPUs (one process per GPU, torch.distributed).

Every rank holds a contiguous shard of the database -- columns [begin, end) of the distance
matrix, or points [begin, end) -- and the full set of queries.  A search is: local top-k on
the shard with global labels (label offset / index base = `begin`, the mechanism the
reference uses for row slices, src/topk/singlepass/bits_knn.cu:67-76), an all-gather of the
q x k candidate pairs of every rank (NCCL over NVLink on GPUs; 8 bytes per pair), and the
bitonic merge kernel over the `world` lists of each query.  The reference is single-GPU;
its split-row two-pass scheme (bits_knn.cu:116-186) is the template for this exchange.

`kernels` is the access layer of the C-ABI library (select / fused / merge on CUDA tensors).
The CPU tests of this module pass a stand-in with the same three functions so that the
sharding arithmetic and the gather layout can be exercised with the gloo backend.
"""
import torch


def shard_bounds(n, world, rank):
    """Contiguous, nearly equal shards: the first n % world shards hold one element more."""
    base, extra = divmod(n, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class ShardedSearch:
    def __init__(self, kernels, rank=0, world=1, group=None):
        self.kernels = kernels
        self.rank = rank
        self.world = world
        self.group = group
        self._gather = {}

    def _buffers(self, q, k, device):
        key = (q, k, str(device))
        if key not in self._gather:
            self._gather[key] = (torch.empty((self.world, q, k), dtype=torch.float32, device=device),
                                 torch.empty((self.world, q, k), dtype=torch.int32, device=device))
        return self._gather[key]

    def _exchange_and_merge(self, local_d, local_i, out=None):
        if self.world == 1:
            return local_d, local_i
        import torch.distributed as dist
        q, k = local_d.shape
        all_d, all_i = self._buffers(q, k, local_d.device)
        # (world*q, k) output view: the concatenated form every backend accepts
        dist.all_gather_into_tensor(all_d.view(self.world * q, k), local_d.contiguous(), group=self.group)
        dist.all_gather_into_tensor(all_i.view(self.world * q, k), local_i.contiguous(), group=self.group)
        return self.kernels.merge(all_d, all_i, out=out)

    def select(self, local_matrix, k, shard_begin, offsets=None, local_out=None, out=None):
        """Top-k of the rows of the full matrix whose columns [shard_begin, ...) this rank holds."""
        q = local_matrix.shape[0]
        if offsets is None:
            offsets = torch.full((q,), shard_begin, dtype=torch.int32, device=local_matrix.device)
        d, i = self.kernels.select(local_matrix, k, label_offsets=offsets, out=local_out)
        return self._exchange_and_merge(d, i, out=out)

    def knn(self, local_points, queries, k, shard_begin, local_out=None, out=None, **kw):
        """k nearest points of the full database for every query; this rank holds
        points [shard_begin, shard_begin + len(local_points))."""
        d, i = self.kernels.fused(local_points, queries, k, index_base=shard_begin, out=local_out, **kw)
        return self._exchange_and_merge(d, i, out=out)
