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
        self._packs = {}
        self._pending = None   # (slot, work, q, k, device, out) of the search whose exchange is in flight
        self._submitted = 0

    def _buffers(self, q, k, device, slot=0):
        """One float32 buffer [2][q][k] for this rank's candidates (plane 0: distances, plane 1:
        the int32 labels, bit-cast) and one [world][2][q][k] for the gathered ones, so that the
        exchange is a single collective.  `slot` 0 / 1: the two sets a stream of searches alternates
        between."""
        key = (q, k, str(device), slot)
        if key not in self._packs:
            self._packs[key] = (torch.empty((2, q, k), dtype=torch.float32, device=device),
                                torch.empty((self.world, 2, q, k), dtype=torch.float32, device=device))
        return self._packs[key]

    def local_views(self, q, k, device, slot=0):
        """(distances, labels) views of the local candidate buffer: kernels write straight into it."""
        local, _ = self._buffers(q, k, device, slot)
        return local[0], local.view(torch.int32)[1]

    def _exchange_and_merge(self, q, k, device, out=None):
        local, gathered = self._buffers(q, k, device)
        if self.world == 1:
            return local[0], local.view(torch.int32)[1]
        import torch.distributed as dist
        # (world*2*q, k) / (2*q, k) views: the concatenated form every backend accepts
        dist.all_gather_into_tensor(gathered.view(self.world * 2 * q, k), local.view(2 * q, k), group=self.group)
        return self.kernels.merge_strided(gathered[:, 0], gathered.view(torch.int32)[:, 1], list_stride=2 * q * k,
                                          query_stride=k, q=q, lists=self.world, k=k, out=out)

    def select(self, local_matrix, k, shard_begin, offsets=None, out=None):
        """Top-k of the rows of the full matrix whose columns [shard_begin, ...) this rank holds."""
        q = local_matrix.shape[0]
        if offsets is None:
            offsets = torch.full((q,), shard_begin, dtype=torch.int32, device=local_matrix.device)
        views = self.local_views(q, k, local_matrix.device)
        self.kernels.select(local_matrix, k, label_offsets=offsets, out=views)
        return self._exchange_and_merge(q, k, local_matrix.device, out=out)

    # ---- a stream of searches: the exchange of one overlaps the local selection of the next ----
    def submit_select(self, local_matrix, k, shard_begin, offsets=None, out=None, events=None):
        """Queues one search like `select`, but leaves its all-gather in flight and finishes (merges)
        the search submitted before it, whose result is returned (None for the first call).  The
        searches alternate between two buffer sets; `drain()` finishes the last one.  `events`: an
        optional (start, end) pair of CUDA events recorded around the local selection kernel."""
        q = local_matrix.shape[0]
        device = local_matrix.device
        if offsets is None:
            offsets = torch.full((q,), shard_begin, dtype=torch.int32, device=device)
        if self.world == 1:
            views = self.local_views(q, k, device)
            if events is not None:
                events[0].record()
            self.kernels.select(local_matrix, k, label_offsets=offsets, out=views if out is None else out)
            if events is not None:
                events[1].record()
            return views if out is None else out
        import torch.distributed as dist
        slot = self._submitted & 1
        self._submitted += 1
        local, gathered = self._buffers(q, k, device, slot)
        if events is not None:
            events[0].record()
        self.kernels.select(local_matrix, k, label_offsets=offsets, out=(local[0], local.view(torch.int32)[1]))
        if events is not None:
            events[1].record()
        work = dist.all_gather_into_tensor(gathered.view(self.world * 2 * q, k), local.view(2 * q, k), group=self.group,
                                           async_op=True)
        previous = self.drain()
        self._pending = (slot, work, q, k, device, out)
        return previous

    def drain(self):
        """Finishes the search whose exchange is in flight; returns its (distances, labels) or None."""
        if self._pending is None:
            return None
        slot, work, q, k, device, out = self._pending
        self._pending = None
        work.wait()
        _, gathered = self._buffers(q, k, device, slot)
        return self.kernels.merge_strided(gathered[:, 0], gathered.view(torch.int32)[:, 1], list_stride=2 * q * k,
                                          query_stride=k, q=q, lists=self.world, k=k, out=out)

    def knn(self, local_points, queries, k, shard_begin, out=None, **kw):
        """k nearest points of the full database for every query; this rank holds
        points [shard_begin, shard_begin + len(local_points))."""
        q = queries.shape[0]
        views = self.local_views(q, k, queries.device)
        self.kernels.fused(local_points, queries, k, index_base=shard_begin, out=views, **kw)
        return self._exchange_and_merge(q, k, queries.device, out=out)
