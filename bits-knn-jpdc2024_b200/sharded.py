"""Database-sharded search over several GPUs, one process per GPU: the test and benchmark harness
over the C-ABI entry points `bitsknn_sharded_*`.

Every rank holds a contiguous shard of the database -- columns [begin, end) of the distance
matrix, or points [begin, end) -- and the full set of queries.  A search is: local top-k on
the shard with global labels (label base / index base = `begin`, the mechanism the
reference uses for row slices, src/topk/singlepass/bits_knn.cu:67-76), an all-gather of the
q x k candidate pairs of every rank (8 bytes per pair), and the bitonic merge kernel over the
`world` lists of each query.  The reference is single-GPU; its split-row two-pass scheme
(bits_knn.cu:116-186) is the template for this exchange.

Two back ends behind one interface:
  * native (CUDA tensors, `kernels` = the access layer of the C-ABI library): the library runs the
    exchange itself -- NCCL all-gather and merge on a stream of its handle.  torch.distributed is
    only used once, to hand the NCCL unique id of rank 0 to the other ranks;
  * host logic (CPU tests): `kernels` is a stand-in with select / fused / merge_strided on CPU
    tensors and the all-gather goes through torch.distributed (gloo), with the same shard bounds,
    labels and packed layout [world][2][q][k] (plane 0: distances, plane 1: the int32 labels'
    bit patterns).
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
        self.native = hasattr(kernels, "sharded_create") and torch.cuda.is_available()
        self.handle = None
        self._ws = {}
        self._packs = {}
        self._pending = None   # host-logic back end: the search whose exchange is in flight
        self._previous = None  # native back end: output of the search submitted last
        self._submitted = 0
        if self.native:
            uid = None
            if world > 1:
                import torch.distributed as dist
                box = [kernels.sharded_unique_id() if rank == 0 else None]
                dist.broadcast_object_list(box, src=0, group=group)
                uid = box[0]
            self.handle = kernels.sharded_create(uid, rank, world)

    def close(self):
        if self.handle is not None:
            torch.cuda.synchronize()
            self.kernels.sharded_destroy(self.handle)
            self.handle = None

    # ---- native back end -----------------------------------------------------------------
    def _workspace(self, q, k, device):
        key = (q, k, str(device))
        if key not in self._ws:
            need = self.kernels.sharded_workspace_bytes(self.handle, q, k)
            self._ws[key] = torch.empty(max(need, 16), dtype=torch.uint8, device=device) if need > 0 else None
        return self._ws[key]

    # ---- host-logic back end ---------------------------------------------------------------
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

    def _local_views(self, q, k, device, slot=0):
        local, _ = self._buffers(q, k, device, slot)
        return local[0], local.view(torch.int32)[1]

    def _merge_gathered(self, q, k, device, slot, out):
        _, gathered = self._buffers(q, k, device, slot)
        return self.kernels.merge_strided(gathered[:, 0], gathered.view(torch.int32)[:, 1], list_stride=2 * q * k,
                                          query_stride=k, q=q, lists=self.world, k=k, out=out)

    def _exchange_and_merge(self, q, k, device, out=None):
        local, gathered = self._buffers(q, k, device)
        if self.world == 1:
            return local[0], local.view(torch.int32)[1]
        import torch.distributed as dist
        # (world*2*q, k) / (2*q, k) views: the concatenated form every backend accepts
        dist.all_gather_into_tensor(gathered.view(self.world * 2 * q, k), local.view(2 * q, k), group=self.group)
        return self._merge_gathered(q, k, device, 0, out)

    # ---- searches ------------------------------------------------------------------------
    def select(self, local_matrix, k, shard_begin, out=None):
        """Top-k of the rows of the full matrix whose columns [shard_begin, ...) this rank holds."""
        q = local_matrix.shape[0]
        device = local_matrix.device
        if self.native:
            return self.kernels.sharded_select(self.handle, local_matrix, k, shard_begin, self._workspace(q, k, device),
                                               out=out)
        offsets = torch.full((q,), shard_begin, dtype=torch.int32, device=device)
        self.kernels.select(local_matrix, k, label_offsets=offsets, out=self._local_views(q, k, device))
        return self._exchange_and_merge(q, k, device, out=out)

    def submit_select(self, local_matrix, k, shard_begin, out=None, events=None):
        """Queues one search like `select` but does not wait for its exchange and merge, which
        overlap the local kernel of the next search (two buffer sets); returns the output of the
        search submitted before it (None for the first call).  `drain()` finishes everything; with
        the native back end a returned output is only complete after `drain()`.  `events`: an
        optional (start, end) pair of CUDA events recorded around the local selection kernel."""
        q = local_matrix.shape[0]
        device = local_matrix.device
        if self.native:
            if events is not None:
                events[0].record()
            result = self.kernels.sharded_select(self.handle, local_matrix, k, shard_begin,
                                                 self._workspace(q, k, device), out=out, wait=False)
            if events is not None:
                events[1].record()
            previous, self._previous = self._previous, result
            return previous
        offsets = torch.full((q,), shard_begin, dtype=torch.int32, device=device)
        if self.world == 1:
            views = self._local_views(q, k, device)
            self.kernels.select(local_matrix, k, label_offsets=offsets, out=views if out is None else out)
            previous, self._previous = self._previous, (views if out is None else out)
            return previous
        import torch.distributed as dist
        slot = self._submitted & 1
        self._submitted += 1
        local, gathered = self._buffers(q, k, device, slot)
        self.kernels.select(local_matrix, k, label_offsets=offsets, out=(local[0], local.view(torch.int32)[1]))
        work = dist.all_gather_into_tensor(gathered.view(self.world * 2 * q, k), local.view(2 * q, k), group=self.group,
                                           async_op=True)
        previous = self.drain()
        self._pending = (slot, work, q, k, device, out)
        return previous

    def drain(self):
        """Finishes the searches still in flight; returns the last one's (distances, labels) or None."""
        if self.native:
            self.kernels.sharded_drain(self.handle)
            previous, self._previous = self._previous, None
            return previous
        if self._pending is None:
            previous, self._previous = self._previous, None
            return previous
        slot, work, q, k, device, out = self._pending
        self._pending = None
        work.wait()
        return self._merge_gathered(q, k, device, slot, out)

    def knn(self, local_points, queries, k, shard_begin, out=None, **kw):
        """k nearest points of the full database for every query; this rank holds
        points [shard_begin, shard_begin + len(local_points))."""
        q = queries.shape[0]
        device = queries.device
        if self.native:
            return self.kernels.sharded_fused(self.handle, local_points, queries, k, shard_begin,
                                              self._workspace(q, k, device), out=out,
                                              mode=kw.get("mode", self.kernels.L2_PARTIAL),
                                              fused_workspace=kw.get("workspace"))
        self.kernels.fused(local_points, queries, k, index_base=shard_begin, out=self._local_views(q, k, device), **kw)
        return self._exchange_and_merge(q, k, device, out=out)
