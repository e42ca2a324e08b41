"""Python access to the bitsknn C ABI (libbitsknn.so), for the tests and the benchmark.

The product is the C-ABI library (include/bitsknn.h) and the C++ host layer above it; this
module only passes torch tensors' device pointers through ctypes.  There is no fallback: if
the library has not been built, importing `lib()` raises.

The directory name is not a Python identifier; load it with `load_package()` from
`__graft_entry__.py` or `importlib` (tests/conftest.py does this).
"""
import ctypes
import pathlib

_PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libbitsknn.so"

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_UNSUPPORTED_K = 2
ERR_UNSUPPORTED_DIM = 3
ERR_WORKSPACE = 4
ERR_CUDA = 5
ERR_DEVICE_TIMEOUT = 6
ERR_UNSUPPORTED_MODE = 7
ERR_COMM = 8
SHARDED_ID_BYTES = 128

L2_EXACT, L2_PARTIAL, L2_TF32, L2_BF16 = 0, 1, 2, 3
STATIC_SCRATCH_BYTES = 8 << 20  # BITSKNN_STATIC_SCRATCH_BYTES

# every symbol include/bitsknn.h declares, with its ctypes signature
_i64 = ctypes.c_int64
_int = ctypes.c_int
_ptr = ctypes.c_void_p
_sz = ctypes.c_size_t
SIGNATURES = {
    "bitsknn_version": (_int, []),
    "bitsknn_last_error_string": (ctypes.c_char_p, []),
    "bitsknn_device_status": (_int, [_ptr]),
    "bitsknn_selftest_bounded_wait": (_int, [_ptr]),
    "bitsknn_set_tuning": (_int, [ctypes.c_char_p, _int]),
    "bitsknn_get_tuning": (_int, [ctypes.c_char_p, ctypes.POINTER(_int)]),
    "bitsknn_tuning_key": (ctypes.c_char_p, [_int]),
    "bitsknn_kernel_ms": (_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_float)]),
    "bitsknn_select": (_int, [_ptr, _i64, _ptr, _i64, _ptr, _i64, _i64, _int, _ptr, _ptr, _ptr]),
    "bitsknn_select_ablation": (_int, [_ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr, _ptr]),
    "bitsknn_select_auto_splits": (_int, [_i64, _i64, _int]),
    "bitsknn_select_split_workspace_bytes": (_sz, [_i64, _int, _int]),
    "bitsknn_select_split": (_int, [_ptr, _i64, _ptr, _i64, _i64, _int, _int, _ptr, _sz, _ptr, _ptr, _ptr]),
    "bitsknn_select_split_static": (_int, [_ptr, _i64, _ptr, _i64, _i64, _int, _int, _ptr, _ptr, _ptr]),
    "bitsknn_merge": (_int, [_ptr, _ptr, _i64, _i64, _i64, _int, _int, _ptr, _ptr, _ptr]),
    "bitsknn_merge_lists": (_int, [_ptr, _ptr, _i64, _i64, _i64, _int, _int, _int, _ptr, _ptr, _ptr]),
    "bitsknn_refine": (_int, [_ptr, _ptr, _i64, _i64, _int, _ptr, _i64, _int, ctypes.c_int32, _int, _ptr, _ptr, _ptr]),
    "bitsknn_sharded_unique_id": (_int, [_ptr]),
    "bitsknn_sharded_create": (_int, [ctypes.POINTER(_ptr), _ptr, _int, _int]),
    "bitsknn_sharded_init": (_int, [ctypes.POINTER(_ptr), _ptr, _int, _int]),
    "bitsknn_sharded_destroy": (_int, [_ptr]),
    "bitsknn_sharded_workspace_bytes": (_sz, [_ptr, _i64, _int]),
    "bitsknn_sharded_search_select": (_int, [_ptr, _ptr, _i64, _i64, _i64, _int, ctypes.c_int32, _ptr, _ptr, _ptr, _sz,
                                             _ptr]),
    "bitsknn_sharded_submit_select": (_int, [_ptr, _ptr, _i64, _i64, _i64, _int, ctypes.c_int32, _ptr, _ptr, _ptr, _sz,
                                             _ptr]),
    "bitsknn_sharded_search_fused": (_int, [_ptr, _ptr, _ptr, _i64, _i64, _int, _int, _int, ctypes.c_int32, _ptr, _ptr,
                                            _ptr, _sz, _ptr, _sz, _ptr]),
    "bitsknn_sharded_drain": (_int, [_ptr, _ptr]),
    "bitsknn_l2_workspace_bytes": (_sz, [_i64, _i64, _int, _int]),
    "bitsknn_transpose": (_int, [_ptr, _i64, _i64, _ptr, _ptr]),
    "bitsknn_l2": (_int, [_ptr, _ptr, _i64, _i64, _int, _int, _ptr, _i64, _ptr, _sz, _ptr]),
    "bitsknn_fused_workspace_bytes": (_sz, [_i64, _i64, _int, _int, _int]),
    "bitsknn_fused": (_int, [_ptr, _ptr, _i64, _i64, _int, _int, _int, ctypes.c_int32, _ptr, _ptr, _ptr, _sz, _ptr]),
}

_LIB = None


class BitsKnnError(RuntimeError):
    """A non-zero status from the C ABI; `.status` holds the code."""

    def __init__(self, status, message):
        super().__init__(f"bitsknn status {status}: {message}")
        self.status = status
        self.message = message


def lib():
    """The loaded C-ABI library.  Raises if it has not been built (no CPU fallback exists)."""
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with bits-knn-jpdc2024_b200/build.py "
                               "(the k-NN kernels have no CPU fallback)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the header and the library diverge
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = handle
    return _LIB


def last_error():
    return lib().bitsknn_last_error_string().decode()


def _check(status):
    if status != OK:
        raise BitsKnnError(status, last_error())


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def set_tuning(key, value):
    _check(lib().bitsknn_set_tuning(key.encode(), int(value)))


def get_tuning(key):
    out = ctypes.c_int(0)
    _check(lib().bitsknn_get_tuning(key.encode(), ctypes.byref(out)))
    return out.value


def tuning_keys():
    keys = []
    while True:
        key = lib().bitsknn_tuning_key(len(keys))
        if key is None:
            return keys
        keys.append(key.decode())


def kernel_ms(name):
    """Device time of the last timed launch of that kernel (knob "profile.kernel_events" = 1)."""
    out = ctypes.c_float(0)
    _check(lib().bitsknn_kernel_ms(name.encode(), ctypes.byref(out)))
    return out.value


def device_status():
    _check(lib().bitsknn_device_status(_stream()))


def selftest_bounded_wait():
    _check(lib().bitsknn_selftest_bounded_wait(_stream()))


def _device_check(t, dtype, name):
    import torch
    if t is None:
        return
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (the library has no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}")
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must be contiguous in its last dimension")


def select(dist, k, labels=None, label_offsets=None, n=None, out=None):
    """k smallest (distance, index) pairs of every row of a (q, ld) float32 CUDA matrix."""
    import torch
    _device_check(dist, torch.float32, "dist")
    _device_check(labels, torch.int32, "labels")
    _device_check(label_offsets, torch.int32, "label_offsets")
    q = dist.shape[0]
    ld = dist.stride(0) if q > 1 else dist.shape[1]
    n = dist.shape[1] if n is None else n
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=dist.device),
               torch.empty((q, k), dtype=torch.int32, device=dist.device))
    ldl = 0 if labels is None else (labels.stride(0) if q > 1 else labels.shape[1])
    _check(lib().bitsknn_select(_p(dist), ld, _p(labels), ldl, _p(label_offsets), q, n, k,
                                _p(out[0]), _p(out[1]), _stream()))
    return out


ABLATION_NO_BUFFER, ABLATION_SHARED_LIST = 0, 1


def select_ablation(dist, k, variant, out=None):
    """The selection without its radius filter / with its list in shared memory (ablations)."""
    import torch
    _device_check(dist, torch.float32, "dist")
    q, n = dist.shape
    ld = dist.stride(0) if q > 1 else n
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=dist.device),
               torch.empty((q, k), dtype=torch.int32, device=dist.device))
    _check(lib().bitsknn_select_ablation(_p(dist), ld, q, n, k, variant, _p(out[0]), _p(out[1]), _stream()))
    return out


def select_auto_splits(q, n, k):
    return int(lib().bitsknn_select_auto_splits(q, n, k))


def select_split_workspace_bytes(q, k, splits):
    return int(lib().bitsknn_select_split_workspace_bytes(q, k, splits))


def select_split(dist, k, splits=0, label_offsets=None, workspace=None, out=None):
    import torch
    _device_check(dist, torch.float32, "dist")
    q, n = dist.shape
    ld = dist.stride(0) if q > 1 else n
    if workspace is None:
        workspace = torch.empty(max(select_split_workspace_bytes(q, k, splits), 8), dtype=torch.uint8,
                                device=dist.device)
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=dist.device),
               torch.empty((q, k), dtype=torch.int32, device=dist.device))
    _check(lib().bitsknn_select_split(_p(dist), ld, _p(label_offsets), q, n, k, splits, _p(workspace),
                                      workspace.numel(), _p(out[0]), _p(out[1]), _stream()))
    return out


def select_split_static(dist, k, splits, label_offsets=None, out=None):
    """Split-row selection whose candidate scratch is the library's built-in device array."""
    import torch
    _device_check(dist, torch.float32, "dist")
    q, n = dist.shape
    ld = dist.stride(0) if q > 1 else n
    if out is None:
        raise ValueError("pass the output tensors: this entry point is for callers that do not allocate")
    _check(lib().bitsknn_select_split_static(_p(dist), ld, _p(label_offsets), q, n, k, splits, _p(out[0]), _p(out[1]),
                                             _stream()))
    return out


def merge(cand_dist, cand_idx, out=None, sorted_lists=False):
    """cand_* of shape (lists, q, k), contiguous -> the k smallest pairs per query."""
    import torch
    _device_check(cand_dist, torch.float32, "cand_dist")
    _device_check(cand_idx, torch.int32, "cand_idx")
    lists, q, k = cand_dist.shape
    assert cand_dist.is_contiguous() and cand_idx.is_contiguous()
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=cand_dist.device),
               torch.empty((q, k), dtype=torch.int32, device=cand_dist.device))
    _check(lib().bitsknn_merge_lists(_p(cand_dist), _p(cand_idx), q * k, k, q, lists, k, 1 if sorted_lists else 0,
                                     _p(out[0]), _p(out[1]), _stream()))
    return out


def merge_strided(cand_dist, cand_idx, list_stride, query_stride, q, lists, k, out=None, sorted_lists=False):
    """Merge with explicit element strides: pair j of list l of query i at
    [l * list_stride + i * query_stride + j] from the first element of each tensor."""
    import torch
    _device_check(cand_dist, torch.float32, "cand_dist")
    _device_check(cand_idx, torch.int32, "cand_idx")
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=cand_dist.device),
               torch.empty((q, k), dtype=torch.int32, device=cand_dist.device))
    _check(lib().bitsknn_merge_lists(_p(cand_dist), _p(cand_idx), list_stride, query_stride, q, lists, k,
                                     1 if sorted_lists else 0, _p(out[0]), _p(out[1]), _stream()))
    return out


def refine(points, queries, cand_idx, k, index_base=0, out=None):
    """Exact FP32 re-ranking of (q, candidates) int32 candidate indices -> the k nearest by it."""
    import torch
    _device_check(points, torch.float32, "points")
    _device_check(queries, torch.float32, "queries")
    _device_check(cand_idx, torch.int32, "cand_idx")
    assert points.is_contiguous() and queries.is_contiguous()
    n, dim = points.shape
    q, cands = cand_idx.shape
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=points.device),
               torch.empty((q, k), dtype=torch.int32, device=points.device))
    _check(lib().bitsknn_refine(_p(points), _p(queries), n, q, dim, _p(cand_idx), cand_idx.stride(0) if q > 1 else cands,
                                cands, index_base, k, _p(out[0]), _p(out[1]), _stream()))
    return out


def l2_workspace_bytes(n, q, dim, mode):
    return int(lib().bitsknn_l2_workspace_bytes(n, q, dim, mode))


def l2(points, queries, mode=L2_EXACT, out=None, workspace=None):
    """(q, n) squared-L2 matrix of row-major (n, dim) points and (q, dim) queries."""
    import torch
    _device_check(points, torch.float32, "points")
    _device_check(queries, torch.float32, "queries")
    assert points.is_contiguous() and queries.is_contiguous()
    n, dim = points.shape
    q = queries.shape[0]
    if out is None:
        out = torch.empty((q, n), dtype=torch.float32, device=points.device)
    need = l2_workspace_bytes(n, q, dim, mode)
    if workspace is None and need > 0:
        workspace = torch.empty(need, dtype=torch.uint8, device=points.device)
    _check(lib().bitsknn_l2(_p(points), _p(queries), n, q, dim, mode, _p(out), out.stride(0) if q > 1 else n,
                            _p(workspace), 0 if workspace is None else workspace.numel(), _stream()))
    return out


def transpose(src, out=None):
    """(rows, cols) float32 CUDA matrix -> its (cols, rows) transpose, on the device."""
    import torch
    _device_check(src, torch.float32, "src")
    assert src.is_contiguous()
    rows, cols = src.shape
    if out is None:
        out = torch.empty((cols, rows), dtype=torch.float32, device=src.device)
    _check(lib().bitsknn_transpose(_p(src), rows, cols, _p(out), _stream()))
    return out


def fused_workspace_bytes(n, q, dim, k, mode):
    return int(lib().bitsknn_fused_workspace_bytes(n, q, dim, k, mode))


def fused(points, queries, k, mode=L2_PARTIAL, index_base=0, out=None, workspace=None):
    """Brute-force k-NN without materialising the distance matrix."""
    import torch
    _device_check(points, torch.float32, "points")
    _device_check(queries, torch.float32, "queries")
    assert points.is_contiguous() and queries.is_contiguous()
    n, dim = points.shape
    q = queries.shape[0]
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=points.device),
               torch.empty((q, k), dtype=torch.int32, device=points.device))
    need = fused_workspace_bytes(n, q, dim, k, mode)
    if workspace is None and need > 0:
        workspace = torch.empty(need, dtype=torch.uint8, device=points.device)
    _check(lib().bitsknn_fused(_p(points), _p(queries), n, q, dim, k, mode, index_base, _p(out[0]), _p(out[1]),
                               _p(workspace), 0 if workspace is None else workspace.numel(), _stream()))
    return out


# ---- database-sharded search (one handle per GPU; NCCL inside the library) --------------------
def sharded_unique_id():
    """An NCCL unique id (bytes) made on the calling rank; distribute it to the other ranks."""
    buf = ctypes.create_string_buffer(SHARDED_ID_BYTES)
    _check(lib().bitsknn_sharded_unique_id(buf))
    return buf.raw


def sharded_create(unique_id, rank, world):
    """Handle with its own communicator (collective over the ranks; the rank's device is current)."""
    handle = ctypes.c_void_p()
    buf = None if unique_id is None else ctypes.create_string_buffer(bytes(unique_id), SHARDED_ID_BYTES)
    _check(lib().bitsknn_sharded_create(ctypes.byref(handle), buf, rank, world))
    return handle


def sharded_destroy(handle):
    _check(lib().bitsknn_sharded_destroy(handle))


def sharded_workspace_bytes(handle, q, k):
    return int(lib().bitsknn_sharded_workspace_bytes(handle, q, k))


def _sharded_out(q, k, device, out):
    import torch
    if out is None:
        out = (torch.empty((q, k), dtype=torch.float32, device=device),
               torch.empty((q, k), dtype=torch.int32, device=device))
    return out


def sharded_select(handle, dist, k, shard_begin, workspace, out=None, wait=True):
    """One sharded selection; `wait=False` is the submit form (finish with `sharded_drain`)."""
    import torch
    _device_check(dist, torch.float32, "dist")
    q, n = dist.shape
    ld = dist.stride(0) if q > 1 else n
    out = _sharded_out(q, k, dist.device, out)
    fn = lib().bitsknn_sharded_search_select if wait else lib().bitsknn_sharded_submit_select
    _check(fn(handle, _p(dist), ld, q, n, k, shard_begin, _p(out[0]), _p(out[1]), _p(workspace),
              0 if workspace is None else workspace.numel(), _stream()))
    return out


def sharded_fused(handle, points, queries, k, shard_begin, workspace, mode=L2_PARTIAL, fused_workspace=None, out=None):
    import torch
    _device_check(points, torch.float32, "points")
    _device_check(queries, torch.float32, "queries")
    assert points.is_contiguous() and queries.is_contiguous()
    n, dim = points.shape
    q = queries.shape[0]
    out = _sharded_out(q, k, points.device, out)
    need = fused_workspace_bytes(n, q, dim, k, mode)
    if fused_workspace is None and need > 0:
        fused_workspace = torch.empty(need, dtype=torch.uint8, device=points.device)
    _check(lib().bitsknn_sharded_search_fused(handle, _p(points), _p(queries), n, q, dim, k, mode, shard_begin,
                                              _p(out[0]), _p(out[1]), _p(fused_workspace),
                                              0 if fused_workspace is None else fused_workspace.numel(), _p(workspace),
                                              0 if workspace is None else workspace.numel(), _stream()))
    return out


def sharded_drain(handle):
    _check(lib().bitsknn_sharded_drain(handle, _stream()))
