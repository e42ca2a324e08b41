"""ctypes binding of the CPU oracle (oracle.cpp -> liboracle.so).  TEST INFRASTRUCTURE.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module;
the product library never does.  Arrays are numpy, row-major, float32 / int32.
"""
import ctypes
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int32)
_sz = ctypes.c_size_t


def build(force=False):
    """Compile liboracle.so with the Makefile beside this file (g++, OpenMP)."""
    so = _HERE / "liboracle.so"
    src = _HERE / "oracle.cpp"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = _HERE / "liboracle.so"
        if not so.exists():
            build()
        L = ctypes.CDLL(str(so))
        L.oracle_num_threads.restype = ctypes.c_int
        L.oracle_generate_uniform.restype = ctypes.c_int
        L.oracle_generate_uniform.argtypes = [ctypes.c_uint64, ctypes.c_float, ctypes.c_float,
                                              _sz, _sz, _sz, _f32p, _f32p]
        L.oracle_generate_normal.restype = ctypes.c_int
        L.oracle_generate_normal.argtypes = [ctypes.c_uint64, ctypes.c_float, ctypes.c_float,
                                             _sz, _sz, _sz, _f32p, _f32p]
        L.oracle_preprocess_ordering.restype = None
        L.oracle_preprocess_ordering.argtypes = [_f32p, _sz, _f32p, _sz, ctypes.c_int]
        for name in ("oracle_l2", "oracle_l2_partial"):
            fn = getattr(L, name)
            fn.restype = None
            fn.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _f32p, _sz]
        L.oracle_select.restype = None
        L.oracle_select.argtypes = [_f32p, _sz, _i32p, _sz, _i32p, _sz, _sz, _sz, _f32p, _i32p]
        L.oracle_select_heap.restype = None
        L.oracle_select_heap.argtypes = [_f32p, _sz, _sz, _sz, _sz, _f32p, _i32p]
        L.oracle_knn.restype = None
        L.oracle_knn.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _sz, ctypes.c_int, ctypes.c_int32,
                                 _f32p, _i32p]
        L.oracle_knn_heap.restype = None
        L.oracle_knn_heap.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _sz, ctypes.c_int, _f32p, _i32p]
        L.oracle_merge.restype = None
        L.oracle_merge.argtypes = [_f32p, _i32p, _sz, _sz, _sz, _sz, _sz, _f32p, _i32p]
        L.oracle_checksum.restype = ctypes.c_uint32
        L.oracle_checksum.argtypes = [_i32p, _sz]
        L.oracle_verify.restype = _sz
        L.oracle_verify.argtypes = [_f32p, _i32p, _f32p, _i32p, _sz, _sz]
        _LIB = L
    return _LIB


def _f(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


def _i(a):
    if a is None:
        return None
    assert a.dtype == np.int32 and a.flags.c_contiguous
    return a.ctypes.data_as(_i32p)


def num_threads():
    return int(lib().oracle_num_threads())


def generate(generator, seed, n, q, dim, a=None, b=None):
    """Points (n x dim) then queries (q x dim) from one engine, like the reference CLI."""
    points = np.empty((n, dim), dtype=np.float32)
    queries = np.empty((q, dim), dtype=np.float32)
    if generator == "uniform":
        lo, hi = (0.0, 1.0) if a is None else ((0.0, a) if b is None else (a, b))
        rc = lib().oracle_generate_uniform(seed, lo, hi, n, q, dim, _f(points), _f(queries))
    elif generator == "normal":
        mean, std = (0.0 if a is None else a), (1.0 if b is None else b)
        rc = lib().oracle_generate_normal(seed, mean, std, n, q, dim, _f(points), _f(queries))
    else:
        raise ValueError(generator)
    if rc != 0:
        raise ValueError("invalid generator arguments (seed must be non-zero)")
    return points, queries


def preprocess(points, queries, order):
    """'ascending' / 'descending' preprocessors (in place); 'identity' does nothing."""
    if order != "identity":
        lib().oracle_preprocess_ordering(_f(points), points.size, _f(queries), queries.size,
                                         1 if order == "descending" else 0)


def l2(points, queries, partial=False):
    n, dim = points.shape
    q = queries.shape[0]
    out = np.empty((q, n), dtype=np.float32)
    fn = lib().oracle_l2_partial if partial else lib().oracle_l2
    fn(_f(points), _f(queries), n, q, dim, _f(out), n)
    return out


def select(dist, k, labels=None, label_offsets=None, n=None):
    """k smallest (distance, index) pairs per row, ties to the lowest index."""
    q, ld = dist.shape
    n = ld if n is None else n
    out_d = np.empty((q, k), dtype=np.float32)
    out_i = np.empty((q, k), dtype=np.int32)
    ldl = labels.shape[1] if labels is not None else 0
    lib().oracle_select(_f(dist), ld, _i(labels), ldl, _i(label_offsets), q, n, k,
                        _f(out_d), _i(out_i))
    return out_d, out_i


def select_heap(dist, k):
    q, n = dist.shape
    out_d = np.empty((q, k), dtype=np.float32)
    out_i = np.empty((q, k), dtype=np.int32)
    lib().oracle_select_heap(_f(dist), n, q, n, k, _f(out_d), _i(out_i))
    return out_d, out_i


def knn(points, queries, k, partial=True, index_base=0):
    n, dim = points.shape
    q = queries.shape[0]
    out_d = np.empty((q, k), dtype=np.float32)
    out_i = np.empty((q, k), dtype=np.int32)
    lib().oracle_knn(_f(points), _f(queries), n, q, dim, k, 1 if partial else 0, index_base,
                     _f(out_d), _i(out_i))
    return out_d, out_i


def knn_heap(points, queries, k, partial=True):
    """The CPU k-NN flow (distance chains + max-heap per query, OpenMP over the queries)."""
    n, dim = points.shape
    q = queries.shape[0]
    out_d = np.empty((q, k), dtype=np.float32)
    out_i = np.empty((q, k), dtype=np.int32)
    lib().oracle_knn_heap(_f(points), _f(queries), n, q, dim, k, 1 if partial else 0, _f(out_d), _i(out_i))
    return out_d, out_i


def merge(cand_dist, cand_idx):
    """cand_* of shape (lists, q, k) -> the k smallest pairs per query."""
    lists, q, k = cand_dist.shape
    out_d = np.empty((q, k), dtype=np.float32)
    out_i = np.empty((q, k), dtype=np.int32)
    lib().oracle_merge(_f(cand_dist), _i(cand_idx), q * k, k, q, lists, k, _f(out_d), _i(out_i))
    return out_d, out_i


def checksum(indices_query0):
    a = np.ascontiguousarray(indices_query0, dtype=np.int32)
    return int(lib().oracle_checksum(_i(a), a.size))


def verify(dist_a, idx_a, dist_b, idx_b):
    """Number of slots the reference's tolerant comparison would report (0 = agree)."""
    q, k = dist_a.shape
    return int(lib().oracle_verify(_f(np.ascontiguousarray(dist_a)), _i(np.ascontiguousarray(idx_a)),
                                   _f(np.ascontiguousarray(dist_b)), _i(np.ascontiguousarray(idx_b)),
                                   q, k))
