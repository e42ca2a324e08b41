"""ctypes binding of oracle/_ref/libref_knn.so: the REFERENCE's own algorithms (CPU selection
`serial` / `parallel`, its `bits` kernel, `fused-cache`, GEMM-form distance) compiled from its
sources by `make -C oracle ref`.  TEST INFRASTRUCTURE: used as a second checker beside the
restatement in oracle.cpp and as the timed reference arm of the benchmark.  The reference's
objects create CUDA events when constructed, so every call needs a GPU."""
import ctypes
import pathlib

import numpy as np

_SO = pathlib.Path(__file__).resolve().parent / "_ref" / "libref_knn.so"
_LIB = None
_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int32)
_sz = ctypes.c_size_t


def available():
    """True when the library was built (the reference checkout was present at build time)."""
    return _SO.exists()


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(str(_SO))
        L.ref_last_error.restype = ctypes.c_char_p
        L.ref_select.restype = ctypes.c_int
        L.ref_select.argtypes = [ctypes.c_char_p, _f32p, _sz, _sz, _sz, _sz, _sz, ctypes.c_int, _f32p, _i32p,
                                 ctypes.POINTER(ctypes.c_double)]
        L.ref_fused_cache.restype = ctypes.c_int
        L.ref_fused_cache.argtypes = [_f32p, _f32p, _sz, _sz, _sz, _sz, _sz, _sz, ctypes.c_int, _f32p, _i32p,
                                      ctypes.POINTER(ctypes.c_double)]
        L.ref_l2.restype = ctypes.c_int
        L.ref_l2.argtypes = [_f32p, _f32p, _sz, _sz, _sz, ctypes.c_int, ctypes.c_int, _f32p,
                             ctypes.POINTER(ctypes.c_double)]
        _LIB = L
    return _LIB


def _f(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


def _check(rc):
    if rc != 0:
        raise RuntimeError("reference: " + lib().ref_last_error().decode())


def select(alg, dist, k, block_size=256, batch=13, repeats=0):
    """Reference selection `alg` in {'serial','parallel','bits','bits-prefetch'} on a host matrix.
    Returns (distances, indices, seconds of the fastest selection() call)."""
    q, n = dist.shape
    out_d = np.empty((q, k), dtype=np.float32)
    out_i = np.empty((q, k), dtype=np.int32)
    sec = ctypes.c_double(0.0)
    _check(lib().ref_select(alg.encode(), _f(dist), q, n, k, block_size, batch, repeats, _f(out_d),
                            out_i.ctypes.data_as(_i32p), ctypes.byref(sec)))
    return out_d, out_i, sec.value


def select_parallel(dist, k):
    return select("parallel", dist, k)[:2]


def fused_cache(points, queries, k, block_query_dim=1, dim_mult=1, repeats=0):
    n, dim = points.shape
    q = queries.shape[0]
    out_d = np.empty((q, k), dtype=np.float32)
    out_i = np.empty((q, k), dtype=np.int32)
    sec = ctypes.c_double(0.0)
    _check(lib().ref_fused_cache(_f(points), _f(queries), n, q, dim, k, block_query_dim, dim_mult, repeats,
                                 _f(out_d), out_i.ctypes.data_as(_i32p), ctypes.byref(sec)))
    return out_d, out_i, sec.value


def l2(points, queries, partial=False, repeats=0):
    n, dim = points.shape
    q = queries.shape[0]
    out = np.empty((q, n), dtype=np.float32)
    sec = ctypes.c_double(0.0)
    _check(lib().ref_l2(_f(points), _f(queries), n, q, dim, 1 if partial else 0, repeats, _f(out),
                        ctypes.byref(sec)))
    return out, sec.value
