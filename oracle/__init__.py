"""TEST INFRASTRUCTURE - ctypes access to the CPU checkers.

``oracle.port``  : the plain-C restatement (``oracle/kmeans_oracle.c``), always available
                   (built on first use with gcc).
``oracle.ref()`` : the reference project's own serial k-means compiled from its headers
                   (``oracle/_ref/libkmref.so``), or ``None`` where neither the reference
                   checkout nor a prebuilt library exists.

Only tests, the smoke check and the CPU-baseline legs of the benchmark may import this
package; the product library never does.
"""
import ctypes
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import build_oracle as _b

AOS = 0
SOA = 1

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_u64 = ctypes.c_uint64
_u32 = ctypes.c_uint32
_int = ctypes.c_int


def _load_port():
    lib = ctypes.CDLL(_b.build_oracle())
    lib.okm_assign_range_f32.argtypes = [_f32p, _f32p, _u32p, _u64, _u32, _u32, _int, _int, _u64, _u64]
    lib.okm_assign_range_f32.restype = None
    lib.okm_best2_range_f32.argtypes = [_f32p, _f32p, _f32p, _f32p, _u64, _u32, _u32, _int, _int, _u64, _u64]
    lib.okm_best2_range_f32.restype = None
    lib.okm_dist_to_f32.argtypes = [_f32p, _f32p, _u32p, _f32p, _u64, _u32, _u32, _int, _int, _u64, _u64]
    lib.okm_dist_to_f32.restype = None
    lib.okm_update_f32.argtypes = [_f32p, _u32p, _f32p, _u32p, _u64, _u32, _u32, _int, _int]
    lib.okm_update_f32.restype = None
    lib.okm_update_f64.argtypes = [_f32p, _u32p, _f64p, _u32p, _u64, _u32, _u32, _int, _int]
    lib.okm_update_f64.restype = None
    lib.okm_kmeans_f32.argtypes = [_f32p, _f32p, _f32p, _u32p, _u32p, ctypes.c_void_p, _u64, _u32, _u32, _u32, _int, _int]
    lib.okm_kmeans_f32.restype = None
    lib.okm_assign_range_d.argtypes = [_f64p, _f64p, _u32p, _u64, _u32, _u32, _int, _int, _u64, _u64]
    lib.okm_assign_range_d.restype = None
    lib.okm_update_d.argtypes = [_f64p, _u32p, _f64p, _u32p, _u64, _u32, _u32, _int, _int]
    lib.okm_update_d.restype = None
    lib.okm_kmeans_d.argtypes = [_f64p, _f64p, _f64p, _u32p, _u32p, _u64, _u32, _u32, _u32, _int, _int]
    lib.okm_kmeans_d.restype = None
    return lib


_port_lib = None
_ref_lib = False


def _port():
    global _port_lib
    if _port_lib is None:
        _port_lib = _load_port()
    return _port_lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _u32a(a):
    return np.ascontiguousarray(a, dtype=np.uint32).reshape(-1)


def _threads(threads):
    return max(1, threads or 1)


def _ranges(n, threads):
    t = min(_threads(threads), max(1, n))
    edges = np.linspace(0, n, t + 1).astype(np.uint64)
    return [(int(edges[i]), int(edges[i + 1])) for i in range(t) if edges[i + 1] > edges[i]]


def _parallel(fn, n, threads):
    rs = _ranges(n, threads)
    if len(rs) <= 1:
        for r in rs:
            fn(*r)
        return
    with ThreadPoolExecutor(len(rs)) as ex:
        list(ex.map(lambda r: fn(*r), rs))


def assign(data, means, n, k, d, layout=AOS, layout_means=None, threads=1):
    """Nearest-mean index of every point (serial.hpp:21-42).  ``threads`` > 1 splits the point
    range; the result is identical because points are independent."""
    layout_means = layout if layout_means is None else layout_means
    data, means = _f32(data), _f32(means)
    out = np.empty(n, dtype=np.uint32)
    lib = _port()
    _parallel(lambda b, e: lib.okm_assign_range_f32(data, means, out, n, k, d, layout, layout_means, b, e), n, threads)
    return out


def best2(data, means, n, k, d, layout=AOS, layout_means=None, threads=1):
    """(best, second-best) reference distances of every point."""
    layout_means = layout if layout_means is None else layout_means
    data, means = _f32(data), _f32(means)
    best = np.empty(n, dtype=np.float32)
    second = np.empty(n, dtype=np.float32)
    lib = _port()
    _parallel(lambda b, e: lib.okm_best2_range_f32(data, means, best, second, n, k, d, layout, layout_means, b, e), n, threads)
    return best, second


def dist_to(data, means, which, n, k, d, layout=AOS, layout_means=None, threads=1):
    """Reference distance of every point i to mean ``which[i]``."""
    layout_means = layout if layout_means is None else layout_means
    data, means, which = _f32(data), _f32(means), _u32a(which)
    out = np.empty(n, dtype=np.float32)
    lib = _port()
    _parallel(lambda b, e: lib.okm_dist_to_f32(data, means, which, out, n, k, d, layout, layout_means, b, e), n, threads)
    return out


def update(data, assignment, n, k, d, layout=AOS, layout_means=None):
    """(means, sizes) of the update step (serial.hpp:44-73), float, sequential."""
    layout_means = layout if layout_means is None else layout_means
    data, assignment = _f32(data), _u32a(assignment)
    means = np.empty(k * d, dtype=np.float32)
    sizes = np.empty(k, dtype=np.uint32)
    _port().okm_update_f32(data, assignment, means, sizes, n, k, d, layout, layout_means)
    return means, sizes


def update_f64(data, assignment, n, k, d, layout=AOS, layout_means=None):
    """Same update accumulated in double (arbitration value, not the reference arithmetic)."""
    layout_means = layout if layout_means is None else layout_means
    data, assignment = _f32(data), _u32a(assignment)
    means = np.empty(k * d, dtype=np.float64)
    sizes = np.empty(k, dtype=np.uint32)
    _port().okm_update_f64(data, assignment, means, sizes, n, k, d, layout, layout_means)
    return means, sizes


def kmeans(data, means, n, k, d, iters, layout=AOS, layout_means=None, trace=False):
    """Full fixed-iteration run (serial.hpp:89-96).  Returns (means, assignment[, trace])."""
    layout_means = layout if layout_means is None else layout_means
    data = _f32(data)
    cur = _f32(means).copy()
    prev = np.empty_like(cur)
    asg = np.zeros(n, dtype=np.uint32)
    sizes = np.zeros(k, dtype=np.uint32)
    tr = np.empty((iters, k * d), dtype=np.float32) if trace else None
    _port().okm_kmeans_f32(data, cur, prev, asg, sizes, tr.ctypes.data if trace else None,
                           n, k, d, iters, layout, layout_means)
    return (cur, asg, tr) if trace else (cur, asg)


class _Ref:
    """The reference project's own serial implementation (compiled from its headers)."""

    def __init__(self, path):
        lib = ctypes.CDLL(path)
        lib.ref_kmeans_f32.argtypes = [_int, _int, _u64, _u64, _u64, _u64, _f32p, _f32p, _f32p, _u32p]
        lib.ref_kmeans_f32.restype = _int
        lib.ref_assign_f32.argtypes = [_int, _int, _u64, _u64, _u64, _f32p, _f32p, _u32p]
        lib.ref_assign_f32.restype = _int
        lib.ref_kmeans_f64.argtypes = [_int, _int, _u64, _u64, _u64, _u64, _f64p, _f64p, _f64p, _u32p]
        lib.ref_kmeans_f64.restype = _int
        self._lib = lib
        self.path = path

    def kmeans(self, data, means, n, k, d, iters, layout=AOS, layout_means=None):
        layout_means = layout if layout_means is None else layout_means
        data, means = _f32(data), _f32(means)
        out_means = np.empty(k * d, dtype=np.float32)
        out_asg = np.empty(n, dtype=np.uint32)
        rc = self._lib.ref_kmeans_f32(layout, layout_means, d, k, n, iters, data, means, out_means, out_asg)
        if rc != 0:
            raise RuntimeError("ref_kmeans_f32 failed")
        return out_means, out_asg

    def kmeans_f64(self, data, means, n, k, d, iters, layout=AOS, layout_means=None):
        layout_means = layout if layout_means is None else layout_means
        data, means = _f64(data), _f64(means)
        out_means = np.empty(k * d, dtype=np.float64)
        out_asg = np.empty(n, dtype=np.uint32)
        if self._lib.ref_kmeans_f64(layout, layout_means, d, k, n, iters, data, means, out_means, out_asg) != 0:
            raise RuntimeError("ref_kmeans_f64 failed")
        return out_means, out_asg

    def assign(self, data, means, n, k, d, layout=AOS, layout_means=None):
        layout_means = layout if layout_means is None else layout_means
        data, means = _f32(data), _f32(means)
        out_asg = np.empty(n, dtype=np.uint32)
        rc = self._lib.ref_assign_f32(layout, layout_means, d, k, n, data, means, out_asg)
        if rc != 0:
            raise RuntimeError("ref_assign_f32 failed")
        return out_asg


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64).reshape(-1)


def kmeans_f64(data, means, n, k, d, iters, layout=AOS, layout_means=None):
    """Full fixed-iteration run in double (serial.hpp:89-96 with F = double): (means, assignment)."""
    layout_means = layout if layout_means is None else layout_means
    data = _f64(data)
    cur = _f64(means).copy()
    prev = np.empty_like(cur)
    asg = np.zeros(n, dtype=np.uint32)
    sizes = np.zeros(k, dtype=np.uint32)
    _port().okm_kmeans_d(data, cur, prev, asg, sizes, n, k, d, iters, layout, layout_means)
    return cur, asg


def assign_f64(data, means, n, k, d, layout=AOS, layout_means=None, threads=1):
    """Nearest-mean index of every point in double (serial.hpp:21-42 with F = double)."""
    layout_means = layout if layout_means is None else layout_means
    data, means = _f64(data), _f64(means)
    out = np.empty(n, dtype=np.uint32)
    lib = _port()
    _parallel(lambda b, e: lib.okm_assign_range_d(data, means, out, n, k, d, layout, layout_means, b, e), n, threads)
    return out


def update_d(data, assignment, n, k, d, layout=AOS, layout_means=None):
    """(means, sizes) of the update step in double (serial.hpp:44-73 with F = double)."""
    layout_means = layout if layout_means is None else layout_means
    data, assignment = _f64(data), _u32a(assignment)
    means = np.empty(k * d, dtype=np.float64)
    sizes = np.empty(k, dtype=np.uint32)
    _port().okm_update_d(data, assignment, means, sizes, n, k, d, layout, layout_means)
    return means, sizes


class _RefData:
    """The reference project's own input generators (headers/data.hpp, compiled)."""

    def __init__(self, path):
        lib = ctypes.CDLL(path)
        lib.ref_make_inputs_f32.argtypes = [_int, _int, _u64, _u64, _u64, _u64, _f32p, _f32p]
        lib.ref_make_inputs_f32.restype = _int
        lib.ref_make_bucketing_inputs_f32.argtypes = [_u64, _u64, _u32, _u64, _f32p, _u32p]
        lib.ref_make_bucketing_inputs_f32.restype = _int
        lib.ref_make_inputs_f64.argtypes = [_int, _int, _u64, _u64, _u64, _u64, _f64p, _f64p]
        lib.ref_make_inputs_f64.restype = _int
        self._lib = lib
        self.path = path

    def kmeans_inputs(self, n, k, d, seed, layout=AOS, layout_means=None):
        """(data, initial means) the reference's k-means executable generates for these arguments."""
        layout_means = layout if layout_means is None else layout_means
        data = np.empty(n * d, dtype=np.float32)
        means = np.empty(k * d, dtype=np.float32)
        if self._lib.ref_make_inputs_f32(layout, layout_means, n, k, d, seed, data, means) != 0:
            raise RuntimeError("ref_make_inputs_f32 failed")
        return data, means

    def kmeans_inputs_f64(self, n, k, d, seed, layout=AOS, layout_means=None):
        """The same for the reference executable's --double mode."""
        layout_means = layout if layout_means is None else layout_means
        data = np.empty(n * d, dtype=np.float64)
        means = np.empty(k * d, dtype=np.float64)
        if self._lib.ref_make_inputs_f64(layout, layout_means, n, k, d, seed, data, means) != 0:
            raise RuntimeError("ref_make_inputs_f64 failed")
        return data, means

    def bucketing_inputs(self, count, count_idx, k, seed):
        """(data, indices) the reference's bucketing executable generates: `count` floats, `count_idx` indices."""
        data = np.empty(count, dtype=np.float32)
        idx = np.empty(count_idx, dtype=np.uint32)
        if self._lib.ref_make_bucketing_inputs_f32(count, count_idx, k, seed, data, idx) != 0:
            raise RuntimeError("ref_make_bucketing_inputs_f32 failed")
        return data, idx


_ref_data_lib = False


def ref_data():
    """The compiled reference generators, or None if they are neither buildable nor prebuilt here."""
    global _ref_data_lib
    if _ref_data_lib is False:
        path = _b.build_ref_data()
        _ref_data_lib = _RefData(path) if path else None
    return _ref_data_lib


def ref():
    """The compiled reference, or None if it is neither buildable nor prebuilt here."""
    global _ref_lib
    if _ref_lib is False:
        path = _b.build_ref()
        _ref_lib = _Ref(path) if path else None
    return _ref_lib
