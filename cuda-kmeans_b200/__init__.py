"""Python access to libbkm.so - the B200 k-means iteration library (C ABI in include/bkm.h).

This module is a thin ctypes binding plus `KMeans`, a class with the call sequence of the
reference's IKMeansAlgorithm (experimental/k-means/k-means/headers/interface.hpp:8-49 of
krulis-martin/cuda-kmeans): initialize / run / getMeans / getAssignment / cleanup.  All
computation happens in the CUDA library; there is no Python or CPU fallback, and importing
works without a GPU only so that the binding itself can be checked.

The directory name contains a hyphen, so load it with importlib (see `load()` in
__graft_entry__.py) or put the directory itself on sys.path under another name.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbkm.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NCCL, ERR_UNSUPPORTED, ERR_STATE, ERR_DEVICE = range(7)
LAYOUT_AOS, LAYOUT_SOA = 0, 1
ASSIGN_AUTO, ASSIGN_EXACT, ASSIGN_SIMT, ASSIGN_TC = 0, 1, 2, 3
UPDATE_AUTO, UPDATE_SHARED, UPDATE_GLOBAL, UPDATE_ROWS = 0, 1, 2, 3
ASSIGN_NAMES = {ASSIGN_AUTO: "auto", ASSIGN_EXACT: "exact", ASSIGN_SIMT: "simt", ASSIGN_TC: "tc"}
PLAN_NAMES = {0: "exact", 1: "simt", 2: "tc_resident", 3: "tc_kloop", 4: "tc_pair"}
UPDATE_FUSED = 4   # reported by counters() only
UPDATE_SORTED = 5
UPDATE_NAMES = {UPDATE_AUTO: "auto", UPDATE_SHARED: "shared", UPDATE_GLOBAL: "global", UPDATE_ROWS: "rows",
                UPDATE_FUSED: "fused", UPDATE_SORTED: "sorted"}

# Every symbol include/bkm.h declares (the CPU test suite checks the library exports them all).
SYMBOLS = [
    "bkm_last_error", "bkm_version", "bkm_device_count", "bkm_workspace_bytes", "bkm_assign_f32",
    "bkm_update_f32", "bkm_iterate_f32", "bkm_workspace_check", "bkm_create", "bkm_destroy",
    "bkm_set_stream", "bkm_set_option", "bkm_initialize", "bkm_initialize_device", "bkm_run",
    "bkm_run_async", "bkm_synchronize", "bkm_get_means", "bkm_get_assignment", "bkm_get_sizes",
    "bkm_device_means", "bkm_device_assignment", "bkm_set_means", "bkm_iterations_done",
    "bkm_phase_ms", "bkm_counters", "bkm_comm_unique_id", "bkm_comm_init", "bkm_shard_range",
    "bkm_kmeans_host_f32", "bkm_update_noalloc_f32", "bkm_selftest_wait_timeout", "bkm_assign_plan",
    "bkm_noalloc_check", "bkm_peer_export", "bkm_peer_open", "bkm_peer_buffer", "bkm_peer_attach", "bkm_peer_enable",
    "bkm_peer_layout", "bkm_run_ready", "bkm_bucket_sums_f32", "bkm_probe_atomics_f32",
    "bkm_kmeans_host_f64",
]


class BkmError(RuntimeError):
    """A libbkm call returned a non-zero status; `.code` holds it."""

    def __init__(self, code, message):
        super().__init__("libbkm error %d: %s" % (code, message))
        self.code = code


class Config(ctypes.Structure):
    _fields_ = [
        ("n", ctypes.c_uint64), ("k", ctypes.c_uint32), ("dim", ctypes.c_uint32),
        ("layout", ctypes.c_int32), ("layout_means", ctypes.c_int32), ("device", ctypes.c_int32),
        ("variant_assign", ctypes.c_int32), ("variant_update", ctypes.c_int32), ("num_gpus", ctypes.c_int32),
    ]


_lib = None


def lib():
    """The loaded C library.  Fails loudly when it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing - build it with `python cuda-kmeans_b200/build.py` "
                          "(or __graft_entry__.build()); there is no fallback path" % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    vp, u64, u32, ci, sz = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int, ctypes.c_size_t
    L.bkm_last_error.restype = ctypes.c_char_p
    L.bkm_last_error.argtypes = []
    L.bkm_version.restype = ci
    L.bkm_device_count.restype = ci
    L.bkm_workspace_bytes.restype = sz
    L.bkm_workspace_bytes.argtypes = [u64, u32, u32]
    L.bkm_assign_f32.argtypes = [vp, vp, vp, u64, u32, u32, ci, ci, ci, vp, sz, vp]
    L.bkm_update_f32.argtypes = [vp, vp, vp, vp, u64, u32, u32, ci, ci, ci, vp, sz, vp]
    L.bkm_iterate_f32.argtypes = [vp, vp, vp, vp, vp, u64, u32, u32, ci, ci, ci, ci, vp, sz, vp]
    L.bkm_workspace_check.argtypes = [vp, vp]
    L.bkm_create.argtypes = [ctypes.POINTER(Config), ctypes.POINTER(vp)]
    L.bkm_destroy.argtypes = [vp]
    L.bkm_set_stream.argtypes = [vp, vp]
    L.bkm_set_option.argtypes = [vp, ctypes.c_char_p, ctypes.c_double]
    L.bkm_initialize.argtypes = [vp, vp, vp]
    L.bkm_initialize_device.argtypes = [vp, vp, vp]
    L.bkm_run.argtypes = [vp, u32]
    L.bkm_run_async.argtypes = [vp, u32]
    L.bkm_synchronize.argtypes = [vp]
    L.bkm_get_means.argtypes = [vp, vp]
    L.bkm_get_assignment.argtypes = [vp, vp]
    L.bkm_get_sizes.argtypes = [vp, vp]
    L.bkm_device_means.argtypes = [vp, ctypes.POINTER(vp)]
    L.bkm_device_assignment.argtypes = [vp, ctypes.POINTER(vp)]
    L.bkm_set_means.argtypes = [vp, vp]
    L.bkm_iterations_done.argtypes = [vp, ctypes.POINTER(u64)]
    L.bkm_phase_ms.argtypes = [vp, ctypes.POINTER(ctypes.c_float)]
    L.bkm_counters.argtypes = [vp, ctypes.POINTER(u64)]
    L.bkm_comm_unique_id.argtypes = [vp, sz]
    L.bkm_comm_init.argtypes = [vp, vp, sz, ci, ci]
    L.bkm_shard_range.argtypes = [u64, ci, ci, ctypes.POINTER(u64), ctypes.POINTER(u64)]
    L.bkm_kmeans_host_f32.argtypes = [vp, vp, vp, u64, u32, u32, u32, ci, ci, ci]
    L.bkm_update_noalloc_f32.argtypes = [vp, vp, vp, vp, u64, u32, u32, ci, ci, vp]
    L.bkm_selftest_wait_timeout.argtypes = [vp, u32, vp]
    L.bkm_assign_plan.argtypes = [vp, ctypes.POINTER(u32)]
    L.bkm_noalloc_check.argtypes = [vp]
    L.bkm_peer_export.argtypes = [vp, vp, sz]
    L.bkm_peer_open.argtypes = [vp, vp, sz, ci, ci]
    L.bkm_peer_buffer.argtypes = [vp, ctypes.POINTER(vp), ctypes.POINTER(sz)]
    L.bkm_peer_attach.argtypes = [vp, ctypes.POINTER(vp), ci, ci]
    L.bkm_peer_enable.argtypes = [vp, ci]
    L.bkm_peer_layout.argtypes = [u32, u32, ctypes.POINTER(u64)]
    L.bkm_run_ready.argtypes = [vp]
    L.bkm_bucket_sums_f32.argtypes = [vp, vp, vp, u64, u32, u32, ci, ci, vp, sz, vp]
    L.bkm_probe_atomics_f32.argtypes = [vp, u64, u32, u32, ci, ci, u32, vp]
    L.bkm_kmeans_host_f64.argtypes = [vp, vp, vp, u64, u32, u32, u32, ci, ci, ci]
    for name in SYMBOLS:
        fn = getattr(L, name)
        if name not in ("bkm_last_error", "bkm_workspace_bytes"):
            fn.restype = ci
    _lib = L
    return L


def check(rc):
    if rc != OK:
        raise BkmError(rc, lib().bkm_last_error().decode("utf-8", "replace"))


def device_count():
    return lib().bkm_device_count()


def workspace_bytes(n, k, dim):
    return lib().bkm_workspace_bytes(n, k, dim)


def shard_range(n_total, world_size, rank):
    """(begin, count) of the contiguous shard of `rank` (pure host arithmetic)."""
    b, c = ctypes.c_uint64(), ctypes.c_uint64()
    check(lib().bkm_shard_range(n_total, world_size, rank, ctypes.byref(b), ctypes.byref(c)))
    return b.value, c.value


def _preload_nccl():
    """Loads the NCCL that ships as a Python wheel (the one PyTorch links) before libbkm looks for
    one, so that a process that imports torch later does not end up with the system copy bound
    under the same soname.  No effect when that wheel is absent or NCCL is already loaded."""
    import importlib.util
    try:
        spec = importlib.util.find_spec("nvidia")
    except (ImportError, ValueError):
        spec = None
    for base in (list(spec.submodule_search_locations) if spec and spec.submodule_search_locations else []):
        path = os.path.join(base, "nccl", "lib", "libnccl.so.2")
        if os.path.exists(path):
            try:
                ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
            except OSError:
                pass
            return


def agree(dist, torch, code, device="cpu"):
    """Host-side agreement of all ranks of a torch.distributed process group on one status code:
    every rank passes its own (OK or an error code) and receives the largest.  Used before a
    step in which one failing rank would leave the others waiting for it: when the result is not
    OK, no rank may enter that step."""
    t = torch.tensor([int(code)], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(t.item())


PEER_BLOB_BYTES = 128


def peer_layout(k, dim):
    """dict with the layout of an exchange buffer (bkm_peer_layout)."""
    arr = (ctypes.c_uint64 * 4)()
    check(lib().bkm_peer_layout(k, dim, arr))
    return {"bytes": int(arr[0]), "packets_per_sender": int(arr[1]), "senders": int(arr[2]), "slot_bytes": int(arr[3])}


def comm_unique_id():
    """128 bytes identifying a new NCCL communicator (rank 0 creates, all ranks receive)."""
    _preload_nccl()
    buf = ctypes.create_string_buffer(128)
    check(lib().bkm_comm_unique_id(buf, 128))
    return buf.raw


# ---- kernel-runner entry points on raw device pointers (ints) -------------------------------

def assign(points, means, assignment, n, k, dim, layout, layout_means, workspace, workspace_size,
           variant=ASSIGN_AUTO, stream=0):
    check(lib().bkm_assign_f32(points, means, assignment, n, k, dim, layout, layout_means, variant,
                               workspace, workspace_size, stream))


def update(points, assignment, means, sizes, n, k, dim, layout, layout_means, workspace, workspace_size,
           variant=UPDATE_AUTO, stream=0):
    check(lib().bkm_update_f32(points, assignment, means, sizes, n, k, dim, layout, layout_means, variant,
                               workspace, workspace_size, stream))


def bucket_sums(points, indices, sums, n, k, dim, layout, workspace, workspace_size, variant=UPDATE_AUTO, stream=0):
    """bkm_bucket_sums_f32: per-bucket sums (no sizes, no divide), result in the points' layout."""
    check(lib().bkm_bucket_sums_f32(points, indices, sums, n, k, dim, layout, variant, workspace, workspace_size, stream))


def probe_atomics(result, n, k, dim, layout, shared_cache=False, items_per_thread=1, stream=0):
    """bkm_probe_atomics_f32: the write-only atomic-add probe."""
    check(lib().bkm_probe_atomics_f32(result, n, k, dim, layout, 1 if shared_cache else 0, items_per_thread, stream))


def update_noalloc(points, assignment, means, sizes, n, k, dim, layout, layout_means, stream=0):
    """bkm_update_noalloc_f32: the update step on the library's built-in scratch (no workspace, no
    allocation); k*dim + k is limited to NOALLOC_MAX_WORDS and calls on one device must not overlap."""
    check(lib().bkm_update_noalloc_f32(points, assignment, means, sizes, n, k, dim, layout, layout_means, stream))


def noalloc_check(stream=0):
    """bkm_noalloc_check: raises BkmError(ERR_DEVICE) if the last update_noalloc call on the current
    device saw an assignment value >= k."""
    check(lib().bkm_noalloc_check(stream))


NOALLOC_MAX_WORDS = 512 * 1024 - 128


def iterate(points, means_in, means_out, sizes, assignment, n, k, dim, layout, layout_means,
            workspace, workspace_size, variant_assign=ASSIGN_AUTO, variant_update=UPDATE_AUTO, stream=0):
    check(lib().bkm_iterate_f32(points, means_in, means_out, sizes, assignment, n, k, dim, layout,
                                layout_means, variant_assign, variant_update, workspace, workspace_size, stream))


def workspace_check(workspace, stream=0):
    check(lib().bkm_workspace_check(workspace, stream))


def selftest_wait_timeout(workspace, limit_ms=50, stream=0):
    """Enqueues the bounded-wait self-test (bkm_selftest_wait_timeout): a wait that runs out after
    limit_ms and records the time-out status in the workspace's control block."""
    check(lib().bkm_selftest_wait_timeout(workspace, int(limit_ms), stream))


def kmeans_host(points, means, n, k, dim, iters, layout=LAYOUT_AOS, layout_means=None, device=0):
    """Whole job on HOST arrays (bkm_kmeans_host_f32): returns (final means, assignment)."""
    layout_means = layout if layout_means is None else layout_means
    pts = np.ascontiguousarray(points, dtype=np.float32).reshape(-1)
    out_means = np.ascontiguousarray(means, dtype=np.float32).reshape(-1).copy()
    if pts.size != n * dim or out_means.size != k * dim:
        raise ValueError("array sizes do not match n, k, dim")
    asg = np.empty(n, dtype=np.uint32)
    check(lib().bkm_kmeans_host_f32(pts.ctypes.data, out_means.ctypes.data, asg.ctypes.data,
                                    n, k, dim, iters, layout, layout_means, device))
    return out_means, asg


def kmeans_host_f64(points, means, n, k, dim, iters, layout=LAYOUT_AOS, layout_means=None, device=0):
    """Whole job in fp64 on HOST arrays (bkm_kmeans_host_f64): returns (final means, assignment)."""
    layout_means = layout if layout_means is None else layout_means
    pts = np.ascontiguousarray(points, dtype=np.float64).reshape(-1)
    out_means = np.ascontiguousarray(means, dtype=np.float64).reshape(-1).copy()
    if pts.size != n * dim or out_means.size != k * dim:
        raise ValueError("array sizes do not match n, k, dim")
    asg = np.empty(n, dtype=np.uint32)
    check(lib().bkm_kmeans_host_f64(pts.ctypes.data, out_means.ctypes.data, asg.ctypes.data,
                                    n, k, dim, iters, layout, layout_means, device))
    return out_means, asg


class KMeans:
    """Fixed-iteration k-means on one GPU (or one rank's shard), over the driver handle.

    Mirrors IKMeansAlgorithm / CudaKMeansAlgorithm of the reference
    (headers/interface.hpp:8-49, headers/cuda.hpp:19-112): `initialize` uploads data and
    initial means, `run` performs the configured number of iterations, `getMeans` /
    `getAssignment` fetch the results, `cleanup` releases the device state.
    """

    def __init__(self, layout=LAYOUT_AOS, layout_means=None, device=0, variant_assign=ASSIGN_AUTO,
                 variant_update=UPDATE_AUTO, num_gpus=1):
        self.layout = layout
        self.layout_means = layout if layout_means is None else layout_means
        self.device = device
        self.variant_assign = variant_assign
        self.variant_update = variant_update
        self.num_gpus = num_gpus      # > 1: this one process drives GPUs device .. device+num_gpus-1
        self._h = None
        self.dim = self.k = self.n = 0
        self.iters = 1
        self._options = {}
        self._stream = None

    # -- reference-style interface --
    def initialize(self, dim, k, n, iters, data, means):
        """`data`/`means`: host numpy arrays in the configured layouts (n*dim and k*dim floats)."""
        self._create(dim, k, n, iters)
        pts = np.ascontiguousarray(data, dtype=np.float32).reshape(-1)
        mns = np.ascontiguousarray(means, dtype=np.float32).reshape(-1)
        if pts.size != n * dim or mns.size != k * dim:
            raise ValueError("array sizes do not match n, k, dim")
        check(lib().bkm_initialize(self._h, pts.ctypes.data, mns.ctypes.data))

    def initialize_device(self, dim, k, n, iters, data_ptr, means_ptr):
        """Same with device pointers (ints); the points are borrowed and must stay alive."""
        self._create(dim, k, n, iters)
        check(lib().bkm_initialize_device(self._h, data_ptr, means_ptr))

    def run(self, iters=None):
        check(lib().bkm_run(self._need(), self.iters if iters is None else iters))

    def run_async(self, iters=None):
        check(lib().bkm_run_async(self._need(), self.iters if iters is None else iters))

    def synchronize(self):
        check(lib().bkm_synchronize(self._need()))

    def getMeans(self):
        out = np.empty(self.k * self.dim, dtype=np.float32)
        check(lib().bkm_get_means(self._need(), out.ctypes.data))
        return out

    def getAssignment(self):
        out = np.empty(self.n, dtype=np.uint32)
        check(lib().bkm_get_assignment(self._need(), out.ctypes.data))
        return out

    def getSizes(self):
        out = np.empty(self.k, dtype=np.uint32)
        check(lib().bkm_get_sizes(self._need(), out.ctypes.data))
        return out

    def getIterations(self):
        return self.iters

    def cleanup(self):
        if self._h is not None:
            lib().bkm_destroy(self._h)
            self._h = None

    # -- extras --
    def set_means(self, means):
        mns = np.ascontiguousarray(means, dtype=np.float32).reshape(-1)
        if mns.size != self.k * self.dim:
            raise ValueError("means size does not match k*dim")
        check(lib().bkm_set_means(self._need(), mns.ctypes.data))

    def set_option(self, name, value):
        self._options[name] = float(value)
        if self._h is not None:
            check(lib().bkm_set_option(self._h, name.encode(), float(value)))

    def set_stream(self, stream_ptr):
        self._stream = stream_ptr
        if self._h is not None:
            check(lib().bkm_set_stream(self._h, stream_ptr))

    def comm_init(self, unique_id, world_size, rank):
        _preload_nccl()
        buf = ctypes.create_string_buffer(bytes(unique_id), 128)
        check(lib().bkm_comm_init(self._need(), buf, 128, world_size, rank))

    # -- exchange through peer memory (see bkm.h) --
    def peer_export(self):
        buf = ctypes.create_string_buffer(PEER_BLOB_BYTES)
        check(lib().bkm_peer_export(self._need(), buf, PEER_BLOB_BYTES))
        return buf.raw

    def peer_open(self, blobs, world_size, rank):
        data = bytes(blobs)
        if len(data) != PEER_BLOB_BYTES * world_size:
            raise ValueError("expected %d blobs of %d bytes" % (world_size, PEER_BLOB_BYTES))
        check(lib().bkm_peer_open(self._need(), ctypes.create_string_buffer(data, len(data)), PEER_BLOB_BYTES, world_size, rank))

    def peer_buffer(self):
        p, n = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().bkm_peer_buffer(self._need(), ctypes.byref(p), ctypes.byref(n)))
        return p.value, n.value

    def peer_attach(self, bases, rank):
        arr = (ctypes.c_void_p * len(bases))(*[ctypes.c_void_p(b) for b in bases])
        check(lib().bkm_peer_attach(self._need(), arr, len(bases), rank))

    def peer_enable(self, on=True):
        check(lib().bkm_peer_enable(self._need(), 1 if on else 0))

    def run_ready(self):
        """Status code of bkm_run_ready (OK = an iteration could start now); never raises."""
        return lib().bkm_run_ready(self._h) if self._h is not None else ERR_STATE

    def peer_exchange_init(self, dist, torch, device="cuda"):
        """Sets the peer-memory exchange up over a torch.distributed process group: gathers every
        rank's blob, opens the peers' buffers, and switches the exchange on only if EVERY rank
        succeeded (the ranks agree through the process group); returns whether it is on."""
        world, rank = dist.get_world_size(), dist.get_rank()
        ok = 1
        try:
            mine = torch.frombuffer(bytearray(self.peer_export()), dtype=torch.uint8).to(device)
        except BkmError:
            ok = 0
            mine = torch.zeros(PEER_BLOB_BYTES, dtype=torch.uint8, device=device)
        blobs = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(blobs, mine)
        if ok:
            try:
                self.peer_open(b"".join(bytes(b.cpu().numpy().tobytes()) for b in blobs), world, rank)
            except BkmError:
                ok = 0
        if agree(dist, torch, 0 if ok else ERR_CUDA, device) != OK:
            return False
        self.peer_enable(True)
        return True

    def device_means(self):
        p = ctypes.c_void_p()
        check(lib().bkm_device_means(self._need(), ctypes.byref(p)))
        return p.value

    def device_assignment(self):
        p = ctypes.c_void_p()
        check(lib().bkm_device_assignment(self._need(), ctypes.byref(p)))
        return p.value

    def iterations_done(self):
        v = ctypes.c_uint64()
        check(lib().bkm_iterations_done(self._need(), ctypes.byref(v)))
        return v.value

    def phase_ms(self):
        """dict of mean device milliseconds per phase over the most recent run."""
        arr = (ctypes.c_float * 6)()
        check(lib().bkm_phase_ms(self._need(), arr))
        names = ["assign", "recheck", "update", "allreduce", "finalize", "iteration"]
        return dict(zip(names, [float(x) for x in arr]))

    def counters(self):
        arr = (ctypes.c_uint64 * 4)()
        check(lib().bkm_counters(self._need(), arr))
        return {"rechecked": int(arr[0]), "launches_per_iter": int(arr[1]),
                "assign_variant": ASSIGN_NAMES.get(int(arr[2]), "?"),
                "update_variant": UPDATE_NAMES.get(int(arr[3]), "?")}

    def assign_plan(self):
        """dict describing the assignment kernel the handle launches (bkm_assign_plan)."""
        arr = (ctypes.c_uint32 * 4)()
        check(lib().bkm_assign_plan(self._need(), arr))
        return {"kernel": PLAN_NAMES.get(int(arr[0]), "?"), "mean_tiles": int(arr[1]), "block_split": int(arr[2]),
                "fused_update": bool(arr[3])}

    def _create(self, dim, k, n, iters):
        self.cleanup()
        self.dim, self.k, self.n, self.iters = int(dim), int(k), int(n), int(iters)
        cfg = Config(n=self.n, k=self.k, dim=self.dim, layout=self.layout, layout_means=self.layout_means,
                     device=self.device, variant_assign=self.variant_assign,
                     variant_update=self.variant_update, num_gpus=self.num_gpus)
        h = ctypes.c_void_p()
        check(lib().bkm_create(ctypes.byref(cfg), ctypes.byref(h)))
        self._h = h
        if self._stream is not None:
            check(lib().bkm_set_stream(self._h, self._stream))
        for name, value in self._options.items():
            check(lib().bkm_set_option(self._h, name.encode(), value))

    def _need(self):
        if self._h is None:
            raise BkmError(ERR_STATE, "initialize() has not been called")
        return self._h

    def __del__(self):
        try:
            self.cleanup()
        except Exception:
            pass
