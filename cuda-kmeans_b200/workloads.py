"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark
configurations (they stand in for the reference's own random generator,
experimental/k-means/k-means/headers/data.hpp:33-56 of krulis-martin/cuda-kmeans; no public
dataset is involved).  Initial means are the first k points (prepare_means with shuffle off,
data.hpp:63-81).

Points are produced in row-major (n, dim) order and converted to the requested layout:
AoS = the (n, dim) array flattened, SoA = its transpose flattened.
"""
import numpy as np

AOS, SOA = 0, 1

CONFIGS = {
    # name: (n, dim, k, layout, iterations, generator kind)
    "c1": dict(n=1 << 16, dim=4, k=16, layout=AOS, iters=10, kind="mixture", sigma=0.05, zipf=None),
    "c2": dict(n=1 << 21, dim=32, k=1024, layout=SOA, iters=20, kind="uniform"),
    "c3": dict(n=1 << 24, dim=2, k=64, layout=AOS, iters=20, kind="mixture", sigma=0.01, zipf=1.1),
    "c4": dict(n=1 << 20, dim=512, k=4096, layout=AOS, iters=10, kind="sphere"),
    "c5": dict(n=1 << 28, dim=16, k=256, layout=AOS, iters=10, kind="mixture", sigma=0.02, zipf=None),
}


def to_layout(rows, layout):
    """(items, dim) float32 array -> flat array in the given layout."""
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    return rows.reshape(-1) if layout == AOS else np.ascontiguousarray(rows.T).reshape(-1)


def from_layout(flat, items, dim, layout):
    """Flat array in the given layout -> (items, dim) view/copy."""
    flat = np.asarray(flat)
    return flat.reshape(items, dim) if layout == AOS else flat.reshape(dim, items).T


def mixture_centres(k, dim, seed):
    return np.random.default_rng([seed, 7]).random((k, dim), dtype=np.float32)


def mixture_weights(k, zipf):
    if zipf is None:
        return np.full(k, 1.0 / k)
    w = 1.0 / np.arange(1, k + 1, dtype=np.float64) ** zipf
    return w / w.sum()


def generate_rows(kind, n, dim, k, seed=42, sigma=0.05, zipf=None, begin=0, count=None, chunk=1 << 20):
    """Rows [begin, begin+count) of the workload as an (count, dim) float32 array.

    Generation is chunked with one generator per chunk of `chunk` points, seeded by
    (seed, chunk index), so any range - e.g. one rank's shard - reproduces the same values
    whatever the number of ranks."""
    count = n - begin if count is None else count
    out = np.empty((count, dim), dtype=np.float32)
    centres = mixture_centres(k, dim, seed) if kind == "mixture" else None
    weights = mixture_weights(k, zipf) if kind == "mixture" else None
    first_chunk = begin // chunk
    last_chunk = (begin + count - 1) // chunk if count > 0 else first_chunk - 1
    for c in range(first_chunk, last_chunk + 1):
        c0 = c * chunk
        c1 = min(n, c0 + chunk)
        rng = np.random.default_rng([seed, 1000 + c])
        if kind == "uniform":
            block = rng.random((c1 - c0, dim), dtype=np.float32)
        elif kind == "mixture":
            which = rng.choice(k, size=c1 - c0, p=weights)
            block = centres[which] + sigma * rng.standard_normal((c1 - c0, dim), dtype=np.float32)
        elif kind == "sphere":
            block = rng.standard_normal((c1 - c0, dim), dtype=np.float32)
            block /= np.linalg.norm(block, axis=1, keepdims=True).astype(np.float32)
        else:
            raise ValueError("unknown workload kind %r" % kind)
        lo, hi = max(begin, c0), min(begin + count, c1)
        out[lo - begin:hi - begin] = block[lo - c0:hi - c0]
    return out


def make(name, n=None, seed=42, layout=None, layout_means=None):
    """(points_flat, means_flat, spec) for a named configuration, optionally with fewer points."""
    spec = dict(CONFIGS[name])
    if n is not None:
        spec["n"] = n
    if layout is not None:
        spec["layout"] = layout
    spec["layout_means"] = spec["layout"] if layout_means is None else layout_means
    rows = generate_rows(spec["kind"], spec["n"], spec["dim"], spec["k"], seed,
                         spec.get("sigma", 0.05), spec.get("zipf"))
    means = rows[:spec["k"]].copy()
    return to_layout(rows, spec["layout"]), to_layout(means, spec["layout_means"]), spec
