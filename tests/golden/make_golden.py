"""Generates tests/golden/kmeans_golden.npz from the REFERENCE's own serial k-means.

The expected outputs are produced by oracle/_ref/libkmref.so, i.e. by SerialKMeansAlgorithm and
SerialAssignmentAlgorithm of krulis-martin/cuda-kmeans compiled from the reference headers
(experimental/k-means/k-means/headers/serial.hpp) - not by the restatement in
oracle/kmeans_oracle.c, which these vectors exist to pin.  The reference checkout is needed
to run this script (python tests/golden/make_golden.py); the committed .npz travels without it.

Cases cover both layouts for points and means, dimensions on both sides of the CUDA-core /
tensor-core switch, k that is not a multiple of any tile size, exact ties (duplicated means
and duplicated points: the lowest index must win) and a cluster that ends up empty (its mean
must become all zeros; with more iterations that zero mean competes like any other).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402

AOS, SOA = 0, 1


def to_layout(rows, layout):
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    return rows.reshape(-1) if layout == AOS else np.ascontiguousarray(rows.T).reshape(-1)


def cases():
    rng = np.random.default_rng(20240531)
    out = []

    def add(name, rows, means_rows, iters, layout, layout_means):
        out.append(dict(name=name, rows=rows.astype(np.float32), means=means_rows.astype(np.float32),
                        iters=iters, layout=layout, layout_means=layout_means))

    # uniform data, all four layout combinations, small odd sizes
    for (n, k, d) in [(257, 5, 3), (1000, 16, 4), (513, 33, 32), (300, 7, 17), (640, 40, 2)]:
        for layout in (AOS, SOA):
            for layout_means in (AOS, SOA):
                rows = rng.random((n, d), dtype=np.float32)
                add("uniform_n%d_k%d_d%d_L%d%d" % (n, k, d, layout, layout_means), rows, rows[:k], 4, layout, layout_means)
    # clustered data (mixture of gaussians), initial means = first k points
    for (n, k, d, sigma) in [(2048, 16, 4, 0.05), (1500, 24, 16, 0.02), (999, 8, 8, 0.1)]:
        centres = rng.random((k, d), dtype=np.float32)
        rows = centres[rng.integers(0, k, n)] + sigma * rng.standard_normal((n, d), dtype=np.float32)
        add("mixture_n%d_k%d_d%d" % (n, k, d), rows, rows[:k], 5, AOS, AOS)
        add("mixture_soa_n%d_k%d_d%d" % (n, k, d), rows, rows[:k], 5, SOA, SOA)
    # exact ties: means 0 and 3 identical, 1 and 2 identical; points on a coarse integer grid so
    # that many distances are equal bit for bit
    rows = rng.integers(0, 4, (400, 3)).astype(np.float32)
    means = np.array([[1, 1, 1], [2, 2, 2], [2, 2, 2], [1, 1, 1], [0, 3, 0]], dtype=np.float32)
    add("ties_grid", rows, means, 1, AOS, AOS)
    add("ties_grid_soa", rows, means, 1, SOA, SOA)
    # a mean far from every point: its cluster is empty after the first iteration -> zeros
    rows = rng.random((500, 4), dtype=np.float32)
    means = np.vstack([rows[:5], np.full((1, 4), 100.0, dtype=np.float32)])
    add("empty_cluster", rows, means, 1, AOS, AOS)
    add("empty_cluster_soa_means", rows, means, 1, AOS, SOA)
    add("empty_cluster_then_reused", rows, means, 3, AOS, AOS)
    # k = 1 and n = k
    rows = rng.random((64, 5), dtype=np.float32)
    add("single_cluster", rows, rows[:1], 2, AOS, AOS)
    add("n_equals_k", rows[:12], rows[:12], 2, SOA, AOS)
    return out


def main():
    ref = oracle.ref()
    if ref is None:
        raise SystemExit("the reference checkout is needed to generate golden vectors")
    store = {}
    names = []
    for c in cases():
        n, d = c["rows"].shape
        k = c["means"].shape[0]
        data = to_layout(c["rows"], c["layout"])
        means = to_layout(c["means"], c["layout_means"])
        out_means, out_asg = ref.kmeans(data, means, n, k, d, c["iters"], c["layout"], c["layout_means"])
        first_asg = ref.assign(data, means, n, k, d, c["layout"], c["layout_means"])
        p = c["name"]
        names.append(p)
        store[p + "/data"] = data
        store[p + "/means"] = means
        store[p + "/shape"] = np.array([n, k, d, c["iters"], c["layout"], c["layout_means"]], dtype=np.int64)
        store[p + "/out_means"] = out_means
        store[p + "/out_assignment"] = out_asg
        store[p + "/first_assignment"] = first_asg
    store["names"] = np.array(names)
    path = os.path.join(HERE, "kmeans_golden.npz")
    np.savez_compressed(path, **store)
    print("wrote %s: %d cases, %d bytes" % (path, len(names), os.path.getsize(path)))


if __name__ == "__main__":
    main()
