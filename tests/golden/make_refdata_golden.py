"""Generates tests/golden/refdata_golden.npz from the REFERENCE's own input generators.

The vectors come from oracle/_ref/libkmrefdata.so, i.e. from generate_clustered_data, prepare_means
and generate_random of krulis-martin/cuda-kmeans (experimental/k-means/k-means/headers/data.hpp:19-81)
compiled from the reference headers - not from the restatement in
cuda-kmeans_b200/cli/reference_data.hpp, which these vectors exist to pin.  The reference checkout
is needed to run this script (python tests/golden/make_refdata_golden.py); the committed .npz
travels without it.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402

# (n, k, dim, seed, layout, layout_means): 0 = aos, 1 = soa
KMEANS_CASES = [(1000, 16, 4, 42, 0, 0), (5003, 37, 7, 7, 1, 0), (2048, 128, 20, 123, 0, 1), (300, 300, 2, 1, 1, 1)]
# (n, k, dim, seed, layout, layout_means, iterations) for the --double mode
KMEANS_F64_CASES = [(1500, 12, 5, 42, 0, 0, 4), (1025, 33, 16, 7, 1, 0, 3)]
# (n, k, dim, iterations, seed, layout name): the data array holds size(n, dim) * iterations floats
BUCKETING_CASES = [(2048, 16, 5, 2, 42, "aos"), (1000, 7, 3, 1, 9, "soa"), (2048, 16, 5, 2, 42, "soa32"), (300, 40, 33, 1, 3, "aos32")]


def layout_size(name, items, dim):
    align = 32 if name.endswith("32") else 1
    pad = lambda x: (x + align - 1) // align * align  # noqa: E731
    return pad(items) * dim if name.startswith("soa") else pad(dim) * items


def main():
    ref = oracle.ref_data()
    if ref is None:
        raise SystemExit("the reference checkout is needed to generate these vectors")
    out = {"kmeans_cases": np.array(KMEANS_CASES, dtype=np.int64)}
    for i, (n, k, d, seed, lay, laym) in enumerate(KMEANS_CASES):
        data, means = ref.kmeans_inputs(n, k, d, seed, lay, laym)
        out["kmeans_%d_data" % i] = data
        out["kmeans_%d_means" % i] = means
    # --double: the double-typed distributions give an unrelated stream; two small cases, with the
    # reference's own serial k-means in double run on them (oracle/_ref/libkmref.so)
    out["kmeans_f64_cases"] = np.array(KMEANS_F64_CASES, dtype=np.int64)
    serial = oracle.ref()
    for i, (n, k, d, seed, lay, laym, iters) in enumerate(KMEANS_F64_CASES):
        data, means = ref.kmeans_inputs_f64(n, k, d, seed, lay, laym)
        out["kmeans_f64_%d_data" % i] = data
        out["kmeans_f64_%d_means" % i] = means
        out_means, out_asg = serial.kmeans_f64(data, means, n, k, d, iters, lay, laym)
        out["kmeans_f64_%d_out_means" % i] = out_means
        out["kmeans_f64_%d_out_assignment" % i] = out_asg
    out["bucketing_cases"] = np.array([(n, k, d, it, seed) for (n, k, d, it, seed, _) in BUCKETING_CASES], dtype=np.int64)
    out["bucketing_layouts"] = np.array([c[5] for c in BUCKETING_CASES])
    for i, (n, k, d, it, seed, lay) in enumerate(BUCKETING_CASES):
        data, idx = ref.bucketing_inputs(layout_size(lay, n, d) * it, n * it, k, seed)
        out["bucketing_%d_data" % i] = data
        out["bucketing_%d_indices" % i] = idx
    path = os.path.join(HERE, "refdata_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
