"""GPU: seeded random shapes through the k-means handle (tensor-core assignment + update), every
iteration checked step-wise against the oracle: the assignment bit for bit for the means the GPU
started the iteration with, the new means within 1e-4 (relative to the larger of the value and one
percent of the largest mean coordinate), the sizes exactly."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

DIMS = [9, 12, 16, 17, 20, 23, 24, 28, 31, 32, 33, 40, 64]
KS = [2, 17, 100, 255, 256, 257, 300, 512, 700, 1000, 1024, 1025]
NS = [1, 100, 127, 129, 255, 257, 1000, 4097, 20000]


def _cases(seed, count):
    rng = np.random.default_rng(seed)
    return [(int(rng.choice(NS)), int(rng.choice(KS)), int(rng.choice(DIMS)), int(rng.integers(0, 2)), int(rng.integers(0, 2)),
             int(rng.integers(0, 3))) for _ in range(count)]


@pytest.mark.parametrize("n,k,d,layout,layout_means,kind", _cases(2024, 24))
def test_random_shape_iterations_match_oracle(pkg, torch_cuda, oracle_mod, n, k, d, layout, layout_means, kind):
    rng = np.random.default_rng(n * 7919 + k * 31 + d)
    if kind == 0:        # uniform cloud, means near points
        rows = rng.random((n, d), dtype=np.float32) + rng.normal(0, 0.3, (1, d)).astype(np.float32)
        cent = rows[rng.integers(0, n, k)] + rng.normal(0, 0.01, (k, d)).astype(np.float32)
    elif kind == 1:      # tight clusters far from the origin (cancellation in the GEMM form)
        base = (10.0 + rng.random((k, d))).astype(np.float32)
        rows = (base[rng.integers(0, k, n)] + 0.01 * rng.standard_normal((n, d))).astype(np.float32)
        cent = base
    else:                # duplicated means: exact ties, the lower index must win
        rows = rng.random((n, d), dtype=np.float32)
        cent = rng.random((k, d), dtype=np.float32)
        cent[k // 2:k // 2 * 2] = cent[:k // 2]
    data = np.ascontiguousarray(rows if layout == 0 else rows.T).ravel()
    means = np.ascontiguousarray(cent if layout_means == 0 else cent.T).ravel()
    km = pkg.KMeans(layout=layout, layout_means=layout_means, variant_assign=pkg.ASSIGN_TC)
    try:
        km.initialize(d, k, n, 2, data, means)
        prev = means.copy()
        for it in range(2):
            km.run(1)
            asg, cur, sizes = km.getAssignment(), km.getMeans(), km.getSizes()
            want = oracle_mod.assign(data, prev, n, k, d, layout, layout_means, threads=8)
            assert np.array_equal(asg, want), (it, int((asg != want).sum()))
            want_means, want_sizes = oracle_mod.update(data, asg, n, k, d, layout, layout_means)
            assert np.array_equal(sizes, want_sizes), it
            scale = np.maximum(np.abs(want_means), 0.01 * max(float(np.abs(want_means).max()), 1e-30))
            assert float((np.abs(cur - want_means) / scale).max()) <= 1e-4, it      # tolerance of the means: 1e-4
            prev = cur
    finally:
        km.cleanup()
