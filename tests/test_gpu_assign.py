"""GPU: the assignment entry point (bkm_assign_f32, through the C ABI) against the oracle."""
import numpy as np
import pytest

from helpers import DeviceArrays, assignment_mismatches, rows_to_layout

pytestmark = pytest.mark.gpu


def _variants(pkg, d):
    v = [pkg.ASSIGN_EXACT, pkg.ASSIGN_AUTO]
    if d <= 8:
        v.append(pkg.ASSIGN_SIMT)
    if d <= 4096:
        v.append(pkg.ASSIGN_TC)
    return v


def _run_assign(pkg, torch, data, means, n, k, d, layout, layout_means, variant):
    dev = DeviceArrays(torch, pkg, data, means, n, k, d)
    pkg.assign(dev.points.data_ptr(), dev.means.data_ptr(), dev.assignment.data_ptr(), n, k, d,
               layout, layout_means, dev.ws_ptr, dev.ws_bytes_avail, variant=variant)
    pkg.workspace_check(dev.ws_ptr)
    return dev.asg_host()


def test_golden_first_assignment_all_variants(pkg, torch_cuda, golden):
    for c in golden:
        for variant in _variants(pkg, c["d"]):
            got = _run_assign(pkg, torch_cuda, c["data"], c["means"], c["n"], c["k"], c["d"],
                              c["layout"], c["layout_means"], variant)
            assert np.array_equal(got, c["first_assignment"]), (c["name"], pkg.ASSIGN_NAMES[variant])


@pytest.mark.parametrize("n,k,d", [
    (1, 1, 1), (31, 2, 1), (33, 3, 2), (255, 17, 3), (1000, 100, 4), (4097, 129, 5), (2048, 64, 7),
    (5000, 1000, 8), (3001, 5, 9), (1024, 128, 16), (777, 130, 31), (4096, 256, 32), (513, 1024, 32),
    (2000, 37, 33), (600, 50, 64), (300, 20, 100),
])
def test_ragged_shapes_match_oracle(pkg, torch_cuda, oracle_mod, n, k, d):
    rng = np.random.default_rng(n * 131 + k * 17 + d)
    rows = rng.random((n, d), dtype=np.float32)
    centres = rng.random((k, d), dtype=np.float32)
    for layout, layout_means in ((0, 0), (1, 1), (0, 1), (1, 0)):
        data, means = rows_to_layout(rows, layout), rows_to_layout(centres, layout_means)
        want = oracle_mod.assign(data, means, n, k, d, layout, layout_means, threads=8)
        for variant in _variants(pkg, d):
            got = _run_assign(pkg, torch_cuda, data, means, n, k, d, layout, layout_means, variant)
            assert np.array_equal(got, want), (layout, layout_means, pkg.ASSIGN_NAMES[variant],
                                               int((got != want).sum()))


def test_tight_clusters_far_from_origin(pkg, torch_cuda, oracle_mod):
    """GEMM-form cancellation case: distances ~1e-3 between vectors of norm ~30."""
    rng = np.random.default_rng(5)
    for (n, k, d, variant) in [(20000, 64, 16, 3), (20000, 48, 4, 2), (8192, 256, 32, 3)]:
        centres = (10.0 + rng.random((k, d))).astype(np.float32)
        rows = (centres[rng.integers(0, k, n)] + 0.01 * rng.standard_normal((n, d))).astype(np.float32)
        data, means = rows_to_layout(rows, 0), rows_to_layout(centres, 0)
        want = oracle_mod.assign(data, means, n, k, d, 0, 0, threads=8)
        got = _run_assign(pkg, torch_cuda, data, means, n, k, d, 0, 0, variant)
        assert np.array_equal(got, want), (n, k, d, int((got != want).sum()))


def test_duplicate_means_pick_lowest_index(pkg, torch_cuda):
    rng = np.random.default_rng(9)
    for d, variants in ((4, (1, 2, 3)), (32, (1, 3)), (80, (1, 3))):
        n, k = 3000, 40
        centres = rng.random((k, d), dtype=np.float32)
        centres[20:] = centres[:20]          # every mean exists twice
        rows = rng.random((n, d), dtype=np.float32)
        for variant in variants:
            got = _run_assign(pkg, torch_cuda, rows.reshape(-1), centres.reshape(-1), n, k, d, 0, 0, variant)
            assert got.max() < 20, pkg.ASSIGN_NAMES[variant]


def test_short_recheck_list_is_shared_between_blocks(pkg, torch_cuda, oracle_mod):
    """Every mean exists twice, so every point is queued for the exact re-check; with more than 256
    means and fewer groups of queued points than blocks, the blocks split the means of a group
    between them and merge their partial results (lowest index on equal distances)."""
    rng = np.random.default_rng(21)
    for (n, k, d, layout, layout_means) in [(1200, 600, 24, 0, 0), (900, 1024, 32, 1, 1), (401, 2048, 40, 0, 1)]:
        centres = rng.random((k, d), dtype=np.float32)
        centres[k // 2:] = centres[:k // 2]
        rows = rng.random((n, d), dtype=np.float32)
        data, means = rows_to_layout(rows, layout), rows_to_layout(centres, layout_means)
        want = oracle_mod.assign(data, means, n, k, d, layout, layout_means, threads=8)
        assert want.max() < k // 2
        got = _run_assign(pkg, torch_cuda, data, means, n, k, d, layout, layout_means, pkg.ASSIGN_TC)
        assert np.array_equal(got, want), (n, k, d, int((got != want).sum()))


def test_c2_shape_sample_matches_oracle(pkg, torch_cuda, oracle_mod, workloads):
    """Headline shape (dim 32, k 1024, SoA) on 2^16 points, every point checked."""
    n = 1 << 16
    data, means, spec = workloads.make("c2", n=n, seed=11)
    k, d, lay, laym = spec["k"], spec["dim"], spec["layout"], spec["layout_means"]
    got = _run_assign(pkg, torch_cuda, data, means, n, k, d, lay, laym, pkg.ASSIGN_TC)
    exact, bad = assignment_mismatches(oracle_mod, got, data, means, n, k, d, lay, laym)
    assert bad == 0 and exact == 0, (exact, bad)


def test_unsupported_variant_is_reported(pkg, torch_cuda):
    rows = np.zeros((64, 64), np.float32)
    dev = DeviceArrays(torch_cuda, pkg, rows.reshape(-1), rows[:4].reshape(-1), 64, 4, 64)
    with pytest.raises(pkg.BkmError) as e:
        pkg.assign(dev.points.data_ptr(), dev.means.data_ptr(), dev.assignment.data_ptr(), 64, 4, 64, 0, 0,
                   dev.ws_ptr, dev.ws_bytes_avail, variant=pkg.ASSIGN_SIMT)
    assert e.value.code == pkg.ERR_UNSUPPORTED
    with pytest.raises(pkg.BkmError) as e:
        pkg.assign(dev.points.data_ptr(), dev.means.data_ptr(), dev.assignment.data_ptr(), 64, 4, 64, 0, 0,
                   dev.ws_ptr, 256, variant=pkg.ASSIGN_EXACT)
    assert e.value.code == pkg.ERR_INVALID


def test_bounded_wait_reports_instead_of_hanging(pkg, torch_cuda):
    """A barrier wait that can never complete must give up after its limit, leave the status word
    set for the host to read, and leave the context usable (no trap, no hang)."""
    import time
    ws = torch_cuda.zeros(4096, dtype=torch_cuda.uint8, device="cuda:0")
    torch_cuda.cuda.synchronize()
    t0 = time.perf_counter()
    pkg.selftest_wait_timeout(ws.data_ptr(), limit_ms=100)
    with pytest.raises(pkg.BkmError) as e:
        pkg.workspace_check(ws.data_ptr())
    dt = time.perf_counter() - t0
    assert e.value.code == pkg.ERR_DEVICE
    assert "wait timeout" in str(e.value)
    assert 0.09 <= dt < 2.0, dt                      # it waited for the limit, and only for the limit
    assert int(ws[:4].view(torch_cuda.int32).item()) & 1 == 1
    # the context is alive: a normal assignment runs right after it
    n, k, d = 3000, 300, 20
    rng = np.random.default_rng(5)
    rows = rng.random((n, d), dtype=np.float32)
    dev = DeviceArrays(torch_cuda, pkg, rows.reshape(-1), rows[:k].reshape(-1).copy(), n, k, d)
    pkg.assign(dev.points.data_ptr(), dev.means.data_ptr(), dev.assignment.data_ptr(), n, k, d, 0, 0, dev.ws_ptr, dev.ws_bytes_avail)
    pkg.workspace_check(dev.ws_ptr)
    assert int(dev.assignment.cpu().numpy().astype(np.uint32).max()) < k
