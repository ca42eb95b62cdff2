"""GPU: the update entry point (bkm_update_f32) and the whole-iteration entry point
(bkm_iterate_f32) against the oracle."""
import numpy as np
import pytest

from helpers import DeviceArrays, means_close, rows_to_layout

pytestmark = pytest.mark.gpu


def _run_update(pkg, torch, data, asg, n, k, d, layout, layout_means, variant):
    dev = DeviceArrays(torch, pkg, data, np.zeros(k * d, np.float32), n, k, d)
    dev.assignment = torch.from_numpy(asg.astype(np.int64).astype(np.int32)).to("cuda:0")
    pkg.update(dev.points.data_ptr(), dev.assignment.data_ptr(), dev.means_out.data_ptr(), dev.sizes.data_ptr(),
               n, k, d, layout, layout_means, dev.ws_ptr, dev.ws_bytes_avail, variant=variant)
    pkg.workspace_check(dev.ws_ptr)
    return dev.means_out.cpu().numpy(), dev.sizes.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("n,k,d", [
    (1, 1, 1), (100, 3, 2), (1000, 16, 4), (5000, 64, 2), (4097, 33, 7), (3000, 100, 16),
    (8192, 1024, 32), (2000, 20, 33), (1500, 10, 100), (3000, 2000, 40),
])
def test_update_matches_oracle(pkg, torch_cuda, oracle_mod, n, k, d):
    rng = np.random.default_rng(n + 7 * k + 13 * d)
    rows = rng.random((n, d), dtype=np.float32) + 0.5
    asg = rng.integers(0, k, n).astype(np.uint32)
    if k > 2:
        asg[asg == 1] = 0                       # cluster 1 stays empty
    for layout, layout_means in ((0, 0), (1, 1), (0, 1), (1, 0)):
        data = rows_to_layout(rows, layout)
        want64, want_sizes = oracle_mod.update_f64(data, asg, n, k, d, layout, layout_means)
        want32, _ = oracle_mod.update(data, asg, n, k, d, layout, layout_means)
        variants = [pkg.UPDATE_AUTO, pkg.UPDATE_GLOBAL, pkg.UPDATE_ROWS]
        if k * ((d | 1) + 1) * 4 <= 227 * 1024 - 1024:
            variants.append(pkg.UPDATE_SHARED)
        if k <= 1024:
            variants.append(pkg.UPDATE_SORTED)
        for variant in variants:
            means, sizes = _run_update(pkg, torch_cuda, data, asg, n, k, d, layout, layout_means, variant)
            assert np.array_equal(sizes, want_sizes), (layout, layout_means, variant)
            ok, err = means_close(means, want64, rtol=1e-5)
            assert ok, (layout, layout_means, variant, err)
            ok, err = means_close(means, want32)
            assert ok, (layout, layout_means, variant, err)


def test_empty_cluster_is_all_zero(pkg, torch_cuda):
    n, k, d = 1000, 8, 4
    rows = np.random.default_rng(1).random((n, d), dtype=np.float32)
    asg = (np.arange(n) % 4).astype(np.uint32)          # clusters 4..7 empty
    means, sizes = _run_update(pkg, torch_cuda, rows.reshape(-1), asg, n, k, d, 0, 0, pkg.UPDATE_AUTO)
    assert np.all(means.reshape(k, d)[4:] == 0.0)
    assert np.array_equal(sizes, [250, 250, 250, 250, 0, 0, 0, 0])


def test_hot_cluster_and_zipf(pkg, torch_cuda, oracle_mod):
    """All points in one bucket, and Zipf-distributed buckets (atomic contention cases)."""
    rng = np.random.default_rng(2)
    n, k, d = 200000, 64, 2
    rows = rng.random((n, d), dtype=np.float32)
    w = 1.0 / np.arange(1, k + 1) ** 1.1
    for asg in (np.zeros(n, np.uint32), rng.choice(k, n, p=w / w.sum()).astype(np.uint32)):
        for layout in (0, 1):
            data = rows_to_layout(rows, layout)
            want64, want_sizes = oracle_mod.update_f64(data, asg, n, k, d, layout, layout)
            for variant in (pkg.UPDATE_SHARED, pkg.UPDATE_GLOBAL, pkg.UPDATE_ROWS, pkg.UPDATE_SORTED):
                means, sizes = _run_update(pkg, torch_cuda, data, asg, n, k, d, layout, layout, variant)
                assert np.array_equal(sizes, want_sizes)
                # a single fp32 accumulator summed in arrival order drifts like the reference's own
                # sequential sum; the privatised variant is hierarchical and stays tighter
                ok, err = means_close(means, want64, rtol=1e-5 if variant in (pkg.UPDATE_SHARED, pkg.UPDATE_SORTED) else 1e-4)
                assert ok, (layout, variant, err)


def test_out_of_range_assignment_is_reported_not_faulted(pkg, torch_cuda):
    n, k, d = 512, 4, 3
    rows = np.ones((n, d), np.float32)
    asg = np.zeros(n, np.uint32)
    asg[7] = 99
    dev = DeviceArrays(torch_cuda, pkg, rows.reshape(-1), np.zeros(k * d, np.float32), n, k, d)
    dev.assignment = torch_cuda.from_numpy(asg.astype(np.int32)).to("cuda:0")
    for variant in (pkg.UPDATE_SHARED, pkg.UPDATE_GLOBAL, pkg.UPDATE_ROWS, pkg.UPDATE_SORTED):
        pkg.update(dev.points.data_ptr(), dev.assignment.data_ptr(), dev.means_out.data_ptr(), dev.sizes.data_ptr(),
                   n, k, d, 0, 0, dev.ws_ptr, dev.ws_bytes_avail, variant=variant)
        with pytest.raises(pkg.BkmError) as e:
            pkg.workspace_check(dev.ws_ptr)
        assert e.value.code == pkg.ERR_DEVICE
        sizes = dev.sizes.cpu().numpy()
        assert sizes[0] == n - 1


def test_iterate_entry_point(pkg, torch_cuda, oracle_mod, golden):
    for c in golden[:12]:
        n, k, d = c["n"], c["k"], c["d"]
        dev = DeviceArrays(torch_cuda, pkg, c["data"], c["means"], n, k, d)
        for with_asg in (True, False):
            pkg.iterate(dev.points.data_ptr(), dev.means.data_ptr(), dev.means_out.data_ptr(), dev.sizes.data_ptr(),
                        dev.assignment.data_ptr() if with_asg else None, n, k, d, c["layout"], c["layout_means"],
                        dev.ws_ptr, dev.ws_bytes_avail)
            pkg.workspace_check(dev.ws_ptr)
            want_asg = c["first_assignment"]
            want_means, want_sizes = oracle_mod.update(c["data"], want_asg, n, k, d, c["layout"], c["layout_means"])
            if with_asg:
                assert np.array_equal(dev.asg_host(), want_asg), c["name"]
            assert np.array_equal(dev.sizes.cpu().numpy().view(np.uint32), want_sizes), c["name"]
            ok, err = means_close(dev.means_out.cpu().numpy(), want_means)
            assert ok, (c["name"], err)
