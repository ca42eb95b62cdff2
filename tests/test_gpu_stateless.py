"""GPU: the stateless runner entry points called the way the reference's drivers call their runners -
every iteration, on one workspace, with the same (immutable) points.  The workspace keeps the
operands derived from the points between calls; these tests check that a repeated call gives the
same (oracle) result, that NEW data at the same address and shape is noticed, and that
bkm_iterate_f32's single pass (assignment kernel accumulating the update sums) equals the oracle's
iteration (serial.hpp:21-73 restated in oracle/)."""
import numpy as np
import pytest

from helpers import DeviceArrays, means_close, rows_to_layout

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k,d,layout,variant", [(20000, 512, 32, 1, 3), (9000, 300, 20, 0, 3), (30000, 64, 2, 0, 2), (5000, 17, 7, 1, 2)])
def test_repeated_calls_reuse_the_workspace_and_notice_new_points(pkg, torch_cuda, oracle_mod, n, k, d, layout, variant):
    torch = torch_cuda
    rng = np.random.default_rng(n + k + d)
    rows_a = rng.random((n, d), dtype=np.float32)
    rows_b = (rng.random((n, d), dtype=np.float32) * 3.0 - 1.0).astype(np.float32)       # other values, larger norms
    means_1 = rng.random((k, d), dtype=np.float32)
    means_2 = rng.random((k, d), dtype=np.float32)
    dev = DeviceArrays(torch, pkg, rows_to_layout(rows_a, layout), rows_to_layout(means_1, layout), n, k, d)

    def call(rows, means):
        dev.means.copy_(torch.from_numpy(rows_to_layout(means, layout)).to("cuda:0"))
        pkg.assign(dev.points.data_ptr(), dev.means.data_ptr(), dev.assignment.data_ptr(), n, k, d, layout, layout,
                   dev.ws_ptr, dev.ws_bytes_avail, variant=variant)
        pkg.workspace_check(dev.ws_ptr)
        want = oracle_mod.assign(rows_to_layout(rows, layout), rows_to_layout(means, layout), n, k, d, layout, layout, threads=8)
        got = dev.asg_host()
        assert np.array_equal(got, want), int((got != want).sum())

    call(rows_a, means_1)            # first call: operands are derived
    call(rows_a, means_2)            # same points: operands reused, new means
    call(rows_a, means_1)
    # new data at the same address and shape: the fingerprint differs, the operands are derived again
    dev.points.copy_(torch.from_numpy(rows_to_layout(rows_b, layout)).to("cuda:0"))
    call(rows_b, means_2)
    call(rows_b, means_1)
    # an update on the same workspace in between must not disturb what the assignment keeps there
    pkg.update(dev.points.data_ptr(), dev.assignment.data_ptr(), dev.means_out.data_ptr(), dev.sizes.data_ptr(),
               n, k, d, layout, layout, dev.ws_ptr, dev.ws_bytes_avail)
    pkg.workspace_check(dev.ws_ptr)
    call(rows_b, means_2)


@pytest.mark.parametrize("n,k,d,layout,layout_means,want_asg", [
    (20000, 1024, 32, 1, 1, True),     # CTA-pair kernel: single pass
    (7001, 512, 24, 1, 0, False),      # same, no assignment output, other means layout
    (9000, 300, 20, 0, 0, True),       # row-major points: two passes
    (30000, 64, 2, 0, 0, True),        # CUDA cores: single pass (every warp sorts its points by cluster)
    (12345, 200, 7, 1, 0, False),      # same, dimension-major points, no assignment output
    (5000, 2000, 3, 0, 0, True),       # CUDA cores, more means than the single pass takes: two passes
])
def test_iterate_matches_oracle_iteration(pkg, torch_cuda, oracle_mod, n, k, d, layout, layout_means, want_asg):
    torch = torch_cuda
    rng = np.random.default_rng(n * 3 + k)
    rows = rng.random((n, d), dtype=np.float32)
    data = rows_to_layout(rows, layout)
    means = rows_to_layout(np.ascontiguousarray(rows[:k]), layout_means)
    dev = DeviceArrays(torch, pkg, data, means, n, k, d)
    cur = means.copy()
    for it in range(3):
        dev.means.copy_(torch.from_numpy(cur).to("cuda:0"))
        pkg.iterate(dev.points.data_ptr(), dev.means.data_ptr(), dev.means_out.data_ptr(), dev.sizes.data_ptr(),
                    dev.assignment.data_ptr() if want_asg else 0, n, k, d, layout, layout_means, dev.ws_ptr, dev.ws_bytes_avail)
        pkg.workspace_check(dev.ws_ptr)
        asg = oracle_mod.assign(data, cur, n, k, d, layout, layout_means, threads=8)
        if want_asg:
            assert np.array_equal(dev.asg_host(), asg), it
        want_means, want_sizes = oracle_mod.update(data, asg, n, k, d, layout, layout_means)
        assert np.array_equal(dev.sizes.cpu().numpy().view(np.uint32), want_sizes), it
        got = dev.means_out.cpu().numpy()
        ok, err = means_close(got, want_means)
        assert ok, (it, err)
        cur = got.copy()
