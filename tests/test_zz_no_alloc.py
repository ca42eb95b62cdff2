"""GPU: bkm_update_noalloc_f32 - the update step for callers that can neither pass a workspace
nor allocate one (a runner behind the reference's kernel interface gets only the problem
instance and runs inside the timed loop; an application may have given all device memory to its
own pool).  The entry point works on a fixed array inside the library, so this test checks,
through the C ABI, that it returns what bkm_update_f32 returns and what the CPU oracle's update
(serial.hpp:44-73 restated) returns - twice in a row on different inputs, because the array
keeps the previous call's contents - that it works at exactly its stated size limit, refuses
one value more, and reports an out-of-range assignment through bkm_noalloc_check.  The file
name sorts last on purpose: a run that stops at the first failure has then already run every
other test."""
import numpy as np
import pytest

from helpers import DeviceArrays, means_close, rows_to_layout

pytestmark = pytest.mark.gpu


def _both(pkg, torch, rows, asg, k, layout, layout_means):
    n, d = rows.shape
    data = rows_to_layout(rows, layout)
    dev = DeviceArrays(torch, pkg, data, np.zeros(k * d, np.float32), n, k, d)
    dev.assignment = torch.from_numpy(asg.astype(np.int64).astype(np.int32)).to("cuda:0")
    # existing entry point, caller-provided workspace
    pkg.update(dev.points.data_ptr(), dev.assignment.data_ptr(), dev.means_out.data_ptr(), dev.sizes.data_ptr(),
               n, k, d, layout, layout_means, dev.ws_ptr, dev.ws_bytes_avail)
    pkg.workspace_check(dev.ws_ptr)
    want_means, want_sizes = dev.means_out.cpu().numpy().copy(), dev.sizes.cpu().numpy().copy()
    # new entry point: no workspace argument at all
    got_means = torch.full((k * d,), float("nan"), dtype=torch.float32, device="cuda:0")
    got_sizes = torch.full((k,), -1, dtype=torch.int32, device="cuda:0")
    pkg.update_noalloc(dev.points.data_ptr(), dev.assignment.data_ptr(), got_means.data_ptr(), got_sizes.data_ptr(),
                       n, k, d, layout, layout_means)
    pkg.noalloc_check()
    return data, got_means.cpu().numpy(), got_sizes.cpu().numpy(), want_means, want_sizes


def test_noalloc_update_matches_workspace_update_twice_in_a_row(pkg, torch_cuda, oracle_mod):
    rng = np.random.default_rng(77)
    # two different problems back to back: the second must not see leftovers of the first
    cases = [(30000, 1024, 32, 1, 1), (20011, 37, 5, 0, 1), (4096, 64, 2, 0, 0), (9000, 300, 40, 1, 0)]
    for (n, k, d, layout, layout_means) in cases:
        for call in range(2):
            rows = (rng.random((n, d), dtype=np.float32) + call).astype(np.float32)
            asg = rng.integers(0, k, n).astype(np.uint32)
            if k > 2:
                asg[asg == 1] = 0                      # one empty cluster: its mean must be zero
            data, got_means, got_sizes, want_means, want_sizes = _both(pkg, torch_cuda, rows, asg, k, layout, layout_means)
            assert np.array_equal(got_sizes, want_sizes), (n, k, d, call)
            ok, err = means_close(got_means, want_means)
            assert ok, (n, k, d, call, err)
            # the oracle: sizes exactly, means within 1e-4 (helpers.MEANS_RTOL)
            o_means, o_sizes = oracle_mod.update(data, asg, n, k, d, layout, layout_means)
            assert np.array_equal(got_sizes.view(np.uint32), o_sizes), (n, k, d, call)
            ok, err = means_close(got_means, o_means)
            assert ok, (n, k, d, call, err)


def test_noalloc_update_at_exactly_its_limit(pkg, torch_cuda, oracle_mod):
    """k*dim + k == BKM_NOALLOC_MAX_WORDS: a single copy of the accumulators fills the array."""
    k, d = 8190, 63
    assert k * d + k == pkg.NOALLOC_MAX_WORDS
    n = 20000
    rng = np.random.default_rng(5)
    for call in range(2):
        rows = (rng.random((n, d), dtype=np.float32) - call).astype(np.float32)
        asg = rng.integers(0, k, n).astype(np.uint32)
        data, got_means, got_sizes, want_means, want_sizes = _both(pkg, torch_cuda, rows, asg, k, 0, 0)
        o_means, o_sizes = oracle_mod.update(data, asg, n, k, d, 0, 0)
        assert np.array_equal(got_sizes.view(np.uint32), o_sizes), call
        ok, err = means_close(got_means, o_means)
        assert ok, (call, err)
        assert np.array_equal(got_sizes, want_sizes)


def test_noalloc_update_rejects_sizes_beyond_its_scratch(pkg, torch_cuda):
    torch = torch_cuda
    # far beyond the limit, and exactly one value beyond it (k*dim + k = 524161)
    for (n, k, d) in ((256, 8192, 64), (4, 1, pkg.NOALLOC_MAX_WORDS)):
        assert k * d + k > pkg.NOALLOC_MAX_WORDS
        pts = torch.zeros(n * d, dtype=torch.float32, device="cuda:0")
        asg = torch.zeros(n, dtype=torch.int32, device="cuda:0")
        means = torch.zeros(k * d, dtype=torch.float32, device="cuda:0")
        sizes = torch.zeros(k, dtype=torch.int32, device="cuda:0")
        with pytest.raises(pkg.BkmError) as e:
            pkg.update_noalloc(pts.data_ptr(), asg.data_ptr(), means.data_ptr(), sizes.data_ptr(), n, k, d, 0, 0)
        assert e.value.code == pkg.ERR_UNSUPPORTED
        assert "scratch" in str(e.value)


def test_noalloc_update_reports_an_out_of_range_assignment(pkg, torch_cuda, oracle_mod):
    torch = torch_cuda
    n, k, d = 5000, 50, 8
    rng = np.random.default_rng(9)
    rows = rng.random((n, d), dtype=np.float32)
    asg = rng.integers(0, k, n).astype(np.uint32)
    bad = asg.copy()
    bad[123] = k + 7                                     # not a cluster: skipped and reported
    pts = torch.from_numpy(rows.reshape(-1)).to("cuda:0")
    dasg = torch.from_numpy(bad.astype(np.int64).astype(np.int32)).to("cuda:0")
    means = torch.zeros(k * d, dtype=torch.float32, device="cuda:0")
    sizes = torch.zeros(k, dtype=torch.int32, device="cuda:0")
    pkg.update_noalloc(pts.data_ptr(), dasg.data_ptr(), means.data_ptr(), sizes.data_ptr(), n, k, d, 0, 0)
    with pytest.raises(pkg.BkmError) as e:
        pkg.noalloc_check()
    assert e.value.code == pkg.ERR_DEVICE
    assert int(sizes.sum().item()) == n - 1
    # the next call starts from a clean status
    dasg = torch.from_numpy(asg.astype(np.int64).astype(np.int32)).to("cuda:0")
    pkg.update_noalloc(pts.data_ptr(), dasg.data_ptr(), means.data_ptr(), sizes.data_ptr(), n, k, d, 0, 0)
    pkg.noalloc_check()
    o_means, o_sizes = oracle_mod.update(rows.reshape(-1), asg, n, k, d, 0, 0)
    assert np.array_equal(sizes.cpu().numpy().view(np.uint32), o_sizes)
    ok, err = means_close(means.cpu().numpy(), o_means)
    assert ok, err
