"""GPU: the fixed-iteration driver (bkm_create ... bkm_run) against the oracle: golden
trajectories, the benchmark configurations at reduced size, and size-independent properties
at full size."""
import numpy as np
import pytest

from helpers import assignment_mismatches, means_close

pytestmark = pytest.mark.gpu


def _stepwise(pkg, oracle, data, means, n, k, d, iters, layout, layout_means, **kw):
    """Runs `iters` iterations one at a time; after each, the GPU's assignment must equal the
    oracle's assignment for the GPU's previous means (near-ties excepted), and the GPU's means
    the oracle's update of that assignment."""
    km = pkg.KMeans(layout=layout, layout_means=layout_means, **kw)
    km.initialize(d, k, n, iters, data, means)
    prev = np.asarray(means, dtype=np.float32).reshape(-1).copy()
    total_exact = 0
    for it in range(iters):
        km.run(1)
        asg, cur = km.getAssignment(), km.getMeans()
        exact, bad = assignment_mismatches(oracle, asg, data, prev, n, k, d, layout, layout_means)
        assert bad == 0, (it, exact, bad)
        total_exact += exact
        want, sizes = oracle.update(data, asg, n, k, d, layout, layout_means)
        ok, err = means_close(cur, want)
        assert ok, (it, err)
        assert np.array_equal(km.getSizes(), sizes), it
        prev = cur
    info = km.counters()
    km.cleanup()
    return total_exact, info


def test_golden_trajectories(pkg, torch_cuda, golden):
    for c in golden:
        km = pkg.KMeans(layout=c["layout"], layout_means=c["layout_means"])
        km.initialize(c["d"], c["k"], c["n"], c["iters"], c["data"], c["means"])
        km.run()
        means, asg = km.getMeans(), km.getAssignment()
        assert km.iterations_done() == c["iters"]
        km.cleanup()
        ok, err = means_close(means, c["out_means"])
        assert ok, (c["name"], err)
        assert (asg != c["out_assignment"]).mean() <= 1e-3, c["name"]


def test_golden_stepwise_every_iteration(pkg, torch_cuda, oracle_mod, golden):
    for c in golden:
        _stepwise(pkg, oracle_mod, c["data"], c["means"], c["n"], c["k"], c["d"], c["iters"],
                  c["layout"], c["layout_means"])


def test_run_is_resumable(pkg, torch_cuda, golden):
    c = golden[1]
    a = pkg.KMeans(layout=c["layout"], layout_means=c["layout_means"])
    a.initialize(c["d"], c["k"], c["n"], 4, c["data"], c["means"])
    a.run(4)
    b = pkg.KMeans(layout=c["layout"], layout_means=c["layout_means"])
    b.initialize(c["d"], c["k"], c["n"], 4, c["data"], c["means"])
    b.run(1)
    b.run(3)
    assert np.array_equal(a.getAssignment(), b.getAssignment())
    ok, _ = means_close(a.getMeans(), b.getMeans(), rtol=1e-6)
    assert ok
    # resume from saved means in a fresh handle
    saved = a.getMeans()
    a.run(1)
    r = pkg.KMeans(layout=c["layout"], layout_means=c["layout_means"])
    r.initialize(c["d"], c["k"], c["n"], 1, c["data"], c["means"])
    r.set_means(saved)
    r.run(1)
    assert np.array_equal(a.getAssignment(), r.getAssignment())
    for km in (a, b, r):
        km.cleanup()


def test_kmeans_host_entry_point(pkg, torch_cuda, golden):
    c = golden[4]
    means, asg = pkg.kmeans_host(c["data"], c["means"], c["n"], c["k"], c["d"], c["iters"], c["layout"], c["layout_means"])
    ok, err = means_close(means, c["out_means"])
    assert ok, err
    assert (asg != c["out_assignment"]).mean() <= 1e-3


@pytest.mark.parametrize("name,n,iters", [("c1", 1 << 16, 10), ("c2", 1 << 15, 3), ("c3", 1 << 18, 4), ("c5", 1 << 17, 3)])
def test_benchmark_configs_stepwise(pkg, torch_cuda, oracle_mod, workloads, name, n, iters):
    data, means, spec = workloads.make(name, n=n)
    _stepwise(pkg, oracle_mod, data, means, n, spec["k"], spec["dim"], iters, spec["layout"], spec["layout_means"])


def test_c4_shape_reduced(pkg, torch_cuda, oracle_mod, workloads):
    """dim 512: dense-contraction regime at a size the oracle finishes quickly."""
    n, k, d = 2048, 256, 512
    rows = workloads.generate_rows("sphere", n, d, k, seed=5)
    data, means = workloads.to_layout(rows, 0), workloads.to_layout(rows[:k], 0)
    _stepwise(pkg, oracle_mod, data, means, n, k, d, 2, 0, 0)


def test_variants_agree(pkg, torch_cuda, oracle_mod, workloads):
    data, means, spec = workloads.make("c1", n=1 << 14)
    outs = []
    for va in (pkg.ASSIGN_EXACT, pkg.ASSIGN_SIMT, pkg.ASSIGN_TC):
        for vu in (pkg.UPDATE_SHARED, pkg.UPDATE_GLOBAL, pkg.UPDATE_ROWS):
            km = pkg.KMeans(layout=spec["layout"], variant_assign=va, variant_update=vu)
            km.initialize(spec["dim"], spec["k"], 1 << 14, 3, data, means)
            km.run()
            outs.append((km.getAssignment(), km.getMeans()))
            km.cleanup()
    for asg, mns in outs[1:]:
        assert (asg != outs[0][0]).mean() <= 1e-3
        ok, err = means_close(mns, outs[0][1])
        assert ok, err


@pytest.mark.parametrize("n,k,d,layout", [
    (5000, 1024, 32, 1),      # four mean tiles, ragged last point tile, odd number of tiles
    (4224, 300, 20, 0),       # k padded to 512: masked columns; dim padded to 32
    (3000, 700, 12, 1),       # 16-float rows: one-CTA kernel either way
    (130, 1000, 17, 0),       # fewer point tiles than SMs
])
def test_tc_pair_kernel_matches_single_cta_kernel(pkg, torch_cuda, oracle_mod, workloads, n, k, d, layout):
    """The CTA-pair tensor-core kernel and the one-CTA kernel must both give the oracle's
    assignment (bit-exact) for the same means."""
    rows = workloads.generate_rows("mixture", n, d, 64, seed=11, sigma=0.05)
    rng = np.random.default_rng(3)
    mrows = np.ascontiguousarray(rows[rng.choice(n, k, replace=k > n)])
    data, means = workloads.to_layout(rows, layout), workloads.to_layout(mrows, layout)
    want = oracle_mod.assign(data, means, n, k, d, layout, layout, threads=8)
    for pair in (0, 1):
        km = pkg.KMeans(layout=layout, variant_assign=pkg.ASSIGN_TC)
        km.initialize(d, k, n, 1, data, means)
        km.set_option("tc_pair", pair)
        km.set_option("use_graph", 0)
        km.run(1)
        got = km.getAssignment()
        km.cleanup()
        assert np.array_equal(got, want), (pair, int((got != want).sum()))


@pytest.mark.parametrize("n,k,d,layout,sigma", [(50000, 64, 2, 0, 0.01), (30011, 16, 4, 0, 0.05), (9000, 1000, 3, 0, 0.05),
                                              (20000, 40, 8, 1, 0.05), (5000, 7, 1, 1, 0.05), (300, 500, 5, 0, 0.05)])
def test_small_dim_fused_update_matches_separate_update(pkg, torch_cuda, oracle_mod, workloads, n, k, d, layout, sigma):
    """The CUDA-core pass (dim <= 8) sorts each block of points it has assigned by cluster and adds
    them to the sums itself; the exact re-check moves the points it reassigns (tight clusters queue
    thousands of them).  Assignment, sizes and means must agree with the oracle step by step, with
    and without the fusion."""
    rows = workloads.generate_rows("mixture", n, d, 16, seed=17, sigma=sigma)
    data, means = workloads.to_layout(rows, layout), workloads.to_layout(np.ascontiguousarray(rows[:k] if k <= n else np.resize(rows, (k, d))), layout)
    for fuse in (1, 0):
        km = pkg.KMeans(layout=layout, variant_assign=pkg.ASSIGN_SIMT)
        km.initialize(d, k, n, 3, data, means)
        km.set_option("fuse_update", 2 * fuse)     # 2 = wherever possible (the default takes it for launch-bound sizes only)
        km.set_option("use_graph", 0)
        prev = np.asarray(means, dtype=np.float32).reshape(-1).copy()
        for it in range(3):
            km.run(1)
            asg, cur, sizes = km.getAssignment(), km.getMeans(), km.getSizes()
            want_asg = oracle_mod.assign(data, prev, n, k, d, layout, layout, threads=8)
            assert np.array_equal(asg, want_asg), (fuse, it, int((asg != want_asg).sum()))
            want, want_sizes = oracle_mod.update(data, asg, n, k, d, layout, layout)
            assert np.array_equal(sizes, want_sizes), (fuse, it)
            ok, err = means_close(cur, want)
            assert ok, (fuse, it, err)
            prev = cur
        assert (km.counters()["update_variant"] == "fused") == (fuse == 1)
        km.cleanup()


@pytest.mark.parametrize("n,k,d,layout", [(20000, 1024, 32, 1), (4224, 300, 20, 0), (777, 512, 24, 1)])
def test_fused_update_matches_separate_update(pkg, torch_cuda, oracle_mod, workloads, n, k, d, layout):
    """The CTA-pair kernel can accumulate the update sums itself; means, sizes and assignment must
    agree with the run that uses the separate update pass, and with the oracle step by step."""
    rows = workloads.generate_rows("mixture", n, d, 64, seed=13, sigma=0.05)
    data, means = workloads.to_layout(rows, layout), workloads.to_layout(np.ascontiguousarray(rows[:k]), layout)
    outs = []
    for fuse in (1, 0):
        km = pkg.KMeans(layout=layout, variant_assign=pkg.ASSIGN_TC)
        km.initialize(d, k, n, 3, data, means)
        km.set_option("fuse_update", fuse)
        km.set_option("use_graph", 0)
        prev = np.asarray(means, dtype=np.float32).reshape(-1).copy()
        for it in range(3):
            km.run(1)
            asg, cur, sizes = km.getAssignment(), km.getMeans(), km.getSizes()
            want_asg = oracle_mod.assign(data, prev, n, k, d, layout, layout, threads=8)
            assert np.array_equal(asg, want_asg), (fuse, it, int((asg != want_asg).sum()))
            want, want_sizes = oracle_mod.update(data, asg, n, k, d, layout, layout)
            assert np.array_equal(sizes, want_sizes), (fuse, it)
            ok, err = means_close(cur, want)
            assert ok, (fuse, it, err)
            prev = cur
        # fusion replaces the row-wise update only (dimension-major points)
        assert (km.counters()["update_variant"] == "fused") == (fuse == 1 and layout == 1)
        outs.append(prev)
        km.cleanup()


@pytest.mark.parametrize("layout,k", [(0, 96), (1, 96), (0, 300), (1, 300)])
def test_host_upload_in_chunks(pkg, torch_cuda, oracle_mod, workloads, layout, k):
    """Host points of 32 MB and more travel in chunks, each split into the tensor-core operands while
    the next is on its way (the centre comes from the first chunk); with k = 300 the kernel runs on
    CTA pairs and the fast pass of the first iteration follows the upload chunk by chunk too.  n is
    no multiple of the chunk or tile sizes.  Every point against the oracle, for both layouts."""
    n, d = 350003, 24
    rows = workloads.generate_rows("mixture", n, d, 32, seed=23, sigma=0.05)
    data, means = workloads.to_layout(rows, layout), workloads.to_layout(np.ascontiguousarray(rows[:k]), layout)
    total_exact, info = _stepwise(pkg, oracle_mod, data, means, n, k, d, 2, layout, layout)
    assert info["assign_variant"] == "tc"


@pytest.mark.parametrize("change", ["means", "fuse_update", "margin_scale"])
def test_first_pass_behind_the_upload_is_dropped_when_its_inputs_change(pkg, torch_cuda, oracle_mod, workloads, change):
    """The fast pass that ran behind the upload used the initial means and the settings of that
    moment; new means or a changed setting before the first run must make the run start over."""
    n, k, d, layout = 350003, 300, 24, 1
    rows = workloads.generate_rows("mixture", n, d, 32, seed=29, sigma=0.05)
    data, means = workloads.to_layout(rows, layout), workloads.to_layout(np.ascontiguousarray(rows[:k]), layout)
    km = pkg.KMeans(layout=layout)
    km.initialize(d, k, n, 1, data, means)
    start = np.asarray(means, dtype=np.float32).reshape(-1)
    if change == "means":
        start = workloads.to_layout(np.ascontiguousarray(rows[1000:1000 + k]), layout).reshape(-1)
        km.set_means(start)
    elif change == "fuse_update":
        km.set_option("fuse_update", 0)
    else:
        km.set_option("margin_scale", 2.0)
    km.run(1)
    asg, cur, sizes = km.getAssignment(), km.getMeans(), km.getSizes()
    info = km.counters()
    km.cleanup()
    want_asg = oracle_mod.assign(data, start, n, k, d, layout, layout, threads=8)
    assert np.array_equal(asg, want_asg), int((asg != want_asg).sum())
    want, want_sizes = oracle_mod.update(data, asg, n, k, d, layout, layout)
    assert np.array_equal(sizes, want_sizes)
    ok, err = means_close(cur, want)
    assert ok, err
    assert (info["update_variant"] == "fused") == (change != "fuse_update")


def test_graph_replay_after_a_chunked_upload(pkg, torch_cuda, workloads):
    """A replayed CUDA graph holds whole iterations: forced on a problem whose first fast pass ran
    behind the upload, it must not inherit that short first iteration.  The trajectory stays that of plain launches."""
    n, k, d, layout = 350003, 300, 24, 1
    rows = workloads.generate_rows("mixture", n, d, 32, seed=31, sigma=0.05)
    data, means = workloads.to_layout(rows, layout), workloads.to_layout(np.ascontiguousarray(rows[:k]), layout)
    outs = []
    for graph in (1, 0):
        km = pkg.KMeans(layout=layout)
        km.initialize(d, k, n, 6, data, means)
        km.set_option("use_graph", graph)
        km.run(6)
        outs.append((km.getAssignment(), km.getMeans(), km.getSizes()))
        km.cleanup()
    # The sums are added in an order that differs from run to run, so two trajectories part by some
    # near-tie points after six iterations (a few hundred of 350 000 were seen); a graph without its
    # fast pass would lose every point.
    differing = int((outs[0][0] != outs[1][0]).sum())
    assert differing <= n // 50, differing
    assert int(np.abs(outs[0][2].astype(np.int64) - outs[1][2].astype(np.int64)).max()) <= 500
    assert float(np.abs(outs[0][1] - outs[1][1]).max()) < 5e-2


def test_full_size_c2_properties(pkg, torch_cuda, oracle_mod, workloads):
    """Headline configuration at full size: conservation laws + a sampled oracle check."""
    data, means, spec = workloads.make("c2")
    n, k, d, lay = spec["n"], spec["k"], spec["dim"], spec["layout"]
    km = pkg.KMeans(layout=lay)
    km.initialize(d, k, n, 3, data, means)
    km.run(2)
    prev = km.getMeans()
    km.run(1)
    asg, cur, sizes = km.getAssignment(), km.getMeans(), km.getSizes()
    info = km.counters()
    km.cleanup()
    assert info["assign_variant"] == "tc"
    assert asg.max() < k
    assert int(sizes.astype(np.int64).sum()) == n
    assert np.array_equal(np.bincount(asg, minlength=k).astype(np.uint32), sizes)
    # sum_c size_c * mean_c == sum of all points (per dimension)
    rows = workloads.from_layout(data, n, d, lay)
    total = rows.astype(np.float64).sum(axis=0)
    got_total = (cur.reshape(d, k).T.astype(np.float64) * sizes[:, None]).sum(axis=0)
    assert np.allclose(got_total, total, rtol=1e-5)
    # sampled points: the oracle on a random subset (sub-sampled SoA columns)
    rng = np.random.default_rng(0)
    pick = np.sort(rng.choice(n, 8192, replace=False))
    sub = workloads.to_layout(rows[pick], lay)
    exact, bad = assignment_mismatches(oracle_mod, asg[pick], sub, prev, pick.size, k, d, lay, lay)
    assert bad == 0, (exact, bad)
    # idempotence of the update: recomputing the means from the returned assignment
    want64, _ = oracle_mod.update_f64(data, asg, n, k, d, lay, lay)
    ok, err = means_close(cur, want64)
    assert ok, err


def test_c4_tile_structure_split_k_loop(pkg, torch_cuda, oracle_mod, workloads):
    """dim 512 with 4096 means - the benchmarked c4 structure: 16 mean tiles through the K loop,
    neighbouring CTAs sharing a point block (split 2) and the partial-result merge kernel, then the
    dim-512 exact re-check.  Step-wise against the oracle (serial.hpp:21-73): assignment bit for bit,
    sizes exactly, means within 1e-4.  n is not a multiple of the 128-point tile."""
    n, k, d = 6007, 4096, 512
    rows = workloads.generate_rows("sphere", n, d, k, seed=17)
    data, means = workloads.to_layout(rows, 0), workloads.to_layout(rows[:k], 0)
    km = pkg.KMeans(layout=0)
    km.initialize(d, k, n, 2, data, means)
    plan = km.assign_plan()
    assert plan["kernel"] == "tc_kloop" and plan["mean_tiles"] == 16 and plan["block_split"] == 2, plan
    prev = means.copy()
    for it in range(2):
        km.run(1)
        asg, cur, sizes = km.getAssignment(), km.getMeans(), km.getSizes()
        want = oracle_mod.assign(data, prev, n, k, d, 0, 0, threads=8)
        assert np.array_equal(asg, want), (it, int((asg != want).sum()))
        want_means, want_sizes = oracle_mod.update(data, asg, n, k, d, 0, 0)
        assert np.array_equal(sizes, want_sizes), it
        ok, err = means_close(cur, want_means)
        assert ok, (it, err)
        prev = cur
    km.cleanup()


def test_c4_structure_with_a_recheck_list_longer_than_the_grid(pkg, torch_cuda, oracle_mod, workloads):
    """The same structure with the near-tie band widened until (nearly) every point is queued: the
    exact re-check then walks a list longer than its grid (blocks loop over groups instead of sharing
    them) and must still reproduce the oracle's assignment bit for bit."""
    n, k, d = 19200, 4096, 512                      # more queued points than 148 SMs x 8 blocks x 16 points
    rows = workloads.generate_rows("sphere", n, d, k, seed=19)
    data, means = workloads.to_layout(rows, 0), workloads.to_layout(rows[:k], 0)
    km = pkg.KMeans(layout=0)
    km.set_option("margin_scale", 1.0e6)
    km.initialize(d, k, n, 1, data, means)
    km.run(1)
    asg = km.getAssignment()
    info = km.counters()
    km.cleanup()
    assert info["rechecked"] > 148 * 8 * 16, info
    want = oracle_mod.assign(data, means, n, k, d, 0, 0, threads=8)
    assert np.array_equal(asg, want), int((asg != want).sum())


def test_legacy_default_stream_with_many_iterations(pkg, torch_cuda, oracle_mod, workloads):
    """bkm_set_stream(h, NULL) selects the legacy default stream (the reference drivers' stream,
    headers/cuda.hpp:70-88), which cannot be captured into a CUDA graph: a launch-bound problem with
    enough iterations for graph replay must fall back to plain launches there."""
    data, means, spec = workloads.make("c1", n=1 << 13)
    k, d, lay = spec["k"], spec["dim"], spec["layout"]
    km = pkg.KMeans(layout=lay)
    km.set_stream(0)
    km.initialize(d, k, 1 << 13, 8, data, means)
    km.run(8)
    got_means, got_asg = km.getMeans(), km.getAssignment()
    km.cleanup()
    want_means, want_asg = oracle_mod.kmeans(data, means, 1 << 13, k, d, 8, lay, lay)
    ok, err = means_close(got_means, want_means)
    assert ok, err
    assert (got_asg != want_asg).mean() <= 1e-3
