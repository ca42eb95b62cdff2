"""CPU: the plain-C oracle against the golden vectors (generated from the reference's own
serial implementation) and, where it is available, against that compiled reference directly."""
import numpy as np
import pytest


def test_golden_has_cases(golden):
    assert len(golden) >= 30


def test_oracle_matches_golden_bit_for_bit(golden, oracle_mod):
    for c in golden:
        means, asg = oracle_mod.kmeans(c["data"], c["means"], c["n"], c["k"], c["d"], c["iters"],
                                       c["layout"], c["layout_means"])
        assert np.array_equal(asg, c["out_assignment"]), c["name"]
        assert np.array_equal(means.view(np.uint32), c["out_means"].view(np.uint32)), c["name"]
        first = oracle_mod.assign(c["data"], c["means"], c["n"], c["k"], c["d"], c["layout"], c["layout_means"])
        assert np.array_equal(first, c["first_assignment"]), c["name"]


def test_oracle_threads_do_not_change_results(golden, oracle_mod):
    c = golden[5]
    a1 = oracle_mod.assign(c["data"], c["means"], c["n"], c["k"], c["d"], c["layout"], c["layout_means"], threads=1)
    a4 = oracle_mod.assign(c["data"], c["means"], c["n"], c["k"], c["d"], c["layout"], c["layout_means"], threads=4)
    assert np.array_equal(a1, a4)


def test_ties_pick_lowest_index(golden):
    c = next(c for c in golden if c["name"] == "ties_grid")
    # means 0/3 and 1/2 are duplicates: indices 3 and 2 can never be chosen
    assert not np.isin(c["first_assignment"], [2, 3]).any()


def test_empty_cluster_becomes_zero(golden):
    c = next(c for c in golden if c["name"] == "empty_cluster")
    means = c["out_means"].reshape(c["k"], c["d"])
    assert np.all(means[5] == 0.0)
    assert not np.isin(c["out_assignment"], [5]).any()


def test_oracle_matches_compiled_reference(oracle_mod):
    ref = oracle_mod.ref()
    if ref is None:
        pytest.skip("reference checkout / prebuilt oracle/_ref not present")
    rng = np.random.default_rng(3)
    for (n, k, d) in [(777, 9, 5), (1024, 64, 2), (600, 20, 40)]:
        for layout in (0, 1):
            for layout_means in (0, 1):
                rows = rng.random((n, d), dtype=np.float32)
                data = rows.reshape(-1) if layout == 0 else np.ascontiguousarray(rows.T).reshape(-1)
                m = rows[:k]
                means = m.reshape(-1) if layout_means == 0 else np.ascontiguousarray(m.T).reshape(-1)
                rm, ra = ref.kmeans(data, means, n, k, d, 3, layout, layout_means)
                om, oa = oracle_mod.kmeans(data, means, n, k, d, 3, layout, layout_means)
                assert np.array_equal(ra, oa)
                assert np.array_equal(rm.view(np.uint32), om.view(np.uint32))


def test_update_f64_close_to_f32(golden, oracle_mod):
    c = golden[0]
    m32, s32 = oracle_mod.update(c["data"], c["out_assignment"], c["n"], c["k"], c["d"], c["layout"], c["layout_means"])
    m64, s64 = oracle_mod.update_f64(c["data"], c["out_assignment"], c["n"], c["k"], c["d"], c["layout"], c["layout_means"])
    assert np.array_equal(s32, s64)
    assert np.allclose(m32, m64, rtol=1e-5, atol=1e-7)


def test_best2_consistent_with_assign(golden, oracle_mod):
    c = golden[2]
    best, second = oracle_mod.best2(c["data"], c["means"], c["n"], c["k"], c["d"], c["layout"], c["layout_means"])
    asg = oracle_mod.assign(c["data"], c["means"], c["n"], c["k"], c["d"], c["layout"], c["layout_means"])
    d = oracle_mod.dist_to(c["data"], c["means"], asg, c["n"], c["k"], c["d"], c["layout"], c["layout_means"])
    assert np.array_equal(best, d)
    assert np.all(second >= best)
