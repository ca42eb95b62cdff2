"""CPU: the command-line harnesses work on the reference executables' own inputs.

cuda-kmeans_b200/cli/reference_data.hpp restates the reference's generators
(experimental/k-means/k-means/headers/data.hpp:19-81: generate_clustered_data, prepare_means,
generate_random) call for call.  The fixture tests/golden/refdata_golden.npz was taken from the
reference's own code (tests/golden/make_refdata_golden.py); where the compiled reference is at hand
(oracle/_ref/libkmrefdata.so) further seeds are compared with it directly."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LAYOUTS = ["aos", "soa"]


@pytest.fixture(scope="module")
def cli_dir():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    builder = ge._load_file("bkm_build", os.path.join(ge.PKG_DIR, "build.py"))
    return os.path.dirname(builder.build_cli())


@pytest.fixture(scope="module")
def refdata_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "refdata_golden.npz"))


def _dump(cli_dir, tmp_path, n, k, d, seed, lay, laym):
    path = str(tmp_path / "inputs.bin")
    p = subprocess.run([os.path.join(cli_dir, "bkm-kmeans"), "--N", str(n), "--k", str(k), "--dim", str(d), "--seed", str(seed),
                        "--layout", LAYOUTS[lay], "--layoutMeans", LAYOUTS[laym], "--dumpInputs", path, "--dryRun"],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, (p.stdout, p.stderr)
    raw = np.fromfile(path, dtype=np.uint8)
    assert list(raw[:24].view(np.uint64)) == [n, k, d]
    body = raw[24:].view(np.float32)
    return body[:n * d], body[n * d:]


def test_kmeans_inputs_equal_the_reference_generator_golden(cli_dir, tmp_path, refdata_golden):
    for i, (n, k, d, seed, lay, laym) in enumerate(refdata_golden["kmeans_cases"].tolist()):
        data, means = _dump(cli_dir, tmp_path, n, k, d, seed, lay, laym)
        assert np.array_equal(data, refdata_golden["kmeans_%d_data" % i]), (n, k, d, seed)
        assert np.array_equal(means, refdata_golden["kmeans_%d_means" % i]), (n, k, d, seed)


def test_kmeans_inputs_equal_the_compiled_reference(cli_dir, tmp_path, oracle_mod):
    ref = oracle_mod.ref_data()
    if ref is None:
        pytest.skip("compiled reference generators not available")
    for (n, k, d, seed, lay, laym) in [(777, 9, 3, 5, 0, 1), (4096, 64, 32, 2024, 1, 1)]:
        data, means = _dump(cli_dir, tmp_path, n, k, d, seed, lay, laym)
        want_data, want_means = ref.kmeans_inputs(n, k, d, seed, lay, laym)
        assert np.array_equal(data, want_data) and np.array_equal(means, want_means), (n, k, d, seed)


def _size(name, items, dim):
    align = 32 if name.endswith("32") else 1
    pad = lambda x: (x + align - 1) // align * align  # noqa: E731
    return pad(items) * dim if name.startswith("soa") else pad(dim) * items


def _at(name, flat, items, dim):
    """(items, dim) view of one padded batch."""
    align = 32 if name.endswith("32") else 1
    pad = lambda x: (x + align - 1) // align * align  # noqa: E731
    if name.startswith("soa"):
        return flat.reshape(dim, pad(items))[:, :items].T
    return flat.reshape(items, pad(dim))[:, :dim]


def test_bucketing_serial_sums_on_the_reference_inputs(cli_dir, tmp_path, refdata_golden):
    """bkm-bucketing --algorithm serial --out must print the per-bucket sums of the REFERENCE's inputs
    for the same arguments (which pins the restated generate_random streams and the layout padding)."""
    for i, ((n, k, d, iters, seed), lay) in enumerate(zip(refdata_golden["bucketing_cases"].tolist(), refdata_golden["bucketing_layouts"].tolist())):
        out = str(tmp_path / ("sums_%d.txt" % i))
        p = subprocess.run([os.path.join(cli_dir, "bkm-bucketing"), "--N", str(n), "--k", str(k), "--dim", str(d), "--iterations", str(iters),
                            "--seed", str(seed), "--layout", lay, "--algorithm", "serial", "--out", out],
                           capture_output=True, text=True, timeout=120)
        assert p.returncode == 0, (p.stdout, p.stderr)
        ms, ns = p.stdout.split()
        assert float(ms) >= 0 and float(ns) >= 0
        got = np.loadtxt(out, dtype=np.float64).reshape(iters, k, d)
        data, idx = refdata_golden["bucketing_%d_data" % i], refdata_golden["bucketing_%d_indices" % i]
        per = _size(lay, n, d)
        for it in range(iters):
            rows = _at(lay, data[it * per:(it + 1) * per], n, d)
            want = np.zeros((k, d), dtype=np.float32)
            np.add.at(want, idx[it * n:(it + 1) * n], rows)
            assert np.allclose(got[it], want, rtol=2e-5, atol=1e-6), (lay, it)


def test_bucketing_flags_defaults_and_errors(cli_dir):
    exe = os.path.join(cli_dir, "bkm-bucketing")
    p = subprocess.run([exe, "--dryRun"], capture_output=True, text=True)
    assert p.returncode == 0 and "N=10240 k=512 dim=20 iterations=1 seed=42 layout=aos algorithm=serial" in p.stdout
    p = subprocess.run([exe, "--N", "8M", "--k", "1k", "--dim", "32", "--layout", "soa32", "--algorithm", "b200_fake", "--itemsPerThread", "4",
                        "--privatizedCopies", "2", "--emul", "--cudaBlockSize", "256", "--dryRun"], capture_output=True, text=True)
    assert p.returncode == 0 and "N=8388608 k=1024 dim=32" in p.stdout and "itemsPerThread=4" in p.stdout
    for bad in (["--double"], ["--layout", "aos64"], ["--N", "64"], ["--bogus"]):
        p = subprocess.run([exe] + bad, capture_output=True, text=True)
        assert p.returncode == 1 and p.stdout.startswith("Invalid arguments:"), bad
    p = subprocess.run([exe, "--algorithm", "nope"], capture_output=True, text=True)
    assert p.returncode == 2 and p.stdout.startswith("Error: Unkown algorithm 'nope'.")


@pytest.mark.gpu
@pytest.mark.parametrize("args", [
    ["--N", "64k", "--k", "1k", "--dim", "32", "--iterations", "2", "--layout", "aos", "--algorithm", "b200"],
    ["--N", "20000", "--k", "100", "--dim", "7", "--layout", "soa", "--algorithm", "b200"],
    ["--N", "20000", "--k", "100", "--dim", "7", "--layout", "soa32", "--algorithm", "b200"],
    ["--N", "8k", "--k", "50", "--dim", "20", "--layout", "aos32", "--algorithm", "b200_sorted"],
    ["--N", "16k", "--k", "64", "--dim", "16", "--layout", "soa", "--algorithm", "b200_rows"],
    ["--N", "16k", "--k", "64", "--dim", "4", "--layout", "soa", "--algorithm", "b200_shared"],
    ["--N", "16k", "--k", "5000", "--dim", "24", "--layout", "aos", "--algorithm", "b200_global"],
    ["--N", "64k", "--k", "256", "--dim", "8", "--layout", "aos", "--algorithm", "b200_fake", "--itemsPerThread", "4"],
    ["--N", "64k", "--k", "256", "--dim", "8", "--layout", "soa", "--algorithm", "b200_fake_shm"],
])
def test_bucketing_verify_on_gpu(cli_dir, args):
    p = subprocess.run([os.path.join(cli_dir, "bkm-bucketing")] + args + ["--verify"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout, p.stderr)
    assert "Verifying results ... OK" in p.stderr
    ms, ns = p.stdout.split()
    assert float(ms) > 0 and float(ns) > 0


# ---- the fp64 path (the reference executable's --double mode) ------------------------------------

def _dump_f64(cli_dir, tmp_path, n, k, d, seed, lay, laym):
    path = str(tmp_path / "inputs64.bin")
    p = subprocess.run([os.path.join(cli_dir, "bkm-kmeans"), "--N", str(n), "--k", str(k), "--dim", str(d), "--seed", str(seed),
                        "--layout", LAYOUTS[lay], "--layoutMeans", LAYOUTS[laym], "--double", "--dumpInputs", path, "--dryRun"],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, (p.stdout, p.stderr)
    raw = np.fromfile(path, dtype=np.uint8)
    assert list(raw[:24].view(np.uint64)) == [n, k, d]
    body = raw[24:].view(np.float64)
    return body[:n * d], body[n * d:]


def test_double_inputs_equal_the_reference_generator_golden(cli_dir, tmp_path, refdata_golden):
    for i, (n, k, d, seed, lay, laym, iters) in enumerate(refdata_golden["kmeans_f64_cases"].tolist()):
        data, means = _dump_f64(cli_dir, tmp_path, n, k, d, seed, lay, laym)
        assert np.array_equal(data, refdata_golden["kmeans_f64_%d_data" % i])
        assert np.array_equal(means, refdata_golden["kmeans_f64_%d_means" % i])


def test_double_oracle_equals_the_reference_serial_golden(oracle_mod, refdata_golden):
    """oracle.kmeans_f64 (serial.hpp restated with F = double) bit for bit against the reference's own
    SerialKMeansAlgorithm<double> on the reference's own --double inputs."""
    for i, (n, k, d, seed, lay, laym, iters) in enumerate(refdata_golden["kmeans_f64_cases"].tolist()):
        means, asg = oracle_mod.kmeans_f64(refdata_golden["kmeans_f64_%d_data" % i], refdata_golden["kmeans_f64_%d_means" % i],
                                           n, k, d, iters, lay, laym)
        assert np.array_equal(means, refdata_golden["kmeans_f64_%d_out_means" % i])
        assert np.array_equal(asg, refdata_golden["kmeans_f64_%d_out_assignment" % i])


@pytest.mark.gpu
def test_double_path_matches_the_oracle_on_gpu(pkg, torch_cuda, oracle_mod, refdata_golden):
    """bkm_kmeans_host_f64: assignments bit for bit for one iteration (same means in), final means of
    the whole run within 1e-9 relative (the sums are accumulated in another order), and the golden
    trajectories of the reference."""
    rng = np.random.default_rng(4)
    for (n, k, d, lay, laym) in [(5000, 37, 7, 0, 1), (3000, 300, 33, 1, 1), (4096, 16, 2, 0, 0)]:
        rows = rng.random((n, d))
        data = rows.reshape(-1) if lay == 0 else np.ascontiguousarray(rows.T).reshape(-1)
        m0 = rows[:k].reshape(-1) if laym == 0 else np.ascontiguousarray(rows[:k].T).reshape(-1)
        got_means, got_asg = pkg.kmeans_host_f64(data, m0, n, k, d, 1, lay, laym)
        assert np.array_equal(got_asg, oracle_mod.assign_f64(data, m0, n, k, d, lay, laym, threads=8))
        want_means, _ = oracle_mod.update_d(data, got_asg, n, k, d, lay, laym)
        assert np.allclose(got_means, want_means, rtol=1e-12, atol=1e-15)
        got_means, got_asg = pkg.kmeans_host_f64(data, m0, n, k, d, 5, lay, laym)
        want_means, want_asg = oracle_mod.kmeans_f64(data, m0, n, k, d, 5, lay, laym)
        assert np.allclose(got_means, want_means, rtol=1e-9, atol=1e-12)
        assert (got_asg != want_asg).mean() <= 1e-3
    for i, (n, k, d, seed, lay, laym, iters) in enumerate(refdata_golden["kmeans_f64_cases"].tolist()):
        got_means, got_asg = pkg.kmeans_host_f64(refdata_golden["kmeans_f64_%d_data" % i], refdata_golden["kmeans_f64_%d_means" % i],
                                                 n, k, d, iters, lay, laym)
        assert np.allclose(got_means, refdata_golden["kmeans_f64_%d_out_means" % i], rtol=1e-9, atol=1e-12)
        assert (got_asg != refdata_golden["kmeans_f64_%d_out_assignment" % i]).mean() <= 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("args", [
    ["--N", "16k", "--k", "64", "--dim", "8", "--iterations", "4"],
    ["--N", "8k", "--k", "100", "--dim", "20", "--iterations", "2", "--layout", "soa", "--layoutMeans", "aos"],
    ["--N", "8k", "--k", "32", "--dim", "4", "--assignmentOnly"],
])
def test_double_verify_on_gpu(cli_dir, args):
    p = subprocess.run([os.path.join(cli_dir, "bkm-kmeans")] + args + ["--double", "--verify"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout, p.stderr)
    assert "Verifying results ... OK" in p.stderr
