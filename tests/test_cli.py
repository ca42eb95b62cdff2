"""The command-line harness (cuda-kmeans_b200/cli/bkm_kmeans.cpp): the reference executable's flag
names, integer suffixes, output format and exit codes (k-means.cpp:297-350 of the reference)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def cli():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    builder = ge._load_file("bkm_build", os.path.join(ge.PKG_DIR, "build.py"))
    return builder.build_cli()


def _run(cli, *args):
    p = subprocess.run([cli] + list(args), capture_output=True, text=True, timeout=600)
    return p.returncode, p.stdout, p.stderr


def test_suffixes_and_defaults(cli):
    rc, out, err = _run(cli, "--N", "2M", "--k", "1k", "--dim", "32", "--iterations", "20", "--layout", "soa", "--dryRun")
    assert rc == 0
    assert "N=2097152 k=1024 dim=32 iterations=20 seed=42 layout=soa layoutMeans=soa" in out
    assert "Selected k-means algorithm: b200" in err
    rc, out, _ = _run(cli, "--dryRun")
    assert rc == 0 and "N=10240 k=128 dim=20 iterations=1" in out          # the reference's defaults


def test_invalid_arguments_exit_code_1(cli):
    for bad in (["--N", "3x"], ["--bogus"], ["--assignmentOnly", "--iterations", "3"], ["--double", "--gpus", "2"], ["--layout", "aos32"],
                ["--Rscript"]):
        rc, out, _ = _run(cli, *bad)
        assert rc == 1, bad
        assert out.startswith("Invalid arguments:"), bad


def test_tuning_flags_of_the_reference_are_accepted(cli):
    rc, _, _ = _run(cli, "--cudaBlockSize", "256", "--privatizedCopies", "4", "--itemsPerThread", "2", "--regsCache", "4",
                    "--cudaBlockCount", "0", "--cudaSharedMemorySize", "0", "--dryRun")
    assert rc == 0


def test_serial_algorithm_output_format(cli):
    rc, out, err = _run(cli, "--N", "2000", "--k", "8", "--dim", "3", "--iterations", "3", "--algorithm", "serial")
    assert rc == 0
    ms, ns = out.split()
    assert float(ms) > 0 and float(ns) > 0
    assert "Running (3 iterations)" in err and "ms/iter" in err and "ns/input float" in err


@pytest.mark.gpu
def test_verify_on_two_gpus(cli):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rc, out, err = _run(cli, "--N", "64k", "--k", "256", "--dim", "16", "--iterations", "4", "--gpus", "2", "--verify")
    assert rc == 0, (out, err)
    assert "Verifying results ... OK" in err


def test_unknown_algorithm_exit_code_2(cli):
    rc, out, _ = _run(cli, "--algorithm", "nope", "--N", "256")
    assert rc == 2 and out.startswith("Error: Unkown algorithm 'nope'.")


@pytest.mark.gpu
@pytest.mark.parametrize("args", [
    ["--N", "64k", "--k", "16", "--dim", "4", "--iterations", "5"],
    ["--N", "16k", "--k", "300", "--dim", "24", "--iterations", "3", "--layout", "soa"],
    ["--N", "8k", "--k", "64", "--dim", "40", "--iterations", "2", "--layout", "aos", "--layoutMeans", "soa"],
    ["--N", "16k", "--k", "512", "--dim", "32", "--assignmentOnly", "--layout", "soa"],
    ["--N", "4k", "--k", "32", "--dim", "8", "--iterations", "3", "--algorithm", "b200_exact"],
])
def test_verify_on_gpu(cli, args):
    rc, out, err = _run(cli, *args, "--verify")
    assert rc == 0, (out, err)
    assert "Verifying results ... OK" in err
    ms, ns = out.split()
    assert float(ms) > 0 and float(ns) > 0
