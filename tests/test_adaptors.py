"""The C++ adaptors (include/bkm_reference_adaptors.hpp) against the reference's own headers.

The check program (tests/cpp/adaptor_check.cpp) can only be compiled where the reference
checkout is present (it includes the reference's kernels.cuh / interface.hpp / serial.hpp);
the binary it produces travels to the GPU machine, where the `gpu` test runs a small k-means
through B200KMeansAlgorithm and compares it with the reference's SerialKMeansAlgorithm in the
same process."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "adaptor_check")
REF_HEADERS = os.path.join(os.environ.get("KMEANS_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference"),
                           "experimental", "k-means", "k-means", "headers")


def build_adaptor_check(pkg_dir):
    """Compiles the check program; returns its path or None when the reference is absent."""
    if not os.path.isfile(os.path.join(REF_HEADERS, "kernels.cuh")):
        return BIN if os.path.exists(BIN) else None
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++14", "-O2", "-I", os.path.join(ROOT, "include"), "-I", REF_HEADERS,
           "-I", os.path.join(cuda, "include"), os.path.join(ROOT, "tests", "cpp", "adaptor_check.cpp"),
           "-o", BIN, "-L", pkg_dir, "-lbkm", "-L", os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath," + pkg_dir, "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    subprocess.check_call(cmd)
    return BIN


def test_adaptors_compile_against_reference_headers(pkg):
    path = build_adaptor_check(os.path.dirname(pkg.LIB_PATH))
    if path is None:
        pytest.skip("reference checkout absent and no prebuilt check program")
    out = subprocess.run([path], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "adaptor check ok" in out.stdout


@pytest.mark.gpu
def test_adaptors_match_reference_serial_on_gpu(pkg, torch_cuda):
    if not os.path.exists(BIN):
        pytest.skip("check program was not built (needs the reference checkout at build time)")
    out = subprocess.run([BIN, "gpu"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "adaptor check ok" in out.stdout
