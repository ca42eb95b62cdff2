"""Shared fixtures.  Tests marked `gpu` need a CUDA device; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pkg():
    """The cuda-kmeans_b200 package with libbkm.so loaded (built on demand where nvcc exists)."""
    p = entry.load()
    if not os.path.exists(p.LIB_PATH):
        entry.build()
    p.lib()
    return p


@pytest.fixture(scope="session")
def workloads(pkg):
    import importlib
    return importlib.import_module("cuda_kmeans_b200.workloads")


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    return oracle


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "kmeans_golden.npz")
    z = np.load(path)
    cases = []
    for name in z["names"]:
        name = str(name)
        n, k, d, iters, layout, layout_means = [int(v) for v in z[name + "/shape"]]
        cases.append(dict(name=name, n=n, k=k, d=d, iters=iters, layout=layout, layout_means=layout_means,
                          data=z[name + "/data"], means=z[name + "/means"], out_means=z[name + "/out_means"],
                          out_assignment=z[name + "/out_assignment"], first_assignment=z[name + "/first_assignment"]))
    return cases


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch
