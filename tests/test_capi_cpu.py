"""CPU: the C-ABI library loads, exports what include/bkm.h declares, validates arguments and
fails loudly (never falls back) when no GPU is present."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "bkm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bkm_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(pkg):
    declared = _declared_symbols()
    assert len(declared) >= 25
    lib = ctypes.CDLL(pkg.LIB_PATH)
    missing = [s for s in declared if not hasattr(lib, s)]
    assert missing == []


def test_python_symbol_list_matches_header(pkg):
    assert sorted(pkg.SYMBOLS) == _declared_symbols()


def test_version(pkg):
    assert pkg.lib().bkm_version() >= 100


def test_shard_range_partitions_exactly(pkg):
    for n_total in (0, 1, 7, 1000, (1 << 28), (1 << 28) + 5):
        for world in (1, 2, 3, 4, 8):
            pos = 0
            counts = []
            for rank in range(world):
                b, c = pkg.shard_range(n_total, world, rank)
                assert b == pos
                pos += c
                counts.append(c)
            assert pos == n_total
            assert max(counts) - min(counts) <= 1


def test_shard_range_rejects_bad_rank(pkg):
    with pytest.raises(pkg.BkmError) as e:
        pkg.shard_range(10, 2, 2)
    assert e.value.code == pkg.ERR_INVALID


def test_workspace_bytes(pkg):
    assert pkg.workspace_bytes(0, 4, 4) == 0
    assert pkg.workspace_bytes(10, 0, 4) == 0
    small, large = pkg.workspace_bytes(1000, 16, 4), pkg.workspace_bytes(100000, 16, 4)
    assert 0 < small < large
    assert small % 256 == 0


def test_argument_validation_needs_no_gpu(pkg):
    L = pkg.lib()
    rc = L.bkm_assign_f32(None, None, None, 10, 2, 2, 0, 0, 0, None, 0, None)
    assert rc == pkg.ERR_INVALID
    assert b"null" in L.bkm_last_error()
    cfg = pkg.Config(n=0, k=2, dim=2, layout=0, layout_means=0, device=0, variant_assign=0, variant_update=0, num_gpus=0)
    h = ctypes.c_void_p()
    assert L.bkm_create(ctypes.byref(cfg), ctypes.byref(h)) == pkg.ERR_INVALID
    cfg = pkg.Config(n=8, k=2, dim=2, layout=5, layout_means=0, device=0, variant_assign=0, variant_update=0, num_gpus=0)
    assert L.bkm_create(ctypes.byref(cfg), ctypes.byref(h)) == pkg.ERR_INVALID


def test_no_cpu_fallback_without_gpu(pkg):
    if pkg.device_count() > 0:
        pytest.skip("a GPU is present")
    km = pkg.KMeans()
    with pytest.raises(pkg.BkmError) as e:
        km.initialize(2, 2, 4, 1, np.zeros(8, np.float32), np.zeros(4, np.float32))
    assert e.value.code == pkg.ERR_CUDA
    with pytest.raises(pkg.BkmError):
        pkg.kmeans_host(np.zeros(8, np.float32), np.zeros(4, np.float32), 4, 2, 2, 1)


def test_run_before_initialize_is_a_state_error(pkg):
    km = pkg.KMeans()
    with pytest.raises(pkg.BkmError) as e:
        km.run()
    assert e.value.code == pkg.ERR_STATE


def test_unique_id_is_128_bytes(pkg):
    try:
        uid = pkg.comm_unique_id()
    except pkg.BkmError as e:
        assert e.code == pkg.ERR_NCCL
        pytest.skip("NCCL not present")
    assert len(uid) == 128 and any(uid)


def test_workloads_are_seeded_and_sliceable(workloads):
    a = workloads.generate_rows("mixture", 5000, 4, 16, seed=3, sigma=0.05, chunk=1024)
    b = workloads.generate_rows("mixture", 5000, 4, 16, seed=3, sigma=0.05, chunk=1024, begin=1500, count=2000)
    assert np.array_equal(a[1500:3500], b)
    c = workloads.generate_rows("uniform", 5000, 4, 16, seed=4, chunk=1024)
    assert not np.array_equal(a, c)
    s = workloads.generate_rows("sphere", 100, 64, 4, seed=1)
    assert np.allclose(np.linalg.norm(s, axis=1), 1.0, atol=1e-5)
    pts, means, spec = workloads.make("c1", n=4096)
    assert pts.size == 4096 * 4 and means.size == 16 * 4
    assert np.array_equal(workloads.from_layout(pts, 4096, 4, spec["layout"])[:16].reshape(-1), means)
