"""GPU, 2 ranks (needs two devices): the sharded driver - contiguous point shards, the sums and
sizes of every iteration exchanged inside libbkm, by NCCL all-reduce or by the peer-memory
exchange kernel - against the single-GPU run and the oracle."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir, name, n_total, iters, mode):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load()
    import importlib
    wl = importlib.import_module("cuda_kmeans_b200.workloads")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = dict(wl.CONFIGS[name])
        k, d, lay = spec["k"], spec["dim"], spec["layout"]
        begin, count = pkg.shard_range(n_total, world, rank)
        rows = wl.generate_rows(spec["kind"], n_total, d, k, 5, spec.get("sigma", 0.05), spec.get("zipf"),
                                begin=begin, count=count, chunk=4096)
        first = wl.generate_rows(spec["kind"], n_total, d, k, 5, spec.get("sigma", 0.05), spec.get("zipf"),
                                 begin=0, count=k, chunk=4096)
        km = pkg.KMeans(layout=lay, device=rank)
        km.initialize(d, k, count, iters, wl.to_layout(rows, lay), wl.to_layout(first, lay))
        uid = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(pkg.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        km.comm_init(uid.numpy().tobytes(), world, rank)
        if mode == "peer":
            assert km.peer_exchange_init(dist, torch, device="cpu")
        assert pkg.agree(dist, torch, km.run_ready()) == pkg.OK
        km.run()
        np.save(os.path.join(out_dir, "means_%d.npy" % rank), km.getMeans())
        np.save(os.path.join(out_dir, "asg_%d.npy" % rank), km.getAssignment())
        np.save(os.path.join(out_dir, "sizes_%d.npy" % rank), km.getSizes())
        km.cleanup()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name,n_total,iters,mode", [("c1", 50001, 4, "nccl"), ("c2", 40000, 3, "nccl"),
                                                     ("c1", 50001, 4, "peer"), ("c2", 40000, 3, "peer")])
def test_two_ranks_match_single_gpu_and_oracle(tmp_path, pkg, torch_cuda, workloads, oracle_mod, name, n_total, iters, mode):
    if torch_cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), name, n_total, iters, mode), nprocs=world, join=True)
    spec = dict(workloads.CONFIGS[name])
    k, d, lay = spec["k"], spec["dim"], spec["layout"]
    rows = workloads.generate_rows(spec["kind"], n_total, d, k, 5, spec.get("sigma", 0.05), spec.get("zipf"), chunk=4096)
    data, means0 = workloads.to_layout(rows, lay), workloads.to_layout(rows[:k], lay)
    m0, m1 = np.load(tmp_path / "means_0.npy"), np.load(tmp_path / "means_1.npy")
    assert np.array_equal(m0, m1)                                 # identical means on every rank
    assert np.array_equal(np.load(tmp_path / "sizes_0.npy"), np.load(tmp_path / "sizes_1.npy"))
    asg = np.concatenate([np.load(tmp_path / "asg_0.npy"), np.load(tmp_path / "asg_1.npy")])
    # single GPU, same data
    km = pkg.KMeans(layout=lay)
    km.initialize(d, k, n_total, iters, data, means0)
    km.run()
    single_means, single_asg = km.getMeans(), km.getAssignment()
    km.cleanup()
    from helpers import means_close
    ok, err = means_close(m0, single_means)
    assert ok, err
    assert (asg != single_asg).mean() <= 1e-3
    # the oracle
    want_means, want_asg = oracle_mod.kmeans(data, means0, n_total, k, d, iters, lay, lay)
    ok, err = means_close(m0, want_means)
    assert ok, err
    assert (asg != want_asg).mean() <= 1e-3
    assert int(np.load(tmp_path / "sizes_0.npy").astype(np.int64).sum()) == n_total


@pytest.mark.parametrize("name,n_total,iters,gpus", [("c1", 50001, 4, 2), ("c2", 40000, 3, 2), ("c5", 30011, 3, 2)])
def test_one_process_driving_several_gpus(pkg, torch_cuda, workloads, oracle_mod, name, n_total, iters, gpus):
    """bkm_config_t::num_gpus: one handle, the points sharded over the GPUs of this process, sums and
    sizes exchanged through peer memory - against the single-GPU run and, step by step, the oracle."""
    if torch_cuda.cuda.device_count() < gpus:
        pytest.skip("needs %d GPUs" % gpus)
    from helpers import means_close
    spec = dict(workloads.CONFIGS[name])
    k, d, lay = spec["k"], spec["dim"], spec["layout"]
    rows = workloads.generate_rows(spec["kind"], n_total, d, k, 5, spec.get("sigma", 0.05), spec.get("zipf"), chunk=4096)
    data, means0 = workloads.to_layout(rows, lay), workloads.to_layout(rows[:k], lay)
    km = pkg.KMeans(layout=lay, num_gpus=gpus)
    km.initialize(d, k, n_total, iters, data, means0)
    prev = means0.copy()
    for it in range(iters):
        km.run(1)
        asg, cur, sizes = km.getAssignment(), km.getMeans(), km.getSizes()
        want = oracle_mod.assign(data, prev, n_total, k, d, lay, lay, threads=8)
        assert np.array_equal(asg, want), (it, int((asg != want).sum()))
        want_means, want_sizes = oracle_mod.update(data, asg, n_total, k, d, lay, lay)
        assert np.array_equal(sizes, want_sizes), it
        ok, err = means_close(cur, want_means)
        assert ok, (it, err)
        prev = cur
    assert km.iterations_done() == iters
    km.cleanup()
    single = pkg.KMeans(layout=lay)
    single.initialize(d, k, n_total, iters, data, means0)
    single.run(iters)
    ok, err = means_close(prev, single.getMeans())
    assert ok, err
    single.cleanup()
