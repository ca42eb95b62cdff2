"""CPU, world_size 2 over gloo: the host-side pieces of the multi-GPU path.

What runs here without a GPU: the shard arithmetic of the C ABI, the hand-over of the NCCL
unique id from rank 0 to the other ranks through the launcher's process group (the way
bench.py bootstraps the library's communicator), and the exchange protocol itself - per-rank
partial sums and sizes, all-reduced, then divided - emulated with the oracle as the per-shard
compute and checked against the unsharded oracle."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    import oracle
    pkg = entry.load()
    import importlib
    wl = importlib.import_module("cuda_kmeans_b200.workloads")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # 1. unique id travels from rank 0 to everyone
        uid = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(pkg.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        gathered = [torch.zeros(128, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(gathered, uid)
        assert all(torch.equal(g, gathered[0]) for g in gathered) and int(uid.sum()) > 0

        # 2. sharded iteration protocol on a seeded workload, SoA points, 3 iterations
        n_total, k, d, layout = 5003, 12, 6, 1
        begin, count = pkg.shard_range(n_total, world, rank)
        rows = wl.generate_rows("mixture", n_total, d, k, seed=9, sigma=0.05, chunk=512, begin=begin, count=count)
        first = wl.generate_rows("mixture", n_total, d, k, seed=9, sigma=0.05, chunk=512, begin=0, count=k)
        shard = wl.to_layout(rows, layout)
        means = wl.to_layout(first, 0)
        for _ in range(3):
            asg = oracle.assign(shard, means, count, k, d, layout, 0)
            sums = np.zeros((k, d), dtype=np.float32)
            np.add.at(sums, asg, rows)
            sizes = np.bincount(asg, minlength=k).astype(np.int64)
            t_sums, t_sizes = torch.from_numpy(sums), torch.from_numpy(sizes)
            dist.all_reduce(t_sums)
            dist.all_reduce(t_sizes)
            new = np.zeros((k, d), dtype=np.float32)
            nz = sizes_np = t_sizes.numpy()
            nz = sizes_np > 0
            new[nz] = t_sums.numpy()[nz] / sizes_np[nz, None].astype(np.float32)
            means = new.reshape(-1)
        np.save(os.path.join(out_dir, "means_%d.npy" % rank), means)
        np.save(os.path.join(out_dir, "asg_%d.npy" % rank), asg)
    finally:
        dist.destroy_process_group()


def _agree_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        entered = []
        # step 1: every rank is ready -> all enter the collective step
        if pkg.agree(dist, torch, pkg.OK) == pkg.OK:
            entered.append(1)
            t = torch.ones(1)
            dist.all_reduce(t)
        # step 2: rank 1's set-up failed (its local code is an error) -> NO rank may enter
        local = pkg.ERR_CUDA if rank == 1 else pkg.OK
        verdict = pkg.agree(dist, torch, local)
        if verdict == pkg.OK:
            entered.append(2)
        # a handle that was never initialised reports "not ready" without raising
        km = pkg.KMeans()
        assert km.run_ready() == pkg.ERR_STATE
        with open(os.path.join(out_dir, "agree_%d.txt" % rank), "w") as f:
            f.write("%s %d" % (",".join(map(str, entered)), verdict))
    finally:
        dist.destroy_process_group()


def test_failing_rank_keeps_every_rank_out_of_the_collective(tmp_path, pkg):
    """Host-side agreement before a step that would strand the peers of a failed rank: the ranks
    reduce their readiness codes over the launcher's process group; one error code makes every
    rank skip the step."""
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mp.spawn(_agree_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        entered, verdict = open(tmp_path / ("agree_%d.txt" % rank)).read().split()
        assert entered == "1"                            # step 1 entered, step 2 entered by nobody
        assert int(verdict) == pkg.ERR_CUDA              # every rank learned of the failure


def test_peer_exchange_layout(pkg):
    lay = pkg.peer_layout(1024, 32)
    words = 1024 * 32 + 1024
    assert lay["senders"] == 8 and lay["packets_per_sender"] >= words and lay["packets_per_sender"] % 64 == 0
    assert lay["slot_bytes"] == lay["senders"] * lay["packets_per_sender"] * 8
    assert lay["bytes"] == 2 * lay["slot_bytes"]


def test_two_rank_protocol_matches_unsharded_oracle(tmp_path, pkg, workloads, oracle_mod):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    n_total, k, d, layout = 5003, 12, 6, 1
    rows = workloads.generate_rows("mixture", n_total, d, k, seed=9, sigma=0.05, chunk=512)
    want_means, want_asg = oracle_mod.kmeans(workloads.to_layout(rows, layout), rows[:k].reshape(-1),
                                             n_total, k, d, 3, layout, 0)
    m0 = np.load(tmp_path / "means_0.npy")
    m1 = np.load(tmp_path / "means_1.npy")
    assert np.array_equal(m0, m1)                      # every rank ends with identical means
    assert np.allclose(m0, want_means, rtol=1e-4, atol=1e-6)
    asg = np.concatenate([np.load(tmp_path / "asg_0.npy"), np.load(tmp_path / "asg_1.npy")])
    assert (asg != want_asg).mean() <= 1e-3            # shards concatenate to the global assignment


def test_shards_of_soa_points_are_column_slices(pkg, workloads):
    n_total, d = 1000, 3
    rows = workloads.generate_rows("uniform", n_total, d, 4, seed=1, chunk=128)
    full = workloads.to_layout(rows, 1).reshape(d, n_total)
    for world in (2, 3):
        for rank in range(world):
            b, c = pkg.shard_range(n_total, world, rank)
            part = workloads.generate_rows("uniform", n_total, d, 4, seed=1, chunk=128, begin=b, count=c)
            assert np.array_equal(workloads.to_layout(part, 1).reshape(d, c), full[:, b:b + c])
