"""GPU (one device): the peer-memory exchange kernel - send tagged totals, bounded wait for every
sender's packets, rank-ordered sum, divide - driven as ONE rank of a 3-rank job whose other two
ranks are emulated: this test writes the packets they would have sent (sums and sizes from the CPU
oracle, tagged with the iteration count) into the handle's receive buffer beforehand, and gives
the handle scratch buffers to send into, so no kernel ever waits for another kernel on the same
GPU.  Checked against the oracle's update of the whole data set (serial.hpp:44-73 restated): sizes
exactly, means within 1e-4.  A second test leaves one sender's packets out and checks that the
wait gives up after its limit with an error status, without hanging, and that the handle works
again afterwards."""
import ctypes
import time

import numpy as np
import pytest

from helpers import means_close

pytestmark = pytest.mark.gpu


def _cudart():
    """The CUDA runtime PyTorch has loaded (for a copy to a raw device address)."""
    for name in ("libcudart.so.12", "libcudart.so"):
        try:
            return ctypes.CDLL(name)
        except OSError:
            continue
    pytest.skip("no libcudart to copy with")


def _deliver(torch, pkg, km, k, d, sender, sums, sizes, epoch):
    """Writes the packets rank `sender` sends in iteration `epoch` into km's receive buffer."""
    lay = pkg.peer_layout(k, d)
    base, nbytes = km.peer_buffer()
    assert nbytes == lay["bytes"]
    words = np.concatenate([np.ascontiguousarray(sums, dtype=np.float32).reshape(-1).view(np.uint32),
                            np.asarray(sizes).astype(np.uint32)]).astype(np.uint64)
    packets = words | (np.uint64(epoch) << np.uint64(32))
    dst = base + (epoch & 1) * lay["slot_bytes"] + sender * lay["packets_per_sender"] * 8
    src = torch.from_numpy(packets.view(np.int64)).to("cuda:0")
    rc = _cudart().cudaMemcpy(ctypes.c_void_p(dst), ctypes.c_void_p(src.data_ptr()), ctypes.c_size_t(packets.nbytes), 3)   # 3 = device to device
    assert int(rc) == 0
    torch.cuda.synchronize()


def _scratch(torch, pkg, k, d):
    return torch.zeros(pkg.peer_layout(k, d)["bytes"] // 8, dtype=torch.int64, device="cuda:0")


@pytest.mark.parametrize("n,k,d,layout,layout_means,name", [
    (30000, 1024, 32, 1, 1, "tensor cores, fused sums"),
    (20000, 16, 4, 0, 0, "CUDA cores"),
    (9001, 300, 20, 0, 1, "tensor cores, one CTA"),
])
def test_exchange_kernel_as_one_rank_of_three(pkg, torch_cuda, oracle_mod, workloads, n, k, d, layout, layout_means, name):
    torch = torch_cuda
    world, rank = 3, 1
    rows = workloads.generate_rows("mixture", n, d, 32, seed=21, sigma=0.08)
    means0 = np.ascontiguousarray(rows[:k])
    data = workloads.to_layout(rows, layout)
    m0 = workloads.to_layout(means0, layout_means)
    asg = oracle_mod.assign(data, m0, n, k, d, layout, layout_means, threads=8)
    shards = [pkg.shard_range(n, world, r) for r in range(world)]
    b, c = shards[rank]
    km = pkg.KMeans(layout=layout, layout_means=layout_means)
    km.initialize(d, k, c, 1, workloads.to_layout(rows[b:b + c], layout), m0)
    scratch = [_scratch(torch, pkg, k, d) for _ in range(world)]
    bases = [p.data_ptr() for p in scratch]
    bases[rank] = 0                                      # the handle uses its own buffer for its own rank
    km.peer_attach(bases, rank)
    km.peer_enable(True)
    for r in range(world):
        if r == rank:
            continue
        pb, pc = shards[r]
        sums = np.zeros((k, d), dtype=np.float64)
        np.add.at(sums, asg[pb:pb + pc], rows[pb:pb + pc].astype(np.float64))
        _deliver(torch, pkg, km, k, d, r, sums.astype(np.float32), np.bincount(asg[pb:pb + pc], minlength=k), 1)
    km.run(1)
    got_means, got_sizes, got_asg = km.getMeans(), km.getSizes(), km.getAssignment()
    km.cleanup()
    assert np.array_equal(got_asg, asg[b:b + c])
    want_means, want_sizes = oracle_mod.update(data, asg, n, k, d, layout, layout_means)
    assert np.array_equal(got_sizes, want_sizes), name
    ok, err = means_close(got_means, want_means)
    assert ok, (name, err)


def test_exchange_wait_gives_up_after_its_limit(pkg, torch_cuda, oracle_mod, workloads):
    torch = torch_cuda
    n, k, d = 5000, 16, 4
    rows = workloads.generate_rows("mixture", n, d, 16, seed=3, sigma=0.05)
    data, m0 = workloads.to_layout(rows, 0), workloads.to_layout(rows[:k], 0)
    km = pkg.KMeans(layout=0)
    km.initialize(d, k, n, 1, data, m0)
    km.set_option("exchange_wait_ms", 50)
    silent = _scratch(torch, pkg, k, d)
    km.peer_attach([0, silent.data_ptr()], 0)
    km.peer_enable(True)
    t0 = time.perf_counter()
    with pytest.raises(pkg.BkmError) as e:
        km.run(1)                                        # rank 1 never sends
    assert e.value.code == pkg.ERR_DEVICE
    assert time.perf_counter() - t0 < 5.0                # the limit, not a hang
    # the peer "arrives" for the next iteration: the same handle carries on
    assert km.run_ready() == pkg.OK
    _deliver(torch, pkg, km, k, d, 1, np.zeros((k, d), np.float32), np.zeros(k, np.int64), 2)
    km.run(1)
    assert int(km.getSizes().astype(np.int64).sum()) == n
    km.cleanup()
