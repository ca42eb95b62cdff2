"""GPU (one device): the peer-memory exchange kernel - publish, bounded wait, rank-ordered sum,
divide - driven as ONE rank of a 3-rank job whose other two ranks are emulated by buffers that
this test fills beforehand (their sums, sizes and "published" flags come from the CPU oracle), so
no kernel ever waits for another kernel on the same GPU.  Checked against the oracle's update of
the whole data set (serial.hpp:44-73 restated): sizes exactly, means within 1e-4.  A second test
leaves one peer's flags unset and checks that the wait gives up after its limit with an error
status, without hanging, and that the handle works again afterwards."""
import time

import numpy as np
import pytest

from helpers import means_close

pytestmark = pytest.mark.gpu


def _peer_buffer(torch, pkg, k, d, sums, sizes, published):
    lay = pkg.peer_layout(k, d)
    buf = torch.zeros(lay["bytes"] // 4, dtype=torch.int32, device="cuda:0")
    if published:
        buf[:lay["flag_words"]] = 0x7FFFFFF0            # "has published every iteration so far"
    host = np.zeros(lay["bytes"] // 4, dtype=np.uint32)
    for slot in range(2):
        o = (lay["slot0_offset"] + slot * lay["slot_stride"]) // 4
        host[o:o + k * d] = np.ascontiguousarray(sums, dtype=np.float32).reshape(-1).view(np.uint32)
        host[o + k * d:o + k * d + k] = sizes.astype(np.uint32)
    body = torch.from_numpy(host[lay["flag_words"]:].view(np.int32)).to("cuda:0")
    buf[lay["flag_words"]:] = body
    return buf


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
    peers = []
    for r in range(world):
        b, c = shards[r]
        sums = np.zeros((k, d), dtype=np.float64)
        np.add.at(sums, asg[b:b + c], rows[b:b + c].astype(np.float64))
        peers.append(_peer_buffer(torch, pkg, k, d, sums.astype(np.float32), np.bincount(asg[b:b + c], minlength=k), True))
    b, c = shards[rank]
    km = pkg.KMeans(layout=layout, layout_means=layout_means)
    km.initialize(d, k, c, 1, workloads.to_layout(rows[b:b + c], layout), m0)
    bases = [p.data_ptr() for p in peers]
    bases[rank] = 0                                      # the handle uses its own buffer for its own rank
    km.peer_attach(bases, rank)
    km.peer_enable(True)
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
    silent = _peer_buffer(torch, pkg, k, d, np.zeros((k, d), np.float32), np.zeros(k, np.int64), False)
    km = pkg.KMeans(layout=0)
    km.initialize(d, k, n, 1, data, m0)
    km.set_option("exchange_wait_ms", 50)
    km.peer_attach([0, silent.data_ptr()], 0)
    km.peer_enable(True)
    t0 = time.perf_counter()
    with pytest.raises(pkg.BkmError) as e:
        km.run(1)
    assert e.value.code == pkg.ERR_DEVICE
    assert time.perf_counter() - t0 < 5.0                # the limit, not a hang
    # the peer "arrives": the same handle carries on
    lay = pkg.peer_layout(k, d)
    silent[:lay["flag_words"]] = 0x7FFFFFF0
    torch.cuda.synchronize()
    assert km.run_ready() == pkg.OK
    km.run(1)
    assert int(km.getSizes().astype(np.int64).sum()) == n
    km.cleanup()
