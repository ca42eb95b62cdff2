"""Comparison helpers shared by the GPU parity tests.

Tolerances (stated by the project's acceptance rule for this path):
  * assignments must equal the reference's except for points whose best and second-best
    reference distances differ by less than 1e-5 relative;
  * means must match within 1e-4 relative.
"""
import numpy as np

ASSIGN_TIE_RTOL = 1e-5
MEANS_RTOL = 1e-4


def assignment_mismatches(oracle, got, data, means, n, k, d, layout, layout_means, threads=8, sample=None):
    """Returns (exact_mismatches, disallowed_mismatches) of `got` against the oracle.

    A mismatch is allowed only when the point is a near-tie: the reference distance to the
    cluster the GPU picked is within ASSIGN_TIE_RTOL (relative) of the best distance."""
    if sample is None:
        want = oracle.assign(data, means, n, k, d, layout, layout_means, threads=threads)
        diff = np.nonzero(got != want)[0]
    else:
        raise NotImplementedError
    if diff.size == 0:
        return 0, 0
    best, _ = oracle.best2(data, means, n, k, d, layout, layout_means, threads=threads)
    picked = oracle.dist_to(data, means, got.astype(np.uint32), n, k, d, layout, layout_means, threads=threads)
    gap = (picked[diff] - best[diff]) / np.maximum(best[diff], 1e-30)
    bad = int((gap >= ASSIGN_TIE_RTOL).sum())
    return int(diff.size), bad


def means_close(got, want, rtol=MEANS_RTOL):
    """Element-wise |got-want| <= rtol * max(|want|, 1% of the largest magnitude)."""
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    scale = np.maximum(np.abs(want), 0.01 * max(np.abs(want).max(), 1e-30))
    err = np.abs(got - want) / scale
    return bool(np.all(err <= rtol)), float(err.max()) if err.size else 0.0


def rows_to_layout(rows, layout):
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    return rows.reshape(-1) if layout == 0 else np.ascontiguousarray(rows.T).reshape(-1)


class DeviceArrays:
    """Device buffers (torch tensors used as plain memory) for the kernel-runner entry points."""

    def __init__(self, torch, pkg, data, means, n, k, d):
        self.torch = torch
        dev = "cuda:0"
        self.points = torch.from_numpy(np.ascontiguousarray(data, dtype=np.float32)).to(dev)
        self.means = torch.from_numpy(np.ascontiguousarray(means, dtype=np.float32)).to(dev)
        self.assignment = torch.full((n,), 0xFFFFFFF, dtype=torch.int32, device=dev)
        self.means_out = torch.full((k * d,), float("nan"), dtype=torch.float32, device=dev)
        self.sizes = torch.full((k,), -1, dtype=torch.int32, device=dev)
        self.ws_bytes = pkg.workspace_bytes(n, k, d)
        assert self.ws_bytes > 0
        # uninitialised on purpose (filled with a pattern): the library must not rely on zeros
        self.workspace = torch.full((self.ws_bytes // 4 + 64,), 0x7FC12345, dtype=torch.int32, device=dev)
        base = self.workspace.data_ptr()
        self.ws_ptr = (base + 255) // 256 * 256
        self.ws_bytes_avail = self.workspace.numel() * 4 - (self.ws_ptr - base)
        assert self.ws_bytes_avail >= self.ws_bytes

    def asg_host(self):
        return self.assignment.cpu().numpy().view(np.uint32)
