// Shared definitions of the k-means kernels: status word, layout indexing, launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <cstddef>

namespace bkm {

// Bits of the device status word.  Kernels never trap; a bounded wait that runs out or an
// internal inconsistency sets a bit here and the host turns it into BKM_ERR_DEVICE.
enum : uint32_t {
	STATUS_WAIT_TIMEOUT = 1u,   // an mbarrier / flag wait hit its iteration limit
	STATUS_BAD_INDEX = 2u,      // an assignment >= k was seen by the update
	STATUS_LIST_OVERFLOW = 4u,  // the near-tie list was too short (cannot happen when sized n)
};

// Device-resident control block shared by the kernels of one handle / one stateless call.
struct Control {
	uint32_t status;       // STATUS_* bits
	uint32_t flag_count;   // number of points queued for the exact re-check
	float cmax2[2];        // max over clusters of |mean|^2; the preparation of iteration t
	                       // writes slot (t+1)&1 with atomicMax and clears slot t&1
	uint32_t last_flag_count; // flag_count of the last finished iteration (for reporting)
	float xmax2;           // max over the points of |x|^2 (written by the one-off split of the points)
	uint32_t pad[2];
};

// What a stateless workspace remembers about the point set its one-off operands (centre vector,
// largest norm, tf32 planes) were derived from; it lives at byte 64 of the workspace.  `valid` is
// rewritten by every call: 1 when the points of this call are the remembered ones.
struct PointsKey {
	unsigned long long fp_new;   // fingerprint of the points of the current call (accumulated, then compared)
	unsigned long long fp_old;   // fingerprint the operands in the workspace belong to
	unsigned long long ptr, n;
	uint32_t dim, layout, variant, valid;
};
constexpr size_t POINTS_KEY_OFFSET = 64;

// Element offset of (item, dim) in a buffer of `items` vectors of `dims` floats.
// AoS: item*dims + dim, SoA: dim*items + item (the reference's layout policies, ALIGN = 1).
template<bool SOA>
__host__ __device__ __forceinline__ size_t at(size_t item, size_t dim, size_t items, size_t dims)
{
	return SOA ? dim * items + item : item * dims + dim;
}

__host__ __device__ __forceinline__ size_t at_rt(int soa, size_t item, size_t dim, size_t items, size_t dims)
{
	return soa ? dim * items + item : item * dims + dim;
}

__host__ __device__ __forceinline__ uint32_t round_up(uint32_t x, uint32_t m) { return (x + m - 1) / m * m; }
__host__ __device__ __forceinline__ uint64_t round_up64(uint64_t x, uint64_t m) { return (x + m - 1) / m * m; }

// Row stride (floats) of the prepared means used by the CUDA-core assignment:
// [ |c - centre|^2, -2(c_0 - centre_0) ... -2(c_{d-1} - centre_{d-1}), 0-padding ] rounded to a
// multiple of 4 floats; a padding row holds +inf in its first slot (and zeros).
__host__ __device__ __forceinline__ uint32_t simt_row_stride(uint32_t dim) { return round_up(dim + 1, 4); }

// Rows of the prepared means: k rounded to the 32-mean chunk the kernel walks.
__host__ __device__ __forceinline__ uint32_t simt_rows(uint32_t k) { return round_up(k, 32); }

// Geometry of the tensor-core operands: K (dimension) padded to 32 floats (one 128-byte
// swizzle row), point rows padded to 128, mean rows padded to 16.
constexpr uint32_t TC_KCHUNK = 32;
constexpr uint32_t TC_MTILE = 128;
// dim <= 16 uses rows of 16 floats (64-byte swizzle): half the operand bytes of a 32-float row
__host__ __device__ __forceinline__ uint32_t tc_dpad(uint32_t dim) { return dim <= 16 ? 16u : round_up(dim, TC_KCHUNK); }

// The per-iteration accumulators (k*dim float sums directly followed by k integer sizes) exist in
// `acc_replicas` copies so that concurrent global reductions spread over more cache lines; a
// copy starts every acc_replica_stride 32-bit words.
__host__ __device__ __forceinline__ size_t acc_replica_stride(uint32_t k, uint32_t dim)
{
	return ((size_t)k * dim + k + 63) / 64 * 64;
}
__host__ __device__ __forceinline__ uint32_t acc_replicas(uint32_t k, uint32_t dim)
{
	const size_t lines = ((size_t)k * dim + 31) / 32;
	size_t r = (16384 + lines - 1) / lines;
	return (uint32_t)(r < 1 ? 1 : (r > 16 ? 16 : r));
}

// The |c|^2 operand of the tensor-core assignment is one K step (8 tf32) wide and stored
// K-major without swizzle: 8-row x 16-byte core matrices, the two 16-byte chunks of a row group
// 128 B apart, row groups 256 B apart.  Float offset of element (row, k):
__host__ __device__ __forceinline__ uint32_t aug_offset(uint32_t row, uint32_t k)
{
	return (row >> 3) * 64 + (k >> 2) * 32 + (row & 7) * 4 + (k & 3);
}

} // namespace bkm
