// The fp64 counterpart of the iteration, for the reference executable's --double mode
// (k-means.cpp:313-315, 340-345 of krulis-martin/cuda-kmeans instantiate every algorithm for
// double as well).  fp64 is not the path this library is tuned for: one straightforward kernel per
// step, the reference's arithmetic in double - sequential subtract / multiply / add in dimension
// order without fusing, correctly rounded square root, strictly-smaller comparison in ascending
// index order (headers/serial.hpp:21-35, headers/metric_policies.hpp:50-64) - so the assignment is
// the serial algorithm's bit for bit for the same means; the sums are accumulated with double
// atomics (order differs from the serial loop: means agree to rounding, ~1e-15 relative).
#include "../../include/bkm.h"
#include "common.cuh"

#include <algorithm>
#include <cmath>

int bkm_internal_fail(int code, const char* fmt, ...);

namespace bkm {

// One warp per point, lanes over the means; the point's coordinates in shared memory.
template<bool SOA, bool SOAM>
__global__ void __launch_bounds__(256) assign_exact_f64_kernel(const double* __restrict__ pts, const double* __restrict__ means,
	uint32_t* __restrict__ asg, uint64_t n, uint32_t k, uint32_t d)
{
	extern __shared__ double sx64[];
	const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
	double* x = sx64 + (size_t)warp * d;
	for (uint64_t i = (uint64_t)blockIdx.x * wpb + warp; i < n; i += (uint64_t)gridDim.x * wpb) {
		__syncwarp();
		for (uint32_t j = lane; j < d; j += 32) x[j] = pts[at<SOA>(i, j, n, d)];
		__syncwarp();
		double best = INFINITY;
		uint32_t bidx = 0xffffffffu;
		for (uint32_t m = lane; m < k; m += 32) {
			double sum = 0.0;
			for (uint32_t j = 0; j < d; ++j) {
				const double diff = __dsub_rn(x[j], means[at<SOAM>(m, j, k, d)]);
				sum = __dadd_rn(sum, __dmul_rn(diff, diff));
			}
			const double dist = __dsqrt_rn(sum);
			if (dist < best || bidx == 0xffffffffu) { best = dist; bidx = m; }
		}
		// lowest (distance, index) pair over the warp = what the sequential scan keeps
		#pragma unroll
		for (int off = 16; off > 0; off >>= 1) {
			const double ob = __shfl_xor_sync(0xffffffffu, best, off);
			const uint32_t oi = __shfl_xor_sync(0xffffffffu, bidx, off);
			if (oi != 0xffffffffu && (bidx == 0xffffffffu || ob < best || (ob == best && oi < bidx))) { best = ob; bidx = oi; }
		}
		if (lane == 0) asg[i] = bidx;
	}
}

// sums[c][:] += x_i, sizes[c] += 1 (both zero on entry); one thread per coordinate.
template<bool SOA, bool SOAM>
__global__ void __launch_bounds__(256) update_f64_kernel(const double* __restrict__ pts, const uint32_t* __restrict__ asg,
	double* __restrict__ sums, uint32_t* __restrict__ sizes, uint64_t n, uint32_t k, uint32_t d)
{
	const uint64_t total = n * d;
	for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (uint64_t)gridDim.x * blockDim.x) {
		// walk the points array in memory order
		const uint64_t i = SOA ? e % n : e / d;
		const uint32_t j = (uint32_t)(SOA ? e / n : e % d);
		const uint32_t c = asg[i];
		if (c >= k) continue;
		atomicAdd(&sums[at<SOAM>(c, j, k, d)], pts[e]);
		if (j == 0) atomicAdd(&sizes[c], 1u);
	}
}

template<bool SOAM>
__global__ void __launch_bounds__(256) divide_f64_kernel(double* __restrict__ sums, const uint32_t* __restrict__ sizes, uint32_t k, uint32_t d)
{
	const size_t kd = (size_t)k * d;
	for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < kd; e += (size_t)gridDim.x * blockDim.x) {
		const uint32_t c = (uint32_t)(SOAM ? e % k : e / d);
		if (sizes[c]) sums[e] = __ddiv_rn(sums[e], (double)sizes[c]);     // an empty cluster keeps its zeros
	}
}

} // namespace bkm

#define F64_TRY(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) { rc = bkm_internal_fail(BKM_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); goto done; } } while (0)

extern "C" int bkm_kmeans_host_f64(const double* host_points, double* means, uint32_t* assignment,
	uint64_t n, uint32_t k, uint32_t dim, uint32_t iters, int layout, int layout_means, int device)
{
	if (!host_points || !means || !assignment) return bkm_internal_fail(BKM_ERR_INVALID, "null argument");
	if (n == 0 || k == 0 || dim == 0 || iters == 0) return bkm_internal_fail(BKM_ERR_INVALID, "n, k, dim and iters must be positive");
	if (n >= (1ull << 32)) return bkm_internal_fail(BKM_ERR_UNSUPPORTED, "at most 2^32-1 points");
	if ((layout != BKM_LAYOUT_AOS && layout != BKM_LAYOUT_SOA) || (layout_means != BKM_LAYOUT_AOS && layout_means != BKM_LAYOUT_SOA))
		return bkm_internal_fail(BKM_ERR_INVALID, "unknown layout code");
	if ((size_t)dim * sizeof(double) * 8 > 96 * 1024) return bkm_internal_fail(BKM_ERR_UNSUPPORTED, "dim too large for the fp64 path (%u)", dim);
	int rc = BKM_OK, sms = 0;
	double *d_pts = nullptr, *d_means[2] = {nullptr, nullptr};
	uint32_t *d_asg = nullptr, *d_sizes = nullptr;
	const size_t kd = (size_t)k * dim, nd = (size_t)n * dim;
	const bool soa = layout == BKM_LAYOUT_SOA, soam = layout_means == BKM_LAYOUT_SOA;
	{
		F64_TRY(cudaSetDevice(device));
		F64_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
		F64_TRY(cudaMalloc(&d_pts, nd * sizeof(double)));
		F64_TRY(cudaMalloc(&d_means[0], kd * sizeof(double)));
		F64_TRY(cudaMalloc(&d_means[1], kd * sizeof(double)));
		F64_TRY(cudaMalloc(&d_asg, n * sizeof(uint32_t)));
		F64_TRY(cudaMalloc(&d_sizes, (size_t)k * sizeof(uint32_t)));
		F64_TRY(cudaMemcpy(d_pts, host_points, nd * sizeof(double), cudaMemcpyHostToDevice));
		F64_TRY(cudaMemcpy(d_means[0], means, kd * sizeof(double), cudaMemcpyHostToDevice));
		const size_t smem = (size_t)8 * dim * sizeof(double);
		const uint32_t grid_a = (uint32_t)std::min<uint64_t>((n + 7) / 8, (uint64_t)sms * 16);
		const uint32_t grid_u = (uint32_t)std::min<uint64_t>((nd + 255) / 256, (uint64_t)sms * 16);
		const uint32_t grid_d = (uint32_t)std::min<uint64_t>((kd + 255) / 256, (uint64_t)sms * 8);
		int cur = 0;
		for (uint32_t it = 0; it < iters; ++it) {
			const int next = cur ^ 1;
#define F64_LAUNCH(SOA, SOAM) do { \
				auto ka = bkm::assign_exact_f64_kernel<SOA, SOAM>; \
				if (smem > 48 * 1024) F64_TRY(cudaFuncSetAttribute(ka, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
				ka<<<grid_a, 256, smem>>>(d_pts, d_means[cur], d_asg, n, k, dim); \
				F64_TRY(cudaMemsetAsync(d_means[next], 0, kd * sizeof(double))); \
				F64_TRY(cudaMemsetAsync(d_sizes, 0, (size_t)k * sizeof(uint32_t))); \
				bkm::update_f64_kernel<SOA, SOAM><<<grid_u, 256>>>(d_pts, d_asg, d_means[next], d_sizes, n, k, dim); \
				bkm::divide_f64_kernel<SOAM><<<grid_d, 256>>>(d_means[next], d_sizes, k, dim); \
			} while (0)
			if (soa && soam) F64_LAUNCH(true, true);
			else if (soa) F64_LAUNCH(true, false);
			else if (soam) F64_LAUNCH(false, true);
			else F64_LAUNCH(false, false);
#undef F64_LAUNCH
			F64_TRY(cudaGetLastError());
			cur = next;
		}
		F64_TRY(cudaDeviceSynchronize());
		F64_TRY(cudaMemcpy(means, d_means[cur], kd * sizeof(double), cudaMemcpyDeviceToHost));
		F64_TRY(cudaMemcpy(assignment, d_asg, n * sizeof(uint32_t), cudaMemcpyDeviceToHost));
	}
done:
	cudaFree(d_pts); cudaFree(d_means[0]); cudaFree(d_means[1]); cudaFree(d_asg); cudaFree(d_sizes);
	return rc;
}
