/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * CPU restatement, in plain C, of the serial Lloyd k-means of krulis-martin/cuda-kmeans.
 * It is the checker the GPU parity tests compare against, and the "port" CPU baseline of the
 * benchmark.  Nothing in the product path may call it.
 *
 * Parity pin: this file is checked bit-for-bit against the reference's own
 * SerialKMeansAlgorithm / SerialAssignmentAlgorithm (compiled from the reference headers by
 * oracle/build_oracle.py into oracle/_ref/) and against the golden vectors under tests/golden/
 * that were generated from that compiled reference (tests/golden/make_golden.py).
 *
 * Every function cites the reference lines (paths relative to
 * experimental/k-means/k-means/) whose arithmetic it restates.  The arithmetic order matters:
 * all sums are sequential in the dimension / point index, in float, with no fused
 * multiply-add (build with -ffp-contract=off and without -ffast-math).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define OKM_AOS 0
#define OKM_SOA 1

/* headers/layout_policies.hpp:22-25 (SoA: data[dim*stride+idx], stride = item count, ALIGN=1)
 * headers/layout_policies.hpp:46-49 (AoS: data[idx*stride+dim], stride = dims, ALIGN=1) */
static inline size_t okm_at(int layout, size_t idx, size_t dim, size_t items, size_t dims)
{
	return layout == OKM_SOA ? dim * items + idx : idx * dims + dim;
}

/* headers/metric_policies.hpp:20-29: sum over d of (a-b)^2, sequential, float. */
static inline float okm_dist_sq(const float *data, size_t i, int layout, size_t n,
	const float *means, size_t m, int layout_means, size_t k, size_t d)
{
	float sum = 0.0f;
	for (size_t j = 0; j < d; ++j) {
		float diff = data[okm_at(layout, i, j, n, d)] - means[okm_at(layout_means, m, j, k, d)];
		sum += diff * diff;
	}
	return sum;
}

/* headers/metric_policies.hpp:37-46: the default metric takes the square root. */
static inline float okm_dist(const float *data, size_t i, int layout, size_t n,
	const float *means, size_t m, int layout_means, size_t k, size_t d)
{
	return sqrtf(okm_dist_sq(data, i, layout, n, means, m, layout_means, k, d));
}

/* headers/serial.hpp:21-35 (findNearestMean): start from mean 0, replace only on a strictly
 * smaller distance, so the lowest index wins exact ties.  Points [begin,end) only, so callers
 * may split the range over threads; points are independent. */
void okm_assign_range_f32(const float *data, const float *means, uint32_t *assignment,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means, uint64_t begin, uint64_t end)
{
	for (uint64_t i = begin; i < end; ++i) {
		uint32_t nearest = 0;
		float min_dist = okm_dist(data, i, layout, n, means, 0, layout_means, k, d);
		for (uint32_t m = 1; m < k; ++m) {
			float dist = okm_dist(data, i, layout, n, means, m, layout_means, k, d);
			if (min_dist > dist) {
				min_dist = dist;
				nearest = m;
			}
		}
		assignment[i] = nearest;
	}
}

/* headers/serial.hpp:37-42 (computeAssignment). */
void okm_assign_f32(const float *data, const float *means, uint32_t *assignment,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means)
{
	okm_assign_range_f32(data, means, assignment, n, k, d, layout, layout_means, 0, n);
}

/* Best and second-best distance (as the reference metric computes them, square root taken)
 * for points [begin,end).  Used by the tests to decide whether a differing assignment is a
 * near-tie that the stated tolerance allows.  Same arithmetic as okm_assign_range_f32. */
void okm_best2_range_f32(const float *data, const float *means, float *best, float *second,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means, uint64_t begin, uint64_t end)
{
	for (uint64_t i = begin; i < end; ++i) {
		float b = INFINITY, s = INFINITY;
		for (uint32_t m = 0; m < k; ++m) {
			float dist = okm_dist(data, i, layout, n, means, m, layout_means, k, d);
			if (dist < b) { s = b; b = dist; }
			else if (dist < s) { s = dist; }
		}
		best[i] = b;
		second[i] = s;
	}
}

/* Distance of point i to one given mean (reference metric); lets a test evaluate the
 * distance to the cluster a GPU result picked. */
void okm_dist_to_f32(const float *data, const float *means, const uint32_t *which, float *out,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means, uint64_t begin, uint64_t end)
{
	for (uint64_t i = begin; i < end; ++i)
		out[i] = okm_dist(data, i, layout, n, means, which[i], layout_means, k, d);
}

/* headers/serial.hpp:44-73 (updateMeans): zero sums and sizes, accumulate in point order in
 * float, divide non-empty clusters; an empty cluster keeps the all-zero vector. */
void okm_update_f32(const float *data, const uint32_t *assignment, float *means, uint32_t *sizes,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means)
{
	for (uint32_t m = 0; m < k; ++m) {
		sizes[m] = 0;
		for (uint32_t j = 0; j < d; ++j) means[okm_at(layout_means, m, j, k, d)] = 0.0f;
	}
	for (uint64_t i = 0; i < n; ++i) {
		uint32_t target = assignment[i];
		++sizes[target];
		for (uint32_t j = 0; j < d; ++j)
			means[okm_at(layout_means, target, j, k, d)] += data[okm_at(layout, i, j, n, d)];
	}
	for (uint32_t m = 0; m < k; ++m) {
		if (sizes[m] == 0) continue;
		float divisor = (float)sizes[m];
		for (uint32_t j = 0; j < d; ++j) means[okm_at(layout_means, m, j, k, d)] /= divisor;
	}
}

/* Same update with double accumulation and a double divide: not the reference's arithmetic,
 * but the exact value both float implementations approximate.  Tests use it to arbitrate when
 * the float oracle itself has drifted on clusters with very many points. */
void okm_update_f64(const float *data, const uint32_t *assignment, double *means, uint32_t *sizes,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means)
{
	for (uint32_t m = 0; m < k; ++m) {
		sizes[m] = 0;
		for (uint32_t j = 0; j < d; ++j) means[okm_at(layout_means, m, j, k, d)] = 0.0;
	}
	for (uint64_t i = 0; i < n; ++i) {
		uint32_t target = assignment[i];
		++sizes[target];
		for (uint32_t j = 0; j < d; ++j)
			means[okm_at(layout_means, target, j, k, d)] += (double)data[okm_at(layout, i, j, n, d)];
	}
	for (uint32_t m = 0; m < k; ++m) {
		if (sizes[m] == 0) continue;
		for (uint32_t j = 0; j < d; ++j) means[okm_at(layout_means, m, j, k, d)] /= (double)sizes[m];
	}
}

/* headers/serial.hpp:89-96 (run): per iteration the current means become the previous means,
 * every point is assigned against them, then the means are recomputed.  `means` holds the
 * initial means on entry and the final means on return; `prev` is scratch of the same size.
 * `assignment` ends as the assignment of the last iteration (against the means before the
 * last update).  If `trace` is non-NULL it receives the means after every iteration
 * (iters * k*d floats). */
void okm_kmeans_f32(const float *data, float *means, float *prev, uint32_t *assignment,
	uint32_t *sizes, float *trace, uint64_t n, uint32_t k, uint32_t d, uint32_t iters,
	int layout, int layout_means)
{
	size_t kd = (size_t)k * d;
	for (uint32_t it = 0; it < iters; ++it) {
		memcpy(prev, means, kd * sizeof(float));
		okm_assign_f32(data, prev, assignment, n, k, d, layout, layout_means);
		okm_update_f32(data, assignment, means, sizes, n, k, d, layout, layout_means);
		if (trace) memcpy(trace + (size_t)it * kd, means, kd * sizeof(float));
	}
}

/* ---- the same algorithm with F = double (the reference executable's --double mode) ----------
 * headers/serial.hpp is a template on F; with F = double every sum, difference and square root
 * below is done in double (headers/metric_policies.hpp:50-64 for the metric). */

static inline double okm_dist_d(const double *data, size_t i, int layout, size_t n,
	const double *means, size_t m, int layout_means, size_t k, size_t d)
{
	double sum = 0.0;
	for (size_t j = 0; j < d; ++j) {
		double diff = data[okm_at(layout, i, j, n, d)] - means[okm_at(layout_means, m, j, k, d)];
		sum += diff * diff;
	}
	return sqrt(sum);
}

/* headers/serial.hpp:21-42 with F = double. */
void okm_assign_range_d(const double *data, const double *means, uint32_t *assignment,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means, uint64_t begin, uint64_t end)
{
	for (uint64_t i = begin; i < end; ++i) {
		uint32_t nearest = 0;
		double min_dist = okm_dist_d(data, i, layout, n, means, 0, layout_means, k, d);
		for (uint32_t m = 1; m < k; ++m) {
			double dist = okm_dist_d(data, i, layout, n, means, m, layout_means, k, d);
			if (min_dist > dist) {
				min_dist = dist;
				nearest = m;
			}
		}
		assignment[i] = nearest;
	}
}

/* headers/serial.hpp:44-73 with F = double. */
void okm_update_d(const double *data, const uint32_t *assignment, double *means, uint32_t *sizes,
	uint64_t n, uint32_t k, uint32_t d, int layout, int layout_means)
{
	for (uint32_t m = 0; m < k; ++m) {
		sizes[m] = 0;
		for (uint32_t j = 0; j < d; ++j) means[okm_at(layout_means, m, j, k, d)] = 0.0;
	}
	for (uint64_t i = 0; i < n; ++i) {
		uint32_t target = assignment[i];
		++sizes[target];
		for (uint32_t j = 0; j < d; ++j)
			means[okm_at(layout_means, target, j, k, d)] += data[okm_at(layout, i, j, n, d)];
	}
	for (uint32_t m = 0; m < k; ++m) {
		if (sizes[m] == 0) continue;
		double divisor = (double)sizes[m];
		for (uint32_t j = 0; j < d; ++j) means[okm_at(layout_means, m, j, k, d)] /= divisor;
	}
}

/* headers/serial.hpp:89-96 with F = double. */
void okm_kmeans_d(const double *data, double *means, double *prev, uint32_t *assignment,
	uint32_t *sizes, uint64_t n, uint32_t k, uint32_t d, uint32_t iters, int layout, int layout_means)
{
	size_t kd = (size_t)k * d;
	for (uint32_t it = 0; it < iters; ++it) {
		memcpy(prev, means, kd * sizeof(double));
		okm_assign_range_d(data, prev, assignment, n, k, d, layout, layout_means, 0, n);
		okm_update_d(data, assignment, means, sizes, n, k, d, layout, layout_means);
	}
}
