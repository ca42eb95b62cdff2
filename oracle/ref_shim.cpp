/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * C entry points around the reference project's own serial k-means.  This translation unit
 * only #includes the reference headers (headers/serial.hpp and what it pulls in) from where
 * the reference checkout lies; the include path is given on the compiler command line by
 * oracle/build_oracle.py, and no reference source is copied here.  The result,
 * oracle/_ref/libkmref.so, pins oracle/kmeans_oracle.c and serves as the "reference" CPU
 * baseline of the benchmark.
 *
 * Layout codes: 0 = AoSLayoutPolicy<1>, 1 = SoALayoutPolicy<1> (headers/layout_policies.hpp).
 * The metric is the reference default, EuclideanMetricPolicy (headers/metric_policies.hpp:34-47).
 */
#include "serial.hpp"

#include <cstdint>
#include <cstring>
#include <vector>

namespace {

template<class LAYOUT, class LAYOUT_MEANS>
int kmeans(std::size_t dim, std::size_t k, std::size_t n, std::size_t iters, const float* data,
	const float* means, float* meansOut, std::uint32_t* assignmentOut)
{
	std::vector<float> vData(data, data + LAYOUT::size(n, dim));
	std::vector<float> vMeans(means, means + LAYOUT_MEANS::size(k, dim));
	SerialKMeansAlgorithm<float, std::uint32_t, LAYOUT, LAYOUT_MEANS> algorithm;
	algorithm.initialize(dim, k, n, iters, vData, vMeans);
	algorithm.run();
	std::memcpy(meansOut, algorithm.getMeans().data(), sizeof(float) * LAYOUT_MEANS::size(k, dim));
	std::memcpy(assignmentOut, algorithm.getAssignment().data(), sizeof(std::uint32_t) * n);
	algorithm.cleanup();
	return 0;
}

template<class LAYOUT, class LAYOUT_MEANS>
int assign(std::size_t dim, std::size_t k, std::size_t n, const float* data, const float* means,
	std::uint32_t* assignmentOut)
{
	std::vector<float> vData(data, data + LAYOUT::size(n, dim));
	std::vector<float> vMeans(means, means + LAYOUT_MEANS::size(k, dim));
	SerialAssignmentAlgorithm<float, std::uint32_t, LAYOUT, LAYOUT_MEANS> algorithm;
	algorithm.initialize(dim, k, n, vData, vMeans);
	algorithm.run();
	std::memcpy(assignmentOut, algorithm.getAssignment().data(), sizeof(std::uint32_t) * n);
	algorithm.cleanup();
	return 0;
}

template<class LAYOUT, class LAYOUT_MEANS>
int kmeans_double(std::size_t dim, std::size_t k, std::size_t n, std::size_t iters, const double* data,
	const double* means, double* meansOut, std::uint32_t* assignmentOut)
{
	std::vector<double> vData(data, data + LAYOUT::size(n, dim));
	std::vector<double> vMeans(means, means + LAYOUT_MEANS::size(k, dim));
	SerialKMeansAlgorithm<double, std::uint32_t, LAYOUT, LAYOUT_MEANS> algorithm;
	algorithm.initialize(dim, k, n, iters, vData, vMeans);
	algorithm.run();
	std::memcpy(meansOut, algorithm.getMeans().data(), sizeof(double) * LAYOUT_MEANS::size(k, dim));
	std::memcpy(assignmentOut, algorithm.getAssignment().data(), sizeof(std::uint32_t) * n);
	algorithm.cleanup();
	return 0;
}

} // namespace

extern "C" {

/* SerialKMeansAlgorithm<double, ...>: what the reference executable runs with --double. */
int ref_kmeans_f64(int layout, int layoutMeans, std::uint64_t dim, std::uint64_t k, std::uint64_t n,
	std::uint64_t iters, const double* data, const double* means, double* meansOut, std::uint32_t* assignmentOut)
{
	using A = AoSLayoutPolicy<1>;
	using S = SoALayoutPolicy<1>;
	if (layout == 0 && layoutMeans == 0) return kmeans_double<A, A>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	if (layout == 1 && layoutMeans == 1) return kmeans_double<S, S>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	if (layout == 0 && layoutMeans == 1) return kmeans_double<A, S>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	if (layout == 1 && layoutMeans == 0) return kmeans_double<S, A>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	return 1;
}

int ref_kmeans_f32(int layout, int layoutMeans, std::uint64_t dim, std::uint64_t k, std::uint64_t n,
	std::uint64_t iters, const float* data, const float* means, float* meansOut, std::uint32_t* assignmentOut)
{
	using A = AoSLayoutPolicy<1>;
	using S = SoALayoutPolicy<1>;
	if (layout == 0 && layoutMeans == 0) return kmeans<A, A>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	if (layout == 1 && layoutMeans == 1) return kmeans<S, S>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	if (layout == 0 && layoutMeans == 1) return kmeans<A, S>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	if (layout == 1 && layoutMeans == 0) return kmeans<S, A>(dim, k, n, iters, data, means, meansOut, assignmentOut);
	return 1;
}

int ref_assign_f32(int layout, int layoutMeans, std::uint64_t dim, std::uint64_t k, std::uint64_t n,
	const float* data, const float* means, std::uint32_t* assignmentOut)
{
	using A = AoSLayoutPolicy<1>;
	using S = SoALayoutPolicy<1>;
	if (layout == 0 && layoutMeans == 0) return assign<A, A>(dim, k, n, data, means, assignmentOut);
	if (layout == 1 && layoutMeans == 1) return assign<S, S>(dim, k, n, data, means, assignmentOut);
	if (layout == 0 && layoutMeans == 1) return assign<A, S>(dim, k, n, data, means, assignmentOut);
	if (layout == 1 && layoutMeans == 0) return assign<S, A>(dim, k, n, data, means, assignmentOut);
	return 1;
}

} // extern "C"
