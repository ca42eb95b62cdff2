/*
 * TEST INFRASTRUCTURE - not part of the shipped library.
 *
 * C entry points around the reference project's own input generator: generate_clustered_data
 * and prepare_means of headers/data.hpp (:33-56, :63-81), compiled from where the reference
 * checkout lies (include path given by oracle/build_oracle.py; oracle/bpp_stub supplies the one
 * bpplib header data.hpp asks for).  The result, oracle/_ref/libkmrefdata.so, produced the
 * fixture tests/golden/refdata_golden.npz, which pins the restatement of that generator in
 * cuda-kmeans_b200/cli/reference_data.hpp.
 *
 * Layout codes: 0 = AoSLayoutPolicy<1>, 1 = SoALayoutPolicy<1>.
 */
#include "data.hpp"

#include <cstdint>
#include <cstring>
#include <vector>

namespace {

template<class LAYOUT, class LAYOUT_MEANS>
int make(std::size_t n, std::size_t k, std::size_t dim, std::size_t seed, float* dataOut, float* meansOut)
{
	std::vector<float> data, means;
	generate_clustered_data<float, LAYOUT>(data, n, k, dim, seed);
	prepare_means<float, std::uint32_t, LAYOUT, LAYOUT_MEANS>(data, means, n, k, dim, true, seed);
	std::memcpy(dataOut, data.data(), sizeof(float) * LAYOUT::size(n, dim));
	std::memcpy(meansOut, means.data(), sizeof(float) * LAYOUT_MEANS::size(k, dim));
	return 0;
}

} // namespace

/* The inputs the reference's k-means executable builds for (--N n --k k --dim dim --seed seed) in the
 * given layouts (k-means.cpp:205-210): data, then k shuffled data points as initial means. */
extern "C" int ref_make_inputs_f32(int layout, int layoutMeans, std::uint64_t n, std::uint64_t k, std::uint64_t dim,
	std::uint64_t seed, float* dataOut, float* meansOut)
{
	try {
		if (layout == 0 && layoutMeans == 0) return make<AoSLayoutPolicy<1>, AoSLayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
		if (layout == 0 && layoutMeans == 1) return make<AoSLayoutPolicy<1>, SoALayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
		if (layout == 1 && layoutMeans == 0) return make<SoALayoutPolicy<1>, AoSLayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
		if (layout == 1 && layoutMeans == 1) return make<SoALayoutPolicy<1>, SoALayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
	} catch (...) {
		return 2;
	}
	return 1;
}

/* The same with --double: generate_clustered_data<double> and prepare_means<double> draw from
 * double-typed distributions, which consume the generator differently. */
template<class LAYOUT, class LAYOUT_MEANS>
static int make_double(std::size_t n, std::size_t k, std::size_t dim, std::size_t seed, double* dataOut, double* meansOut)
{
	std::vector<double> data, means;
	generate_clustered_data<double, LAYOUT>(data, n, k, dim, seed);
	prepare_means<double, std::uint32_t, LAYOUT, LAYOUT_MEANS>(data, means, n, k, dim, true, seed);
	std::memcpy(dataOut, data.data(), sizeof(double) * LAYOUT::size(n, dim));
	std::memcpy(meansOut, means.data(), sizeof(double) * LAYOUT_MEANS::size(k, dim));
	return 0;
}

extern "C" int ref_make_inputs_f64(int layout, int layoutMeans, std::uint64_t n, std::uint64_t k, std::uint64_t dim,
	std::uint64_t seed, double* dataOut, double* meansOut)
{
	try {
		if (layout == 0 && layoutMeans == 0) return make_double<AoSLayoutPolicy<1>, AoSLayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
		if (layout == 0 && layoutMeans == 1) return make_double<AoSLayoutPolicy<1>, SoALayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
		if (layout == 1 && layoutMeans == 0) return make_double<SoALayoutPolicy<1>, AoSLayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
		if (layout == 1 && layoutMeans == 1) return make_double<SoALayoutPolicy<1>, SoALayoutPolicy<1>>(n, k, dim, seed, dataOut, meansOut);
	} catch (...) {
		return 2;
	}
	return 1;
}

/* The inputs of the reference's bucketing executable (bucketing-cuda.cpp:172-173): `count` uniform
 * floats in [0,1) and `count_idx` uniform indices in [0,k), each from its own generator seeded alike. */
extern "C" int ref_make_bucketing_inputs_f32(std::uint64_t count, std::uint64_t countIdx, std::uint32_t k, std::uint64_t seed,
	float* dataOut, std::uint32_t* indicesOut)
{
	try {
		std::vector<float> data(count);
		std::vector<std::uint32_t> indices(countIdx);
		generate_random(data, std::uniform_real_distribution<float>(0.0f, 1.0f), seed);
		generate_random(indices, std::uniform_int_distribution<std::uint32_t>(0, k - 1), seed);
		std::memcpy(dataOut, data.data(), sizeof(float) * count);
		std::memcpy(indicesOut, indices.data(), sizeof(std::uint32_t) * countIdx);
	} catch (...) {
		return 2;
	}
	return 0;
}
