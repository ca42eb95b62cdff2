/*
 * The input data of the reference's two executables, reproduced call for call so that a run of the
 * harnesses here works on exactly the numbers a run of the reference executables with the same
 * --N --k --dim --seed --layout works on (same standard-library generator and distribution
 * objects, drawn in the same order).
 *
 *   k-means executable (experimental/k-means/k-means/headers/data.hpp of krulis-martin/cuda-kmeans):
 *     generate_clustered_data (:33-56): the first k points are uniform in [0,1)^dim and double as
 *       the cluster centres; every further point picks one of them uniformly and adds N(0, 0.025)
 *       noise per coordinate;
 *     prepare_means (:63-81) with shuffle on: a freshly seeded generator shuffles the n point
 *       indices, the first k of them name the initial means.
 *   bucketing executable (experimental/bucketing-cuda/bucketing-cuda/bucketing-cuda.cpp:172-173,
 *     generate_random, headers/data.hpp:19-26): uniform floats in [0,1) and uniform bucket indices,
 *     each from its own generator with the same seed.
 *
 * The outputs depend on the C++ standard library's distributions; with libstdc++ (what the
 * reference's Makefile builds with) they match the reference bit for bit - tests/golden holds
 * vectors taken from the reference's own code.
 */
#ifndef BKM_CLI_REFERENCE_DATA_HPP
#define BKM_CLI_REFERENCE_DATA_HPP

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <numeric>
#include <random>
#include <stdexcept>
#include <vector>

namespace refdata {

inline std::size_t at(bool soa, std::size_t item, std::size_t d, std::size_t items, std::size_t dim)
{
	return soa ? d * items + item : item * dim + d;
}

// F = float, or double for the reference's --double mode (the double-typed distributions consume
// the generator differently, so the two streams are unrelated).
template<typename F>
inline void clustered_points(std::vector<F>& data, std::size_t n, std::size_t k, std::size_t dim, std::size_t seed, bool soa)
{
	if (n < k) throw std::runtime_error("N must not be smaller than k (the first k points are the cluster centres)");
	std::mt19937 gen((unsigned int)seed);
	std::uniform_real_distribution<F> centre((F)0, (F)1);
	std::uniform_int_distribution<std::size_t> which(0, k - 1);
	std::normal_distribution<F> noise((F)0, (F)0.025);
	data.resize(n * dim);
	for (std::size_t i = 0; i < k; ++i)
		for (std::size_t d = 0; d < dim; ++d) data[at(soa, i, d, n, dim)] = centre(gen);
	for (std::size_t i = k; i < n; ++i) {
		const std::size_t c = which(gen);
		for (std::size_t d = 0; d < dim; ++d) {
			const F offset = noise(gen);
			data[at(soa, i, d, n, dim)] = offset + data[at(soa, c, d, n, dim)];
		}
	}
}

template<typename F>
inline void shuffled_means(const std::vector<F>& data, std::vector<F>& means, std::size_t n, std::size_t k, std::size_t dim,
	std::size_t seed, bool soa, bool soa_means)
{
	std::vector<std::uint32_t> order(n);
	std::iota(order.begin(), order.end(), 0u);
	std::mt19937 gen((unsigned int)seed);
	std::shuffle(order.begin(), order.end(), gen);
	means.resize(k * dim);
	for (std::size_t m = 0; m < k; ++m)
		for (std::size_t d = 0; d < dim; ++d) means[at(soa_means, m, d, k, dim)] = data[at(soa, order[m], d, n, dim)];
}

inline void bucketing_inputs(std::vector<float>& data, std::vector<std::uint32_t>& indices, std::uint32_t k, std::size_t seed)
{
	{
		std::mt19937 gen((unsigned int)seed);
		std::uniform_real_distribution<float> value(0.0f, 1.0f);
		for (float& x : data) x = value(gen);
	}
	{
		std::mt19937 gen((unsigned int)seed);
		std::uniform_int_distribution<std::uint32_t> bucket(0, k - 1);
		for (std::uint32_t& x : indices) x = bucket(gen);
	}
}

} // namespace refdata

#endif
