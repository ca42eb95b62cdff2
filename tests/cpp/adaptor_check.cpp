// Compile-and-run check of include/bkm_reference_adaptors.hpp against the reference's headers:
// the adaptors must be usable wherever the reference names a runner class or an IKMeansAlgorithm.
// Usage: adaptor_check [gpu]   - without "gpu" only the types are exercised (no device needed).
#include "bkm_reference_adaptors.hpp"
#include "serial.hpp"

#include <cstdio>
#include <cstring>
#include <memory>

template<class LAYOUT, class LAYOUT_MEANS>
int run_case(bool gpu)
{
	using METRIC = EuclideanMetricPolicy<float, LAYOUT, LAYOUT_MEANS>;
	// the runner signatures the reference's drivers call (headers/cuda.hpp:74-83, 181-182)
	void (*asg)(const AssignmentProblemInstance<float, std::uint32_t>&, CudaExecParameters&) =
		&B200AssignmentKernel<float, std::uint32_t, LAYOUT, LAYOUT_MEANS, METRIC>::run;
	void (*upd)(const UpdateProblemInstance<float, std::uint32_t>&, CudaExecParameters&) =
		&B200UpdateKernel<float, std::uint32_t, LAYOUT, LAYOUT_MEANS, false>::run;
	void (*fus)(const FusedProblemInstance<float, std::uint32_t>&, CudaExecParameters&) =
		&B200FusedKernel<float, std::uint32_t, LAYOUT, LAYOUT_MEANS, METRIC>::run;
	if (!asg || !upd || !fus) return 1;
	std::unique_ptr<IKMeansAlgorithm<float>> algo = std::make_unique<B200KMeansAlgorithm<float, std::uint32_t, LAYOUT, LAYOUT_MEANS>>(0);
	if (!gpu) return 0;

	const std::size_t n = 4096, k = 16, dim = 4, iters = 5;
	std::vector<float> data(LAYOUT::size(n, dim)), means(LAYOUT_MEANS::size(k, dim));
	unsigned s = 12345;
	for (std::size_t i = 0; i < n; ++i)
		for (std::size_t d = 0; d < dim; ++d) {
			s = s * 1664525u + 1013904223u;
			LAYOUT::at(data.data(), i, d, LAYOUT::precomputeConstants(n, dim)) = (s >> 8) * (1.0f / 16777216.0f);
		}
	for (std::size_t i = 0; i < k; ++i)
		for (std::size_t d = 0; d < dim; ++d)
			LAYOUT_MEANS::at(means.data(), i, d, LAYOUT_MEANS::precomputeConstants(k, dim)) =
				LAYOUT::at(data.data(), i, d, LAYOUT::precomputeConstants(n, dim));
	algo->initialize(dim, k, n, iters, data, means);
	algo->run();
	SerialKMeansAlgorithm<float, std::uint32_t, LAYOUT, LAYOUT_MEANS> serial;
	serial.initialize(dim, k, n, iters, data, means);
	serial.run();
	std::size_t diff = 0;
	for (std::size_t i = 0; i < n; ++i) diff += algo->getAssignment()[i] != serial.getAssignment()[i];
	double maxerr = 0;
	for (std::size_t i = 0; i < means.size(); ++i) {
		double e = std::abs((double)algo->getMeans()[i] - (double)serial.getMeans()[i]);
		if (e > maxerr) maxerr = e;
	}
	std::printf("assignment differences: %zu of %zu, max mean error %.3g\n", diff, n, maxerr);
	algo->cleanup();
	return (diff <= n / 1000 && maxerr < 1e-4) ? 0 : 2;
}

int main(int argc, char** argv)
{
	const bool gpu = argc > 1 && !std::strcmp(argv[1], "gpu");
	int rc = run_case<AoSLayoutPolicy<1>, AoSLayoutPolicy<1>>(gpu);
	rc |= run_case<SoALayoutPolicy<1>, SoALayoutPolicy<1>>(gpu);
	rc |= run_case<SoALayoutPolicy<1>, AoSLayoutPolicy<1>>(gpu);
	std::printf(rc == 0 ? "adaptor check ok\n" : "adaptor check FAILED\n");
	return rc;
}
