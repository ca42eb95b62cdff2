// Compile-and-run check of include/bkm_reference_adaptors.hpp against the reference's headers:
// the adaptors must be usable wherever the reference names a runner class or an IKMeansAlgorithm.
// Usage: adaptor_check [gpu]   - without "gpu" only the types are exercised (no device needed).
//
// With "gpu" three things run, each compared with the reference's SerialKMeansAlgorithm in this
// process:
//   * B200KMeansAlgorithm through the IKMeansAlgorithm call sequence;
//   * B200AssignmentKernel::run + B200UpdateKernel::run driven the way CudaKMeansAlgorithm::run
//     drives its runners (headers/cuda.hpp:70-88 of the reference): buffers owned by the caller,
//     means and assignment double-buffered, the caller's zero-fill of means[next] and of the sizes
//     between the two runners, everything on the legacy default stream, one synchronisation at
//     the end;
//   * B200FusedKernel::run driven the way CudaFusedKMeansAlgorithm::run does (cuda.hpp:174-191).
#include "bkm_reference_adaptors.hpp"
#include "serial.hpp"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>

namespace {

template<class LAYOUT, class LAYOUT_MEANS>
void make_inputs(std::size_t n, std::size_t k, std::size_t dim, std::vector<float>& data, std::vector<float>& means)
{
	data.assign(LAYOUT::size(n, dim), 0.0f);
	means.assign(LAYOUT_MEANS::size(k, dim), 0.0f);
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
}

bool compare(const char* what, const std::vector<float>& got_means, const std::vector<float>& want_means,
	const std::vector<std::uint32_t>* got_asg, const std::vector<std::uint32_t>& want_asg)
{
	std::size_t diff = 0;
	if (got_asg) for (std::size_t i = 0; i < want_asg.size(); ++i) diff += (*got_asg)[i] != want_asg[i];
	double maxerr = 0;
	for (std::size_t i = 0; i < want_means.size(); ++i) {
		const double e = std::fabs((double)got_means[i] - (double)want_means[i]);
		if (!(e <= maxerr)) maxerr = e;      // a NaN counts as an error
	}
	std::printf("%s: assignment differences %zu of %zu, max mean error %.3g\n", what, diff, want_asg.size(), maxerr);
	return diff <= want_asg.size() / 1000 && maxerr < 1e-4;
}

void cuda_ok(cudaError_t e, const char* what)
{
	if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// The reference's combined driver loop with the B200 runners as ASGN_KERNEL / UPDATE_KERNEL.
template<class LAYOUT, class LAYOUT_MEANS>
bool runner_loop(std::size_t n, std::size_t k, std::size_t dim, std::size_t iters, bool fused)
{
	using METRIC = EuclideanMetricPolicy<float, LAYOUT, LAYOUT_MEANS>;
	using ASGN = B200AssignmentKernel<float, std::uint32_t, LAYOUT, LAYOUT_MEANS, METRIC>;
	using UPDATE = B200UpdateKernel<float, std::uint32_t, LAYOUT, LAYOUT_MEANS, false>;
	using FUSED = B200FusedKernel<float, std::uint32_t, LAYOUT, LAYOUT_MEANS, METRIC>;
	std::vector<float> data, means;
	make_inputs<LAYOUT, LAYOUT_MEANS>(n, k, dim, data, means);
	const std::size_t mfloats = LAYOUT_MEANS::size(k, dim);

	float *d_data = nullptr, *d_means[2] = {nullptr, nullptr};
	std::uint32_t *d_asg[2] = {nullptr, nullptr}, *d_sizes = nullptr;
	cuda_ok(cudaSetDevice(0), "cudaSetDevice");
	cuda_ok(cudaMalloc(&d_data, data.size() * sizeof(float)), "cudaMalloc");
	cuda_ok(cudaMalloc(&d_sizes, k * sizeof(std::uint32_t)), "cudaMalloc");
	for (int i = 0; i < 2; ++i) {
		cuda_ok(cudaMalloc(&d_means[i], mfloats * sizeof(float)), "cudaMalloc");
		cuda_ok(cudaMalloc(&d_asg[i], n * sizeof(std::uint32_t)), "cudaMalloc");
	}
	cuda_ok(cudaMemcpy(d_data, data.data(), data.size() * sizeof(float), cudaMemcpyHostToDevice), "copy");
	cuda_ok(cudaMemcpy(d_means[0], means.data(), mfloats * sizeof(float), cudaMemcpyHostToDevice), "copy");
	cuda_ok(cudaMemset(d_asg[0], 0, n * sizeof(std::uint32_t)), "memset");
	cuda_ok(cudaMemset(d_sizes, 0, k * sizeof(std::uint32_t)), "memset");
	cuda_ok(cudaDeviceSynchronize(), "sync");

	CudaExecParameters exec;
	std::size_t last = 0;
	for (std::size_t iter = 0; iter < iters; ++iter) {
		const std::size_t next = (last + 1) % 2;
		if (!fused) {
			AssignmentProblemInstance<float, std::uint32_t> assignment(d_data, d_means[last], d_asg[last], d_asg[next], dim, k, n);
			ASGN::run(assignment, exec);
			cuda_ok(cudaGetLastError(), "assignment runner");
			// the caller's zero-fill (the reference uses its fillZeros kernel on the same stream)
			cuda_ok(cudaMemsetAsync(d_means[next], 0, mfloats * sizeof(float), nullptr), "fill zeros");
			cuda_ok(cudaMemsetAsync(d_sizes, 0, k * sizeof(std::uint32_t), nullptr), "fill zeros");
			UpdateProblemInstance<float, std::uint32_t> update(d_data, d_asg[next], d_means[next], d_sizes, dim, k, n);
			UPDATE::run(update, exec);
			cuda_ok(cudaGetLastError(), "update runner");
		} else {
			cuda_ok(cudaMemsetAsync(d_means[next], 0, mfloats * sizeof(float), nullptr), "fill zeros");
			cuda_ok(cudaMemsetAsync(d_sizes, 0, k * sizeof(std::uint32_t), nullptr), "fill zeros");
			FusedProblemInstance<float, std::uint32_t> instance(d_data, d_means[last], d_means[next], d_sizes, dim, k, n);
			FUSED::run(instance, exec);
			cuda_ok(cudaGetLastError(), "fused runner");
		}
		last = next;
	}
	cuda_ok(cudaDeviceSynchronize(), "sync");
	std::vector<float> got_means(mfloats);
	std::vector<std::uint32_t> got_asg(n), got_sizes(k);
	cuda_ok(cudaMemcpy(got_means.data(), d_means[last], mfloats * sizeof(float), cudaMemcpyDeviceToHost), "copy back");
	cuda_ok(cudaMemcpy(got_asg.data(), d_asg[last], n * sizeof(std::uint32_t), cudaMemcpyDeviceToHost), "copy back");
	cuda_ok(cudaMemcpy(got_sizes.data(), d_sizes, k * sizeof(std::uint32_t), cudaMemcpyDeviceToHost), "copy back");
	cudaFree(d_data); cudaFree(d_sizes);
	for (int i = 0; i < 2; ++i) { cudaFree(d_means[i]); cudaFree(d_asg[i]); }

	SerialKMeansAlgorithm<float, std::uint32_t, LAYOUT, LAYOUT_MEANS> serial;
	serial.initialize(dim, k, n, iters, data, means);
	serial.run();
	std::size_t total = 0;
	for (std::size_t c = 0; c < k; ++c) total += got_sizes[c];
	char label[128];
	std::snprintf(label, sizeof(label), "%s runner loop n=%zu k=%zu dim=%zu", fused ? "fused" : "assignment+update", n, k, dim);
	bool ok = compare(label, got_means, serial.getMeans(), fused ? nullptr : &got_asg, serial.getAssignment());
	if (total != n) { std::printf("  cluster sizes add up to %zu, not %zu\n", total, n); ok = false; }
	return ok;
}

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
	std::vector<float> data, means;
	make_inputs<LAYOUT, LAYOUT_MEANS>(n, k, dim, data, means);
	algo->initialize(dim, k, n, iters, data, means);
	algo->run();
	SerialKMeansAlgorithm<float, std::uint32_t, LAYOUT, LAYOUT_MEANS> serial;
	serial.initialize(dim, k, n, iters, data, means);
	serial.run();
	bool ok = compare("B200KMeansAlgorithm", algo->getMeans(), serial.getMeans(), &algo->getAssignment(), serial.getAssignment());
	algo->cleanup();
	// the runners themselves: a CUDA-core shape and a tensor-core shape (dim 32, 512 means)
	ok = runner_loop<LAYOUT, LAYOUT_MEANS>(4096, 16, 4, 4, false) && ok;
	ok = runner_loop<LAYOUT, LAYOUT_MEANS>(4096, 16, 4, 4, true) && ok;
	ok = runner_loop<LAYOUT, LAYOUT_MEANS>(6000, 512, 32, 3, false) && ok;
	ok = runner_loop<LAYOUT, LAYOUT_MEANS>(6000, 512, 32, 3, true) && ok;
	return ok ? 0 : 2;
}

} // namespace

int main(int argc, char** argv)
{
	const bool gpu = argc > 1 && !std::strcmp(argv[1], "gpu");
	int rc = 0;
	try {
		rc = run_case<AoSLayoutPolicy<1>, AoSLayoutPolicy<1>>(gpu);
		rc |= run_case<SoALayoutPolicy<1>, SoALayoutPolicy<1>>(gpu);
		rc |= run_case<SoALayoutPolicy<1>, AoSLayoutPolicy<1>>(gpu);
	} catch (std::exception& e) {
		std::printf("exception: %s\n", e.what());
		rc = 3;
	}
	std::printf(rc == 0 ? "adaptor check ok\n" : "adaptor check FAILED\n");
	return rc;
}
