/*
 * bkm_reference_adaptors.hpp - the B200 kernels behind the reference's own plug-in interface.
 *
 * Include this header from a translation unit of krulis-martin/cuda-kmeans (it includes the
 * reference's headers/kernels.cuh, headers/layout_policies.hpp, headers/metric_policies.hpp and
 * headers/interface.hpp by name, so the reference's header directory must be on the include
 * path) and link libbkm.so.  It provides
 *
 *   B200AssignmentKernel<F, IDX_T, LAYOUT, LAYOUT_MEANS, METRIC>::run(const AssignmentProblemInstance&, CudaExecParameters&)
 *   B200UpdateKernel<F, IDX_T, LAYOUT, LAYOUT_MEANS, EMUL>::run(const UpdateProblemInstance&, CudaExecParameters&)
 *   B200FusedKernel<F, IDX_T, LAYOUT, LAYOUT_MEANS, METRIC>::run(const FusedProblemInstance&, CudaExecParameters&)
 *
 * with exactly the signatures the reference declares for its runners (headers/kernels.cuh:81-116),
 * so that they can be named as ASGN_KERNEL / UPDATE_KERNEL / KERNEL template arguments of
 * CudaKMeansAlgorithm / CudaFusedKMeansAlgorithm / CudaAssignmentAlgorithm (headers/cuda.hpp:15-19,
 * 115-119, 236-240), and B200KMeansAlgorithm, an IKMeansAlgorithm (headers/interface.hpp:8-49)
 * over the library's own driver.
 *
 * Supported: F = float, IDX_T = std::uint32_t, layouts with ALIGN = 1, the Euclidean and the
 * squared-Euclidean metric policy (same arg-min).  Anything else throws std::runtime_error, the
 * reference's convention for unsupported shapes (kernels/kernels.cu:281-282, 666-667).
 * Like the reference's runners, everything is launched on the legacy default stream.
 */
#ifndef BKM_REFERENCE_ADAPTORS_HPP
#define BKM_REFERENCE_ADAPTORS_HPP

#include "kernels.cuh"
#include "layout_policies.hpp"
#include "metric_policies.hpp"
#include "interface.hpp"

#include "bkm.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

namespace bkm_adaptor {

template<class LAYOUT> struct layout_code;
template<> struct layout_code<AoSLayoutPolicy<1>> { static constexpr int value = BKM_LAYOUT_AOS; };
template<> struct layout_code<SoALayoutPolicy<1>> { static constexpr int value = BKM_LAYOUT_SOA; };

inline void check(int rc)
{
	if (rc != BKM_OK) throw std::runtime_error(std::string("libbkm: ") + bkm_last_error());
}

template<typename F, typename IDX_T>
inline void require_types()
{
	static_assert(std::is_same<F, float>::value, "the B200 kernels are fp32 only");
	static_assert(std::is_same<IDX_T, std::uint32_t>::value, "the B200 kernels use 32-bit cluster indices");
}

/*
 * The reference's problem instances carry no scratch pointer (headers/kernels.cuh:8-52), so the
 * adaptors keep one grow-only device workspace per host thread.  It is allocated on first use
 * and when a larger problem arrives - outside the steady state of the iteration loop.
 */
class Workspace {
public:
	static Workspace& instance()
	{
		static thread_local Workspace ws;
		return ws;
	}

	void* get(std::uint64_t n, std::uint32_t k, std::uint32_t dim, std::size_t& bytes)
	{
		bytes = bkm_workspace_bytes(n, k, dim);
		if (bytes == 0) throw std::runtime_error("libbkm: problem size not supported");
		if (bytes > mBytes) {
			if (mPtr) cudaFree(mPtr);
			mPtr = nullptr;
			mBytes = 0;
			if (cudaMalloc(&mPtr, bytes) != cudaSuccess) throw std::runtime_error("libbkm: cannot allocate the workspace");
			mBytes = bytes;
		}
		bytes = mBytes;
		return mPtr;
	}

	~Workspace() { if (mPtr) cudaFree(mPtr); }

private:
	void* mPtr = nullptr;
	std::size_t mBytes = 0;
};

} // namespace bkm_adaptor


/* Drop-in for the ASGN_KERNEL parameter (replaces e.g. BestCachedAssignmentKernel, kernels/kernels.cu:706-717). */
template<typename F, typename IDX_T, class LAYOUT, class LAYOUT_MEANS, class METRIC>
class B200AssignmentKernel {
public:
	static void run(const AssignmentProblemInstance<F, IDX_T>& in, CudaExecParameters& /*exec*/)
	{
		bkm_adaptor::require_types<F, IDX_T>();
		std::size_t bytes = 0;
		void* ws = bkm_adaptor::Workspace::instance().get(in.n, in.k, in.dim, bytes);
		bkm_adaptor::check(bkm_assign_f32(in.data, in.means, in.assignment, in.n, in.k, in.dim,
			bkm_adaptor::layout_code<LAYOUT>::value, bkm_adaptor::layout_code<LAYOUT_MEANS>::value,
			BKM_ASSIGN_AUTO, ws, bytes, nullptr));
	}
};


/* Drop-in for the UPDATE_KERNEL parameter (replaces e.g. UpdateAtomicShmKernel, kernels/kernels.cu:861-878).
 * On return (stream-ordered) in.means holds the divided means and in.clusterSizes the sizes. */
template<typename F, typename IDX_T, class LAYOUT, class LAYOUT_MEANS, int EMUL = false>
class B200UpdateKernel {
public:
	static void run(const UpdateProblemInstance<F, IDX_T>& in, CudaExecParameters& /*exec*/)
	{
		bkm_adaptor::require_types<F, IDX_T>();
		std::size_t bytes = 0;
		void* ws = bkm_adaptor::Workspace::instance().get(in.n, in.k, in.dim, bytes);
		bkm_adaptor::check(bkm_update_f32(in.data, in.assignment, in.means, in.clusterSizes, in.n, in.k, in.dim,
			bkm_adaptor::layout_code<LAYOUT>::value, bkm_adaptor::layout_code<LAYOUT_MEANS>::value,
			BKM_UPDATE_AUTO, ws, bytes, nullptr));
	}
};


/* Drop-in for the KERNEL parameter of CudaFusedKMeansAlgorithm (replaces FusedCachedRegsKernel,
 * kernels/kernels.cu:1146-1190): meansOut and clusterSizes from meansIn, no assignment output. */
template<typename F, typename IDX_T, class LAYOUT, class LAYOUT_MEANS, class METRIC>
class B200FusedKernel {
public:
	static void run(const FusedProblemInstance<F, IDX_T>& in, CudaExecParameters& /*exec*/)
	{
		bkm_adaptor::require_types<F, IDX_T>();
		std::size_t bytes = 0;
		void* ws = bkm_adaptor::Workspace::instance().get(in.n, in.k, in.dim, bytes);
		bkm_adaptor::check(bkm_iterate_f32(in.data, in.meansIn, in.meansOut, in.clusterSizes, nullptr, in.n, in.k, in.dim,
			bkm_adaptor::layout_code<LAYOUT>::value, bkm_adaptor::layout_code<LAYOUT_MEANS>::value,
			BKM_ASSIGN_AUTO, BKM_UPDATE_AUTO, ws, bytes, nullptr));
	}
};


/* The whole algorithm behind IKMeansAlgorithm, over the library's own driver (the counterpart of
 * CudaKMeansAlgorithm, headers/cuda.hpp:19-112, without bpplib). */
template<typename F = float, typename IDX_T = std::uint32_t, class LAYOUT = AoSLayoutPolicy<1>, class LAYOUT_MEANS = LAYOUT>
class B200KMeansAlgorithm : public IKMeansAlgorithm<F, IDX_T>
{
private:
	bkm_handle_t mHandle = nullptr;
	bool mResultReady = false;

	void fetchResult()
	{
		if (mResultReady) return;
		this->mMeans.resize(LAYOUT_MEANS::size(this->mK, this->mDim));
		this->mAssignment.resize(this->mN);
		bkm_adaptor::check(bkm_get_means(mHandle, this->mMeans.data()));
		bkm_adaptor::check(bkm_get_assignment(mHandle, this->mAssignment.data()));
		mResultReady = true;
	}

public:
	/* gpus > 1: the points are sharded over GPUs device .. device+gpus-1 of this process (bkm_config_t::num_gpus) */
	explicit B200KMeansAlgorithm(int device = 0, int gpus = 1) : mDevice(device), mGpus(gpus) {}
	~B200KMeansAlgorithm() override { if (mHandle) bkm_destroy(mHandle); }

	void initialize(std::size_t dim, std::size_t k, std::size_t n, std::size_t iters,
		const std::vector<F>& data, const std::vector<F>& means) override
	{
		bkm_adaptor::require_types<F, IDX_T>();
		IKMeansAlgorithm<F, IDX_T>::initialize(dim, k, n, iters, data, means);
		mResultReady = false;
		if (mHandle) { bkm_destroy(mHandle); mHandle = nullptr; }
		bkm_config_t cfg{};
		cfg.n = n; cfg.k = (std::uint32_t)k; cfg.dim = (std::uint32_t)dim;
		cfg.layout = bkm_adaptor::layout_code<LAYOUT>::value;
		cfg.layout_means = bkm_adaptor::layout_code<LAYOUT_MEANS>::value;
		cfg.device = mDevice;
		cfg.num_gpus = mGpus;
		bkm_adaptor::check(bkm_create(&cfg, &mHandle));
		bkm_adaptor::check(bkm_initialize(mHandle, data.data(), means.data()));
	}

	void run() override
	{
		mResultReady = false;
		bkm_adaptor::check(bkm_run(mHandle, (std::uint32_t)this->mIters));
	}

	const std::vector<F>& getMeans() override { fetchResult(); return this->mMeans; }
	const std::vector<IDX_T>& getAssignment() override { fetchResult(); return this->mAssignment; }

	void cleanup() override
	{
		IKMeansAlgorithm<F, IDX_T>::cleanup();
		if (mHandle) { bkm_destroy(mHandle); mHandle = nullptr; }
	}

private:
	int mDevice;
	int mGpus;
};

#endif /* BKM_REFERENCE_ADAPTORS_HPP */
