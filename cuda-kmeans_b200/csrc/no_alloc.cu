// bkm_update_noalloc_f32: the update step for callers that cannot hand over (or allocate) device
// scratch.  Its accumulators live in a fixed array that is part of the loaded library image on
// every GPU, so the call itself reserves nothing.
#include "../../include/bkm.h"
#include "kernels.cuh"

#include <mutex>
#include <string>

namespace {

// 2 MiB of device memory per GPU that loads the library, held until the process exits.
// Word 0.. : the Control block (64 words reserved); the accumulator replicas follow.
constexpr size_t NOALLOC_WORDS = BKM_NOALLOC_SCRATCH_WORDS;
constexpr size_t NOALLOC_HEADER_WORDS = 64;
static __device__ __align__(256) uint32_t g_noalloc_scratch[NOALLOC_WORDS];

constexpr int MAX_DEVICES = 64;
std::mutex g_setup_mutex;
uint32_t* g_scratch_ptr[MAX_DEVICES] = {};   // device address of the array, per device ordinal

} // namespace

// defined in api.cu
int bkm_internal_fail(int code, const char* fmt, ...);

// Device address of the built-in array on `device` (looked up once per device, with that device
// current: the array's name is only a host-side handle, the kernels need the address the runtime
// resolves it to on this device).
static int scratch_base(int device, uint32_t** base)
{
	if (device < 0 || device >= MAX_DEVICES) return bkm_internal_fail(BKM_ERR_UNSUPPORTED, "device ordinal %d out of range", device);
	std::lock_guard<std::mutex> lock(g_setup_mutex);
	if (!g_scratch_ptr[device]) {
		void* p = nullptr;
		const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
		if (e != cudaSuccess || !p) return bkm_internal_fail(BKM_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
		g_scratch_ptr[device] = static_cast<uint32_t*>(p);
	}
	*base = g_scratch_ptr[device];
	return BKM_OK;
}

extern "C" int bkm_update_noalloc_f32(const float* points, const uint32_t* assignment, float* means, uint32_t* sizes,
	uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means, void* stream)
{
	if (!points || !assignment || !means || !sizes) return bkm_internal_fail(BKM_ERR_INVALID, "null pointer argument");
	if (n == 0 || k == 0 || dim == 0) return bkm_internal_fail(BKM_ERR_INVALID, "n, k and dim must be positive");
	if (n >= (1ull << 32)) return bkm_internal_fail(BKM_ERR_UNSUPPORTED, "at most 2^32-1 points per call");
	if ((layout != BKM_LAYOUT_AOS && layout != BKM_LAYOUT_SOA) || (layout_means != BKM_LAYOUT_AOS && layout_means != BKM_LAYOUT_SOA))
		return bkm_internal_fail(BKM_ERR_INVALID, "unknown layout code");
	const uint64_t need = (uint64_t)k * dim + k;
	if (need > BKM_NOALLOC_MAX_WORDS)
		return bkm_internal_fail(BKM_ERR_UNSUPPORTED,
			"k*dim + k = %llu exceeds the built-in scratch of %llu values; use bkm_update_f32 with a workspace",
			(unsigned long long)need, (unsigned long long)BKM_NOALLOC_MAX_WORDS);

	int device = 0;
	cudaError_t e = cudaGetDevice(&device);
	if (e != cudaSuccess) return bkm_internal_fail(BKM_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
	uint32_t* base = nullptr;
	const int rc = scratch_base(device, &base);
	if (rc != BKM_OK) return rc;
	int sm_count = 0;
	e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
	if (e != cudaSuccess) return bkm_internal_fail(BKM_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));

	bkm::Shape s;
	s.n = n; s.k = k; s.dim = dim; s.soa = layout == BKM_LAYOUT_SOA; s.soa_means = layout_means == BKM_LAYOUT_SOA;
	const size_t stride = bkm::acc_replica_stride(k, dim);
	uint32_t replicas = bkm::acc_replicas(k, dim);
	const size_t room = (NOALLOC_WORDS - NOALLOC_HEADER_WORDS) / stride;
	if (room < 1) return bkm_internal_fail(BKM_ERR_UNSUPPORTED, "k*dim + k does not fit the built-in scratch");
	if (replicas > room) replicas = (uint32_t)room;

	bkm::Control* ctl = reinterpret_cast<bkm::Control*>(base);
	float* acc = reinterpret_cast<float*>(base + NOALLOC_HEADER_WORDS);
	uint32_t* counts = base + NOALLOC_HEADER_WORDS + (size_t)k * dim;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	// the array keeps whatever the previous call left: everything that is accumulated into starts from zero
	e = cudaMemsetAsync(base, 0, (NOALLOC_HEADER_WORDS + (size_t)replicas * stride) * sizeof(uint32_t), st);
	if (e != cudaSuccess) return bkm_internal_fail(BKM_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
	int variant = BKM_UPDATE_GLOBAL;
	if (dim >= 16) variant = BKM_UPDATE_ROWS;
	else if (bkm::update_shared_fits(s, device)) variant = BKM_UPDATE_SHARED;
	bkm::launch_update(points, assignment, acc, counts, replicas, s, variant, ctl, sm_count, st);
	bkm::launch_finalize(acc, counts, replicas, means, sizes, s, nullptr, nullptr, ctl, 1, st);
	e = cudaGetLastError();
	if (e != cudaSuccess) return bkm_internal_fail(BKM_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
	return BKM_OK;
}

// Reads the status word the kernels of the last bkm_update_noalloc_f32 call on the current device
// left at the head of the built-in array (after waiting for `stream`).
extern "C" int bkm_noalloc_check(void* stream)
{
	int device = 0;
	cudaError_t e = cudaGetDevice(&device);
	if (e != cudaSuccess) return bkm_internal_fail(BKM_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
	uint32_t* base = nullptr;
	const int rc = scratch_base(device, &base);
	if (rc != BKM_OK) return rc;
	bkm::Control c;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	e = cudaMemcpyAsync(&c, base, sizeof(c), cudaMemcpyDeviceToHost, st);
	if (e == cudaSuccess) e = cudaStreamSynchronize(st);
	if (e != cudaSuccess) return bkm_internal_fail(BKM_ERR_CUDA, "reading the status word: %s", cudaGetErrorString(e));
	if (c.status) return bkm_internal_fail(BKM_ERR_DEVICE, "kernel status 0x%x (2=assignment out of range)", c.status);
	return BKM_OK;
}
