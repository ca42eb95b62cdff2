// Host side of libbkm.so: the C ABI declared in include/bkm.h, the fixed-iteration driver and
// the NCCL exchange of the per-iteration sums and sizes.  Mirrors the call sequence of the
// reference's CudaKMeansAlgorithm (headers/cuda.hpp:45-112 of krulis-martin/cuda-kmeans):
// initialize copies data and means to the device, run loops assignment -> update with the
// means double-buffered, results are fetched afterwards.
#include "../../include/bkm.h"
#include "kernels.cuh"

#include <dlfcn.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

namespace {

thread_local std::string g_error;

int fail(int code, const char* fmt, ...)
{
	char buf[512];
	va_list ap;
	va_start(ap, fmt);
	vsnprintf(buf, sizeof(buf), fmt, ap);
	va_end(ap);
	g_error = buf;
	return code;
}

} // namespace

// Same as fail() for the other translation units of the library.
int bkm_internal_fail(int code, const char* fmt, ...)
{
	char buf[512];
	va_list ap;
	va_start(ap, fmt);
	vsnprintf(buf, sizeof(buf), fmt, ap);
	va_end(ap);
	g_error = buf;
	return code;
}

namespace {

#define CUDA_TRY(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) \
	return fail(BKM_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); } while (0)

bool layout_ok(int l) { return l == BKM_LAYOUT_AOS || l == BKM_LAYOUT_SOA; }

// ---- NCCL, resolved at run time so that the library loads on machines without it ----------

typedef struct { char internal[128]; } nccl_unique_id;
struct Nccl {
	void* lib = nullptr;
	int (*GetUniqueId)(nccl_unique_id*) = nullptr;
	int (*CommInitRank)(void**, int, nccl_unique_id, int) = nullptr;
	int (*CommDestroy)(void*) = nullptr;
	int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
	int (*GroupStart)() = nullptr;
	int (*GroupEnd)() = nullptr;
	const char* (*GetErrorString)(int) = nullptr;
	bool ok = false;
};
constexpr int NCCL_UINT32 = 3, NCCL_FLOAT32 = 7, NCCL_SUM = 0;

Nccl* nccl()
{
	static Nccl inst;
	static bool tried = false;
	if (!tried) {
		tried = true;
		// RTLD_NOLOAD first: reuse the copy a host application (e.g. PyTorch) already loaded, so
		// that one process never holds two NCCL versions under the same soname.  Otherwise the
		// file named by BKM_NCCL_LIBRARY, then the system default.
		void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
		const char* named = getenv("BKM_NCCL_LIBRARY");
		if (!lib && named && *named) lib = dlopen(named, RTLD_NOW | RTLD_LOCAL);
		if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
		if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
		if (lib) {
			inst.lib = lib;
			inst.GetUniqueId = reinterpret_cast<decltype(inst.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
			inst.CommInitRank = reinterpret_cast<decltype(inst.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
			inst.CommDestroy = reinterpret_cast<decltype(inst.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
			inst.AllReduce = reinterpret_cast<decltype(inst.AllReduce)>(dlsym(lib, "ncclAllReduce"));
			inst.GroupStart = reinterpret_cast<decltype(inst.GroupStart)>(dlsym(lib, "ncclGroupStart"));
			inst.GroupEnd = reinterpret_cast<decltype(inst.GroupEnd)>(dlsym(lib, "ncclGroupEnd"));
			inst.GetErrorString = reinterpret_cast<decltype(inst.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
			inst.ok = inst.GetUniqueId && inst.CommInitRank && inst.CommDestroy && inst.AllReduce &&
				inst.GroupStart && inst.GroupEnd && inst.GetErrorString;
		}
	}
	return &inst;
}

#define NCCL_TRY(expr) do { int r_ = (expr); if (r_ != 0) \
	return fail(BKM_ERR_NCCL, "%s failed: %s", #expr, nccl()->GetErrorString(r_)); } while (0)

// ---- workspace carving ----------------------------------------------------------------------

struct Workspace {
	bkm::Control* ctl = nullptr;
	void* split_scratch = nullptr; // re-check kernel: partial results of blocks that share a group (kept zeroed)
	float* acc = nullptr;          // k*dim sums (replica 0; further replicas acc_replica_stride words apart)
	uint32_t* counts = nullptr;    // k sizes (directly behind the sums of each replica)
	uint32_t replicas = 1;
	size_t acc_bytes = 0;
	bkm::SimtMeans sm{};           // CUDA-core rows (+ the centre vector, shared with the tensor-core operands)
	size_t cprep_bytes = 0;
	bkm::TcMeans tm{};
	size_t tm_bytes = 0;           // b_hi + b_lo
	uint32_t* flag_list = nullptr; // n entries
	uint32_t* asg_scratch = nullptr; // n entries (iterate without an assignment output)
	bkm::TcPoints tp{};
	size_t bytes = 0;
};

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// Lays the workspace out behind `base` (may be null: only the size is computed).
Workspace carve(char* base, uint64_t n, uint32_t k, uint32_t dim, bool with_tc_points)
{
	Workspace w;
	size_t off = 0;
	auto take = [&](size_t bytes) -> char* {
		char* p = base ? base + off : nullptr;
		off += align256(bytes);
		return p;
	};
	w.ctl = reinterpret_cast<bkm::Control*>(take(sizeof(bkm::Control)));
	w.split_scratch = take(bkm::list_split_scratch_bytes());
	const size_t kd = (size_t)k * dim;
	w.replicas = bkm::acc_replicas(k, dim);
	w.acc_bytes = (size_t)w.replicas * bkm::acc_replica_stride(k, dim) * sizeof(float);
	char* accp = take(w.acc_bytes);
	w.acc = reinterpret_cast<float*>(accp);
	w.counts = accp ? reinterpret_cast<uint32_t*>(accp + kd * sizeof(float)) : nullptr;
	w.cprep_bytes = (size_t)bkm::simt_rows(k) * bkm::simt_row_stride(dim) * sizeof(float);
	w.sm.rows = reinterpret_cast<float*>(take(w.cprep_bytes));
	w.tm.k_pad = bkm::tc_kpad(k);
	w.tm.d_pad = bkm::tc_dpad(dim);
	const size_t plane = (size_t)w.tm.k_pad * w.tm.d_pad * sizeof(float);
	w.tm_bytes = 2 * align256(plane);
	w.tm.b_hi = reinterpret_cast<float*>(take(plane));
	w.tm.b_lo = reinterpret_cast<float*>(take(plane));
	w.tm.cnorm = reinterpret_cast<float*>(take((size_t)w.tm.k_pad * sizeof(float)));
	w.tm.b_aug = reinterpret_cast<float*>(take((size_t)w.tm.k_pad * 8 * sizeof(float)));
	w.tm.center = reinterpret_cast<float*>(take((size_t)w.tm.d_pad * sizeof(float)));
	w.sm.center = w.tm.center;
	w.flag_list = reinterpret_cast<uint32_t*>(take(n * sizeof(uint32_t)));
	w.asg_scratch = reinterpret_cast<uint32_t*>(take(n * sizeof(uint32_t)));
	if (with_tc_points) {
		w.tp.n_pad = bkm::round_up64(n, bkm::TC_MTILE);
		w.tp.d_pad = w.tm.d_pad;
		const size_t aplane = (size_t)w.tp.n_pad * w.tp.d_pad * sizeof(float);
		w.tp.a_hi = reinterpret_cast<float*>(take(aplane));
		w.tp.a_lo = reinterpret_cast<float*>(take(aplane));
		w.tp.xnorm = reinterpret_cast<float*>(take((size_t)w.tp.n_pad * sizeof(float)));
		w.tp.partial = w.tp.d_pad > 32 ? reinterpret_cast<uint32_t*>(take((size_t)bkm::TC_JSPLIT * 3 * w.tp.n_pad * sizeof(uint32_t))) : nullptr;
	}
	w.bytes = off;
	return w;
}

int device_sm_count(int device, int* out)
{
	CUDA_TRY(cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, device));
	return BKM_OK;
}

int resolve_assign(int variant, const bkm::Shape& s, int* out)
{
	switch (variant) {
	case BKM_ASSIGN_AUTO:
		if (bkm::assign_simt_supported(s)) *out = BKM_ASSIGN_SIMT;
		else if (bkm::assign_tc_supported(s)) *out = BKM_ASSIGN_TC;
		else *out = BKM_ASSIGN_EXACT;
		return BKM_OK;
	case BKM_ASSIGN_EXACT:
		*out = variant;
		return BKM_OK;
	case BKM_ASSIGN_SIMT:
		if (!bkm::assign_simt_supported(s)) return fail(BKM_ERR_UNSUPPORTED, "the SIMT assignment handles dim 1..8 only (dim=%u)", s.dim);
		*out = variant;
		return BKM_OK;
	case BKM_ASSIGN_TC:
		if (!bkm::assign_tc_supported(s)) return fail(BKM_ERR_UNSUPPORTED, "the tensor-core assignment does not handle n=%llu k=%u dim=%u",
			(unsigned long long)s.n, s.k, s.dim);
		*out = variant;
		return BKM_OK;
	default:
		return fail(BKM_ERR_INVALID, "unknown assignment variant %d", variant);
	}
}

int resolve_update(int variant, const bkm::Shape& s, int device, int* out)
{
	switch (variant) {
	case BKM_UPDATE_AUTO:
		// row-major points: sort by cluster inside the block, one reduction per cluster and chunk;
		// dimension-major points: rows of at least 16 floats go out as one coalesced L2 reduction
		// per point, shorter ones through shared-memory buckets
		if (!s.soa && bkm::update_sorted_supported(s)) *out = BKM_UPDATE_SORTED;
		else if (s.dim >= 16) *out = BKM_UPDATE_ROWS;
		else *out = bkm::update_shared_fits(s, device) ? BKM_UPDATE_SHARED : BKM_UPDATE_GLOBAL;
		return BKM_OK;
	case BKM_UPDATE_ROWS:
		*out = variant;
		return BKM_OK;
	case BKM_UPDATE_SORTED:
		if (!bkm::update_sorted_supported(s)) return fail(BKM_ERR_UNSUPPORTED, "the sorted update handles at most 1024 clusters (k=%u)", s.k);
		*out = variant;
		return BKM_OK;
	case BKM_UPDATE_SHARED:
		if (!bkm::update_shared_fits(s, device)) return fail(BKM_ERR_UNSUPPORTED, "k*dim = %llu floats do not fit shared memory",
			(unsigned long long)s.k * s.dim);
		*out = variant;
		return BKM_OK;
	case BKM_UPDATE_GLOBAL:
		*out = variant;
		return BKM_OK;
	default:
		return fail(BKM_ERR_INVALID, "unknown update variant %d", variant);
	}
}

int check_shape(uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means)
{
	if (n == 0 || k == 0 || dim == 0) return fail(BKM_ERR_INVALID, "n, k and dim must be positive (n=%llu k=%u dim=%u)",
		(unsigned long long)n, k, dim);
	if (n >= (1ull << 32)) return fail(BKM_ERR_UNSUPPORTED, "at most 2^32-1 points per GPU (n=%llu)", (unsigned long long)n);
	if ((uint64_t)k * dim >= (1ull << 31)) return fail(BKM_ERR_UNSUPPORTED, "k*dim must stay below 2^31");
	if (!layout_ok(layout) || !layout_ok(layout_means)) return fail(BKM_ERR_INVALID, "unknown layout code");
	return BKM_OK;
}

// Enqueues one assignment pass (fast pass + exact re-check, or the exact kernel alone).
// With `fused` set the fast pass also accumulates the update sums and the re-check moves the
// points it reassigns, so no update pass must follow.
int enqueue_assign(int variant, const float* pts, const float* means, uint32_t* asg, const bkm::Shape& s,
	const Workspace& w, int slot, bkm::TcPlan* plan, float margin_scale, int sm_count, cudaStream_t stream,
	cudaEvent_t mid, const bkm::FusedAcc* fused = nullptr, bool fast_pass_done = false)
{
	if (variant == BKM_ASSIGN_EXACT) {
		CUDA_TRY(bkm::launch_assign_exact(pts, means, asg, s, nullptr, nullptr, sm_count, stream));
		if (mid) CUDA_TRY(cudaEventRecord(mid, stream));
		return BKM_OK;
	}
	if (fast_pass_done) {
		// (the pass ran behind the upload of the points: only the near-ties are left)
	} else if (variant == BKM_ASSIGN_SIMT) {
		CUDA_TRY(bkm::launch_assign_simt(pts, w.sm, asg, s, w.ctl, slot, w.flag_list, margin_scale, sm_count, stream, fused));
	} else {
		CUDA_TRY(bkm::launch_assign_tc(plan, asg, w.ctl, slot, w.flag_list, margin_scale, stream, fused));
	}
	if (mid) CUDA_TRY(cudaEventRecord(mid, stream));
	CUDA_TRY(bkm::launch_assign_exact(pts, means, asg, s, w.flag_list, &w.ctl->flag_count, sm_count, stream, fused, w.split_scratch));
	return BKM_OK;
}

} // namespace

// ---------------------------------------------------------------------------------------------

struct bkm_handle_s {
	bkm_config_t cfg{};
	bkm::Shape shape{};
	int sm_count = 0;
	cudaStream_t stream = nullptr;
	cudaStream_t own_stream = nullptr;
	static constexpr uint32_t UPLOAD_CHUNKS = 8;
	cudaStream_t copy_stream = nullptr;            // host points travel here chunk by chunk (tensor-core path)
	cudaEvent_t copy_ev[UPLOAD_CHUNKS] = {};       // chunk c has arrived
	// The fast assignment pass of the first iteration has already run, chunk by chunk behind the upload
	// (against the initial means, with or without the update sums): the first bkm_run only re-checks.
	bool first_pass_done = false, first_pass_fused = false;
	const float* d_points = nullptr;
	float* d_points_owned = nullptr;
	float* d_means[2] = {nullptr, nullptr};
	uint32_t* d_asg = nullptr;
	uint32_t* d_sizes = nullptr;
	char* d_ws = nullptr;
	Workspace ws;
	bkm::TcPlan* plan = nullptr;
	int assign_variant = 0, update_variant = 0;
	int cur = 0, slot = 0;
	bool initialized = false;
	uint64_t iters_done = 0;
	float margin_scale = 1.0f;
	bool phase_timing = true;
	// NCCL
	void* comm = nullptr;
	int world = 1, rank = 0;
	// peer-memory exchange: this rank's buffer, every rank's buffer as addressable from this device
	void* d_xbuf = nullptr;
	void* peer_base[bkm::EXCHANGE_MAX_RANKS] = {};
	bool peer_ipc[bkm::EXCHANGE_MAX_RANKS] = {};   // opened with cudaIpcOpenMemHandle (to be closed)
	int peer_world = 0;
	bool peer_on = false;
	uint32_t epoch = 0;                            // iterations exchanged so far (the same on every rank)
	uint64_t exchange_wait_ns = 2000000000ull;
	// phase events of the most recent run
	// Phase events are recorded for the last EV_RING iterations of a run only: six event records per
	// iteration cost 2-5 % of a 0.5 ms iteration.
	static constexpr int EV_RING = 8, EV_PER = 6;
	cudaEvent_t ev[EV_RING][EV_PER] = {};
	bool ev_made = false;
	uint32_t ev_count = 0;
	uint32_t launches_per_iter = 0;
	// CUDA graph of two iterations (launch-bound problem sizes)
	int use_graph = 2;                 // 0 = never, 1 = always (single GPU), 2 = by problem size
	bool tc_pair = true;               // let the tensor-core assignment use its CTA-pair kernel where it applies
	int fuse_update = 1;               // fast pass accumulates the update sums: 0 never, 1 where it pays, 2 wherever it can
	bool last_fused = false;
	cudaGraphExec_t graph_exec = nullptr;
	int graph_cur = 0, graph_slot = 0;
	cudaStream_t graph_stream = nullptr;
	cudaEvent_t ev_run[2] = {};
	// One process driving several GPUs (config.num_gpus > 1): this handle then owns no device state
	// itself but one handle per GPU, each with a contiguous shard of the points, joined by the
	// peer-memory exchange.
	std::vector<bkm_handle_s*> shards;
	std::vector<uint64_t> shard_begin;
};

extern "C" {

static void drop_graph(bkm_handle_t h);

const char* bkm_last_error(void) { return g_error.c_str(); }

int bkm_version(void) { return 100; }

int bkm_device_count(void)
{
	int n = 0;
	if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
	return n;
}

size_t bkm_workspace_bytes(uint64_t n, uint32_t k, uint32_t dim)
{
	if (n == 0 || k == 0 || dim == 0 || n >= (1ull << 32) || (uint64_t)k * dim >= (1ull << 31)) return 0;
	return carve(nullptr, n, k, dim, true).bytes;
}

int bkm_shard_range(uint64_t n_total, int world_size, int rank, uint64_t* begin, uint64_t* count)
{
	if (world_size <= 0 || rank < 0 || rank >= world_size || !begin || !count)
		return fail(BKM_ERR_INVALID, "bad shard arguments (world_size=%d rank=%d)", world_size, rank);
	const uint64_t base = n_total / (uint64_t)world_size, rem = n_total % (uint64_t)world_size;
	const uint64_t r = (uint64_t)rank;
	*begin = r * base + std::min<uint64_t>(r, rem);
	*count = base + (r < rem ? 1 : 0);
	return BKM_OK;
}

// ---- kernel-runner entry points ---------------------------------------------------------------

static int stateless_common(uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means,
	void* workspace, size_t workspace_bytes, bkm::Shape* s, Workspace* w, int* device, int* sm_count)
{
	int rc = check_shape(n, k, dim, layout, layout_means);
	if (rc) return rc;
	if (!workspace) return fail(BKM_ERR_INVALID, "workspace is null");
	if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(BKM_ERR_INVALID, "workspace must be 256-byte aligned");
	*w = carve(static_cast<char*>(workspace), n, k, dim, true);
	if (workspace_bytes < w->bytes) return fail(BKM_ERR_INVALID, "workspace too small: %zu < %zu bytes", workspace_bytes, w->bytes);
	s->n = n; s->k = k; s->dim = dim; s->soa = layout == BKM_LAYOUT_SOA; s->soa_means = layout_means == BKM_LAYOUT_SOA;
	CUDA_TRY(cudaGetDevice(device));
	return device_sm_count(*device, sm_count);
}

// Bytes of the control block that every stateless call clears: status, flag count and the two
// max |c|^2 slots.  last_flag_count and xmax2 behind them survive (xmax2 belongs to the points).
constexpr size_t CONTROL_CLEAR_BYTES = 16;

// Tensor maps are a function of the workspace address and the shape, so the stateless calls keep
// the few most recent plans instead of encoding six maps per call.
struct PlanSlot {
	void* ws = nullptr; uint64_t n = 0; uint32_t k = 0, dim = 0; int soa = 0, soa_means = 0, device = -1;
	bkm::TcPlan* plan = nullptr; uint64_t stamp = 0;
};
static std::mutex g_plan_mutex;
static PlanSlot g_plan_slots[8];
static uint64_t g_plan_clock = 0;

static bkm::TcPlan* cached_plan(const bkm::Shape& s, const Workspace& w, int device, const char** err)
{
	std::lock_guard<std::mutex> lock(g_plan_mutex);
	PlanSlot* victim = &g_plan_slots[0];
	for (PlanSlot& p : g_plan_slots) {
		if (p.plan && p.ws == (void*)w.ctl && p.n == s.n && p.k == s.k && p.dim == s.dim && p.soa == s.soa && p.soa_means == s.soa_means && p.device == device) {
			p.stamp = ++g_plan_clock;
			return p.plan;
		}
		if (p.stamp < victim->stamp) victim = &p;
	}
	bkm::TcPlan* plan = bkm::tc_plan_create(s, w.tp, w.tm, device, err);
	if (!plan) return nullptr;
	if (victim->plan) bkm::tc_plan_destroy(victim->plan);
	victim->ws = (void*)w.ctl; victim->n = s.n; victim->k = s.k; victim->dim = s.dim; victim->soa = s.soa; victim->soa_means = s.soa_means;
	victim->device = device; victim->plan = plan; victim->stamp = ++g_plan_clock;
	return plan;
}

// One assignment pass on a caller's workspace.  The operands derived from the (immutable) points -
// centre vector, largest norm, tf32 planes - stay in the workspace; a call that finds the same
// point set there (address, shape and a fingerprint of a sample of the values) skips them.
// Whether the fast assignment pass should accumulate the update sums itself.  On CTA pairs the
// epilogue warps send the reductions, which pays where the update would otherwise be the row-wise
// kernel (the sorted update of row-major points costs less than that).  In the CUDA-core pass every
// warp sorts the points it has just assigned by cluster and sends pre-added rows.
static bool fuse_pays(int assign_variant, int update_variant, const bkm::TcPlan* plan, const bkm::FusedAcc& fa, const bkm::Shape& s, bool force = false)
{
	if (assign_variant == BKM_ASSIGN_SIMT) {
		// measured: the warp-private sort adds 0.11 ms to a 0.32 ms pass over 2^24 two-dimensional points
		// where the separate sorted update takes 0.10 ms, so it pays only where a launch less does
		return bkm::assign_simt_can_fuse(s, fa) && (force || (double)s.n * s.k * s.dim <= 1.0e8);
	}
	if (assign_variant != BKM_ASSIGN_TC) return false;
	return update_variant == BKM_UPDATE_ROWS && bkm::tc_plan_can_fuse(plan, fa) && (size_t)s.dim * sizeof(float) * 4 <= 120 * 1024;
}

// With `fa` given and the shape allowing it, the pass also accumulates the update sums (*fused).
static int stateless_assign(const float* points, const float* means, uint32_t* assignment, const bkm::Shape& s,
	const Workspace& w, int variant, int device, int sm_count, cudaStream_t st, const bkm::FusedAcc* fa = nullptr, int variant_update = 0,
	bool* fused_out = nullptr)
{
	int v = 0;
	int rc = resolve_assign(variant, s, &v);
	if (rc) return rc;
	if (fused_out) *fused_out = false;
	CUDA_TRY(cudaMemsetAsync(w.ctl, 0, CONTROL_CLEAR_BYTES, st));
	CUDA_TRY(cudaMemsetAsync(w.split_scratch, 0, bkm::list_split_scratch_bytes(), st));
	bkm::TcPlan* plan = nullptr;
	bool fused = false;
	if (v == BKM_ASSIGN_SIMT || v == BKM_ASSIGN_TC) {
		bkm::PointsKey* key = reinterpret_cast<bkm::PointsKey*>(reinterpret_cast<char*>(w.ctl) + bkm::POINTS_KEY_OFFSET);
		const uint32_t* skip = &key->valid;
		CUDA_TRY(cudaMemsetAsync(&key->fp_new, 0, sizeof(key->fp_new), st));
		CUDA_TRY(bkm::launch_points_fingerprint(points, s.n * s.dim, key, sm_count, st));
		CUDA_TRY(bkm::launch_points_key_decide(key, points, s, v, w.ctl, st));
		CUDA_TRY(bkm::launch_compute_center(points, s, w.tm.center, st, skip));
		if (v == BKM_ASSIGN_SIMT) {
			CUDA_TRY(cudaMemsetAsync(w.sm.rows, 0, w.cprep_bytes, st));
			CUDA_TRY(bkm::launch_points_norm_max(points, s, w.tm.center, w.ctl, sm_count, st, skip));
			bkm::launch_prepare_means(means, s, &w.sm, nullptr, w.ctl, 0, st);
			fused = fa != nullptr && fuse_pays(v, variant_update, nullptr, *fa, s, true);     // the caller asked for the one-pass form
		} else {
			CUDA_TRY(cudaMemsetAsync(w.tm.b_hi, 0, w.tm_bytes, st));
			bkm::launch_prepare_means(means, s, nullptr, &w.tm, w.ctl, 0, st);
			CUDA_TRY(bkm::launch_split_points(points, s, w.tp, w.tm.center, w.ctl, st, skip));
			const char* err = nullptr;
			plan = cached_plan(s, w, device, &err);
			if (!plan) return fail(BKM_ERR_CUDA, "tensor-core plan: %s", err ? err : "unknown");
			bkm::tc_plan_allow_pair(plan, true);
			fused = fa != nullptr && fuse_pays(v, variant_update, plan, *fa, s);
		}
		if (fused) CUDA_TRY(cudaMemsetAsync(w.acc, 0, w.acc_bytes, st));
	}
	CUDA_TRY(cudaGetLastError());
	if (fused_out) *fused_out = fused;
	return enqueue_assign(v, points, means, assignment, s, w, 0, plan, 1.0f, sm_count, st, nullptr, fused ? fa : nullptr);
}

static int stateless_update(const float* points, const uint32_t* assignment, float* means, uint32_t* sizes,
	const bkm::Shape& s, const Workspace& w, int variant, int device, int sm_count, cudaStream_t st, bool clear_ctl)
{
	int v = 0;
	int rc = resolve_update(variant, s, device, &v);
	if (rc) return rc;
	if (clear_ctl) CUDA_TRY(cudaMemsetAsync(w.ctl, 0, CONTROL_CLEAR_BYTES, st));
	CUDA_TRY(cudaMemsetAsync(w.acc, 0, w.acc_bytes, st));
	bkm::launch_update(points, assignment, w.acc, w.counts, w.replicas, s, v, w.ctl, sm_count, st);
	bkm::launch_finalize(w.acc, w.counts, w.replicas, means, sizes, s, nullptr, nullptr, w.ctl, 1, st);
	CUDA_TRY(cudaGetLastError());
	return BKM_OK;
}

int bkm_assign_f32(const float* points, const float* means, uint32_t* assignment,
	uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means,
	int variant, void* workspace, size_t workspace_bytes, void* stream)
{
	if (!points || !means || !assignment) return fail(BKM_ERR_INVALID, "null pointer argument");
	bkm::Shape s; Workspace w; int device = 0, sm = 0;
	int rc = stateless_common(n, k, dim, layout, layout_means, workspace, workspace_bytes, &s, &w, &device, &sm);
	if (rc) return rc;
	return stateless_assign(points, means, assignment, s, w, variant, device, sm, static_cast<cudaStream_t>(stream));
}

int bkm_update_f32(const float* points, const uint32_t* assignment, float* means, uint32_t* sizes,
	uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means,
	int variant, void* workspace, size_t workspace_bytes, void* stream)
{
	if (!points || !means || !assignment || !sizes) return fail(BKM_ERR_INVALID, "null pointer argument");
	bkm::Shape s; Workspace w; int device = 0, sm = 0;
	int rc = stateless_common(n, k, dim, layout, layout_means, workspace, workspace_bytes, &s, &w, &device, &sm);
	if (rc) return rc;
	return stateless_update(points, assignment, means, sizes, s, w, variant, device, sm, static_cast<cudaStream_t>(stream), true);
}

int bkm_bucket_sums_f32(const float* points, const uint32_t* indices, float* sums,
	uint64_t n, uint32_t k, uint32_t dim, int layout, int variant, void* workspace, size_t workspace_bytes, void* stream)
{
	if (!points || !indices || !sums) return fail(BKM_ERR_INVALID, "null pointer argument");
	bkm::Shape s; Workspace w; int device = 0, sm = 0;
	int rc = stateless_common(n, k, dim, layout, layout, workspace, workspace_bytes, &s, &w, &device, &sm);
	if (rc) return rc;
	int v = 0;
	if ((rc = resolve_update(variant, s, device, &v))) return rc;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	CUDA_TRY(cudaMemsetAsync(w.ctl, 0, CONTROL_CLEAR_BYTES, st));
	CUDA_TRY(cudaMemsetAsync(w.acc, 0, w.acc_bytes, st));
	bkm::launch_update(points, indices, w.acc, w.counts, w.replicas, s, v, w.ctl, sm, st);
	bkm::launch_finalize_sums(w.acc, w.counts, w.replicas, sums, s, w.ctl, st);
	CUDA_TRY(cudaGetLastError());
	return BKM_OK;
}

int bkm_probe_atomics_f32(float* result, uint64_t n, uint32_t k, uint32_t dim, int layout, int shared_cache, uint32_t items_per_thread, void* stream)
{
	if (!result) return fail(BKM_ERR_INVALID, "null pointer argument");
	if (n == 0 || k == 0 || dim == 0 || items_per_thread == 0) return fail(BKM_ERR_INVALID, "n, k, dim and items_per_thread must be positive");
	if (!layout_ok(layout)) return fail(BKM_ERR_INVALID, "unknown layout code");
	CUDA_TRY(bkm::launch_probe_atomics(result, n, k, dim, layout == BKM_LAYOUT_SOA, shared_cache != 0, items_per_thread, static_cast<cudaStream_t>(stream)));
	return BKM_OK;
}

int bkm_iterate_f32(const float* points, const float* means_in, float* means_out, uint32_t* sizes,
	uint32_t* assignment, uint64_t n, uint32_t k, uint32_t dim, int layout,
	int layout_means, int variant_assign, int variant_update,
	void* workspace, size_t workspace_bytes, void* stream)
{
	if (!points || !means_in || !means_out || !sizes) return fail(BKM_ERR_INVALID, "null pointer argument");
	if (means_in == means_out) return fail(BKM_ERR_INVALID, "means_in and means_out must differ");
	bkm::Shape s; Workspace w; int device = 0, sm = 0;
	int rc = stateless_common(n, k, dim, layout, layout_means, workspace, workspace_bytes, &s, &w, &device, &sm);
	if (rc) return rc;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	uint32_t* asg = assignment ? assignment : w.asg_scratch;
	// Where the assignment pass can accumulate the sums itself (the CUDA-core pass for up to 8
	// dimensions and 1024 means; the shapes of the CTA-pair kernel with an update that would
	// otherwise be the row-wise kernel) the points are read once.
	int vu = 0;
	if ((rc = resolve_update(variant_update, s, device, &vu))) return rc;
	bkm::FusedAcc fa{w.acc, w.counts, w.replicas, bkm::acc_replica_stride(k, dim), w.tm.center};
	bool fused = false;
	rc = stateless_assign(points, means_in, asg, s, w, variant_assign, device, sm, st, &fa, vu, &fused);
	if (rc) return rc;
	if (fused) {
		bkm::launch_finalize(w.acc, w.counts, w.replicas, means_out, sizes, s, nullptr, nullptr, w.ctl, 1, st);
		CUDA_TRY(cudaGetLastError());
		return BKM_OK;
	}
	return stateless_update(points, asg, means_out, sizes, s, w, variant_update, device, sm, st, false);
}

// Waits for `stream` and returns BKM_ERR_DEVICE if a kernel of the last stateless call on this
// workspace recorded an error.
int bkm_workspace_check(const void* workspace, void* stream)
{
	if (!workspace) return fail(BKM_ERR_INVALID, "workspace is null");
	bkm::Control c;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	CUDA_TRY(cudaMemcpyAsync(&c, workspace, sizeof(c), cudaMemcpyDeviceToHost, st));
	CUDA_TRY(cudaStreamSynchronize(st));
	if (c.status) return fail(BKM_ERR_DEVICE, "kernel status 0x%x (1=wait timeout, 2=assignment out of range, 4=list overflow)", c.status);
	return BKM_OK;
}

// Exercises the failure path of the kernels' bounded waits without breaking anything: a one-thread
// kernel waits `limit_ms` (1..1000) for a barrier nobody arrives on, gives up and records
// STATUS_WAIT_TIMEOUT in the workspace's control block.  Returns BKM_OK after enqueueing; the
// status is then visible to bkm_workspace_check (BKM_ERR_DEVICE), and the workspace must be
// cleared (or passed to a stateless call, which clears the status) before further use.
int bkm_selftest_wait_timeout(void* workspace, uint32_t limit_ms, void* stream)
{
	if (!workspace) return fail(BKM_ERR_INVALID, "workspace is null");
	if (limit_ms < 1 || limit_ms > 1000) return fail(BKM_ERR_INVALID, "limit_ms must be 1..1000");
	CUDA_TRY(bkm::launch_wait_timeout_selftest(reinterpret_cast<bkm::Control*>(workspace), (uint64_t)limit_ms * 1000000ull,
		static_cast<cudaStream_t>(stream)));
	return BKM_OK;
}

// ---- driver -------------------------------------------------------------------------------------

// One process, several GPUs: one shard handle per device, joined by the peer-memory exchange over
// directly attached buffers (peer access between all pairs of the devices is required).
static int create_group(const bkm_config_t* cfg, int ndev, bkm_handle_t* out)
{
	const int g_count = cfg->num_gpus;
	if (cfg->device < 0 || cfg->device + g_count > ndev)
		return fail(BKM_ERR_INVALID, "devices %d..%d requested, %d present", cfg->device, cfg->device + g_count - 1, ndev);
	if (cfg->n < (uint64_t)g_count) return fail(BKM_ERR_INVALID, "fewer points than GPUs");
	if ((uint64_t)cfg->k * cfg->dim + cfg->k > bkm::EXCHANGE_MAX_WORDS)
		return fail(BKM_ERR_UNSUPPORTED, "k*dim + k = %llu is beyond the peer-memory exchange (%llu words): run one process per GPU with bkm_comm_init",
			(unsigned long long)cfg->k * cfg->dim + cfg->k, (unsigned long long)bkm::EXCHANGE_MAX_WORDS);
	for (int a = 0; a < g_count; ++a)
		for (int b = 0; b < g_count; ++b) {
			if (a == b) continue;
			int can = 0;
			CUDA_TRY(cudaDeviceCanAccessPeer(&can, cfg->device + a, cfg->device + b));
			if (!can) return fail(BKM_ERR_UNSUPPORTED, "device %d cannot access the memory of device %d", cfg->device + a, cfg->device + b);
			CUDA_TRY(cudaSetDevice(cfg->device + a));
			const cudaError_t e = cudaDeviceEnablePeerAccess(cfg->device + b, 0);
			if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail(BKM_ERR_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
			cudaGetLastError();
		}
	bkm_handle_s* h = new (std::nothrow) bkm_handle_s();
	if (!h) return fail(BKM_ERR_INVALID, "out of host memory");
	h->cfg = *cfg;
	h->shape.n = cfg->n; h->shape.k = cfg->k; h->shape.dim = cfg->dim;
	h->shape.soa = cfg->layout == BKM_LAYOUT_SOA; h->shape.soa_means = cfg->layout_means == BKM_LAYOUT_SOA;
	auto bail = [&](int code) { std::string keep = g_error; bkm_destroy(h); g_error = keep; return code; };
	void* bases[bkm::EXCHANGE_MAX_RANKS] = {};
	for (int g = 0; g < g_count; ++g) {
		uint64_t begin = 0, count = 0;
		bkm_shard_range(cfg->n, g_count, g, &begin, &count);
		bkm_config_t c = *cfg;
		c.n = count; c.device = cfg->device + g; c.num_gpus = 0;
		bkm_handle_t child = nullptr;
		int rc = bkm_create(&c, &child);
		if (rc) return bail(rc);
		h->shards.push_back(child);
		h->shard_begin.push_back(begin);
		if ((rc = bkm_peer_buffer(child, &bases[g], nullptr))) return bail(rc);
	}
	for (int g = 0; g < g_count; ++g) {
		int rc = bkm_peer_attach(h->shards[g], bases, g_count, g);
		if (rc == BKM_OK) rc = bkm_peer_enable(h->shards[g], 1);
		if (rc) return bail(rc);
	}
	*out = h;
	return BKM_OK;
}

#define NOT_FOR_GROUPS(h, what) do { if (!(h)->shards.empty()) \
	return fail(BKM_ERR_UNSUPPORTED, "%s is not available on a handle that drives several GPUs", what); } while (0)

int bkm_create(const bkm_config_t* cfg, bkm_handle_t* out)
{
	if (!cfg || !out) return fail(BKM_ERR_INVALID, "null argument");
	*out = nullptr;
	if (cfg->num_gpus < 0 || cfg->num_gpus > (int)bkm::EXCHANGE_MAX_RANKS) return fail(BKM_ERR_INVALID, "num_gpus must be 0..%d", (int)bkm::EXCHANGE_MAX_RANKS);
	int rc = check_shape(cfg->n, cfg->k, cfg->dim, cfg->layout, cfg->layout_means);
	if (rc) return rc;
	int ndev = bkm_device_count();
	if (ndev == 0) return fail(BKM_ERR_CUDA, "no CUDA device");
	if (cfg->num_gpus > 1) return create_group(cfg, ndev, out);
	if (cfg->device < 0 || cfg->device >= ndev) return fail(BKM_ERR_INVALID, "device %d out of range (0..%d)", cfg->device, ndev - 1);
	CUDA_TRY(cudaSetDevice(cfg->device));

	bkm_handle_s* h = new (std::nothrow) bkm_handle_s();
	if (!h) return fail(BKM_ERR_INVALID, "out of host memory");
	h->cfg = *cfg;
	h->shape.n = cfg->n; h->shape.k = cfg->k; h->shape.dim = cfg->dim;
	h->shape.soa = cfg->layout == BKM_LAYOUT_SOA; h->shape.soa_means = cfg->layout_means == BKM_LAYOUT_SOA;
	auto bail = [&](int code) { bkm_destroy(h); return code; };
	if ((rc = device_sm_count(cfg->device, &h->sm_count))) return bail(rc);
	if ((rc = resolve_assign(cfg->variant_assign, h->shape, &h->assign_variant))) return bail(rc);
	if ((rc = resolve_update(cfg->variant_update, h->shape, cfg->device, &h->update_variant))) return bail(rc);

	cudaError_t e;
	if ((e = cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking)) != cudaSuccess)
		return bail(fail(BKM_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)));
	h->stream = h->own_stream;
	const size_t kd = (size_t)cfg->k * cfg->dim;
	const bool tc = h->assign_variant == BKM_ASSIGN_TC;
	h->ws = carve(nullptr, cfg->n, cfg->k, cfg->dim, tc);
	if ((e = cudaMalloc(&h->d_means[0], kd * sizeof(float))) != cudaSuccess ||
		(e = cudaMalloc(&h->d_means[1], kd * sizeof(float))) != cudaSuccess ||
		(e = cudaMalloc(&h->d_asg, cfg->n * sizeof(uint32_t))) != cudaSuccess ||
		(e = cudaMalloc(&h->d_sizes, (size_t)cfg->k * sizeof(uint32_t))) != cudaSuccess ||
		(e = cudaMalloc(&h->d_ws, h->ws.bytes)) != cudaSuccess)
		return bail(fail(BKM_ERR_CUDA, "cudaMalloc: %s", cudaGetErrorString(e)));
	h->ws = carve(h->d_ws, cfg->n, cfg->k, cfg->dim, tc);
	if ((e = cudaMemset(h->d_ws, 0, h->ws.bytes)) != cudaSuccess ||
		(e = cudaMemset(h->d_asg, 0, cfg->n * sizeof(uint32_t))) != cudaSuccess ||
		(e = cudaMemset(h->d_sizes, 0, (size_t)cfg->k * sizeof(uint32_t))) != cudaSuccess)
		return bail(fail(BKM_ERR_CUDA, "cudaMemset: %s", cudaGetErrorString(e)));
	for (int i = 0; i < bkm_handle_s::EV_RING; ++i)
		for (int j = 0; j < bkm_handle_s::EV_PER; ++j)
			if ((e = cudaEventCreate(&h->ev[i][j])) != cudaSuccess)
				return bail(fail(BKM_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(e)));
	h->ev_made = true;
	for (int j = 0; j < 2; ++j)
		if ((e = cudaEventCreate(&h->ev_run[j])) != cudaSuccess)
			return bail(fail(BKM_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(e)));
	*out = h;
	return BKM_OK;
}

int bkm_destroy(bkm_handle_t h)
{
	if (!h) return BKM_OK;
	if (!h->shards.empty()) {
		for (bkm_handle_s* c : h->shards) bkm_destroy(c);
		delete h;
		return BKM_OK;
	}
	cudaSetDevice(h->cfg.device);
	if (h->stream) cudaStreamSynchronize(h->stream);
	drop_graph(h);
	if (h->comm && nccl()->ok) nccl()->CommDestroy(h->comm);
	for (uint32_t r = 0; r < bkm::EXCHANGE_MAX_RANKS; ++r)
		if (h->peer_ipc[r] && h->peer_base[r]) cudaIpcCloseMemHandle(h->peer_base[r]);
	cudaFree(h->d_xbuf);
	if (h->plan) bkm::tc_plan_destroy(h->plan);
	for (int i = 0; i < bkm_handle_s::EV_RING; ++i)
		for (int j = 0; j < bkm_handle_s::EV_PER; ++j)
			if (h->ev[i][j]) cudaEventDestroy(h->ev[i][j]);
	for (int j = 0; j < 2; ++j) if (h->ev_run[j]) cudaEventDestroy(h->ev_run[j]);
	cudaFree(h->d_points_owned);
	cudaFree(h->d_means[0]);
	cudaFree(h->d_means[1]);
	cudaFree(h->d_asg);
	cudaFree(h->d_sizes);
	cudaFree(h->d_ws);
	if (h->own_stream) cudaStreamDestroy(h->own_stream);
	if (h->copy_stream) cudaStreamDestroy(h->copy_stream);
	for (cudaEvent_t e : h->copy_ev) if (e) cudaEventDestroy(e);
	delete h;
	return BKM_OK;
}

int bkm_set_stream(bkm_handle_t h, void* stream)
{
	if (!h) return fail(BKM_ERR_INVALID, "null handle");
	NOT_FOR_GROUPS(h, "bkm_set_stream");
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	h->stream = static_cast<cudaStream_t>(stream);   // NULL is the legacy default stream
	return BKM_OK;
}

static int drop_first_pass(bkm_handle_t h);

int bkm_set_option(bkm_handle_t h, const char* name, double value)
{
	if (!h || !name) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->shards.empty()) {
		for (bkm_handle_s* c : h->shards) { const int rc = bkm_set_option(c, name, value); if (rc) return rc; }
		return BKM_OK;
	}
	if (!strcmp(name, "margin_scale") || !strcmp(name, "tc_pair") || !strcmp(name, "fuse_update")) {
		// a first pass that ran behind the upload used the old setting
		CUDA_TRY(cudaSetDevice(h->cfg.device));
		const int rc = drop_first_pass(h);
		if (rc) return rc;
	}
	if (!strcmp(name, "margin_scale")) {
		if (!(value > 0.0)) return fail(BKM_ERR_INVALID, "margin_scale must be positive");
		h->margin_scale = (float)value;
		return BKM_OK;
	}
	if (!strcmp(name, "phase_timing")) { h->phase_timing = value != 0.0; return BKM_OK; }
	if (!strcmp(name, "use_graph")) {
		if (value != 0.0 && value != 1.0 && value != 2.0) return fail(BKM_ERR_INVALID, "use_graph is 0 (never), 1 (always) or 2 (by size)");
		h->use_graph = (int)value;
		drop_graph(h);
		return BKM_OK;
	}
	if (!strcmp(name, "fuse_update")) {
		h->fuse_update = value >= 2.0 ? 2 : (value != 0.0 ? 1 : 0);
		drop_graph(h);
		return BKM_OK;
	}
	if (!strcmp(name, "exchange_wait_ms")) {
		if (!(value >= 1.0 && value <= 600000.0)) return fail(BKM_ERR_INVALID, "exchange_wait_ms must be 1..600000");
		h->exchange_wait_ns = (uint64_t)(value * 1.0e6);
		return BKM_OK;
	}
	if (!strcmp(name, "tc_pair")) {
		h->tc_pair = value != 0.0;
		bkm::tc_plan_allow_pair(h->plan, h->tc_pair);
		drop_graph(h);
		return BKM_OK;
	}
	return fail(BKM_ERR_INVALID, "unknown option '%s'", name);
}

// First part of an initialisation: state reset, means, cleared workspace (all on the handle's stream).
static int initialize_begin(bkm_handle_t h, const float* means, cudaMemcpyKind kind)
{
	const bkm::Shape& s = h->shape;
	const size_t kd = (size_t)s.k * s.dim;
	cudaStream_t st = h->stream;
	h->cur = 0; h->slot = 0; h->iters_done = 0; h->ev_count = 0;
	h->first_pass_done = false;
	drop_graph(h);
	CUDA_TRY(cudaMemcpyAsync(h->d_means[0], means, kd * sizeof(float), kind, st));
	CUDA_TRY(cudaMemsetAsync(h->d_ws, 0, (size_t)(reinterpret_cast<char*>(h->ws.flag_list) - h->d_ws), st));
	CUDA_TRY(cudaMemsetAsync(h->d_asg, 0, s.n * sizeof(uint32_t), st));
	CUDA_TRY(cudaMemsetAsync(h->d_sizes, 0, (size_t)s.k * sizeof(uint32_t), st));
	return BKM_OK;
}

// Second part: what is derived from the points (unless the caller has done that chunk by chunk while
// they arrived: `points_done`), the operands derived from the means, then a wait for all of it.
// The tensor-core plan and the operands derived from the initial means (the centre must be known).
static int prepare_plan_and_means(bkm_handle_t h)
{
	const bkm::Shape& s = h->shape;
	if (h->assign_variant == BKM_ASSIGN_TC) {
		if (h->plan) { bkm::tc_plan_destroy(h->plan); h->plan = nullptr; }
		const char* err = nullptr;
		h->plan = bkm::tc_plan_create(s, h->ws.tp, h->ws.tm, h->cfg.device, &err);
		if (!h->plan) return fail(BKM_ERR_CUDA, "tensor-core plan: %s", err ? err : "unknown");
		bkm::tc_plan_allow_pair(h->plan, h->tc_pair);
	}
	bkm::launch_prepare_means(h->d_means[0], s,
		h->assign_variant == BKM_ASSIGN_SIMT ? &h->ws.sm : nullptr,
		h->assign_variant == BKM_ASSIGN_TC ? &h->ws.tm : nullptr, h->ws.ctl, h->slot, h->stream);
	CUDA_TRY(cudaGetLastError());
	return BKM_OK;
}

static int initialize_finish(bkm_handle_t h, bool points_done)
{
	const bkm::Shape& s = h->shape;
	cudaStream_t st = h->stream;
	if (h->assign_variant == BKM_ASSIGN_SIMT) {
		CUDA_TRY(bkm::launch_compute_center(h->d_points, s, h->ws.tm.center, st));
		CUDA_TRY(bkm::launch_points_norm_max(h->d_points, s, h->ws.tm.center, h->ws.ctl, h->sm_count, st));
	}
	if (!points_done) {
		if (h->assign_variant == BKM_ASSIGN_TC) {
			CUDA_TRY(bkm::launch_compute_center(h->d_points, s, h->ws.tm.center, st));
			CUDA_TRY(bkm::launch_split_points(h->d_points, s, h->ws.tp, h->ws.tm.center, h->ws.ctl, st));
		}
		const int rc = prepare_plan_and_means(h);
		if (rc) return rc;
	}
	CUDA_TRY(cudaGetLastError());
	CUDA_TRY(cudaStreamSynchronize(st));
	h->initialized = true;
	return BKM_OK;
}

static int initialize_common(bkm_handle_t h, const float* means, cudaMemcpyKind kind)
{
	const int rc = initialize_begin(h, means, kind);
	return rc ? rc : initialize_finish(h, false);
}

// Host points of the tensor-core path travel in chunks on a stream of their own, and every chunk is
// split into its operand planes on the handle's stream as soon as it has arrived, while the next one is
// on its way: the splitting (one read and two writes of the points) hides behind the upload.  The
// centre comes from the first chunk (any vector serves).  Returns with the copies and kernels enqueued.
static int upload_and_split(bkm_handle_t h, const float* host_points)
{
	const bkm::Shape& s = h->shape;
	if (!h->copy_stream) CUDA_TRY(cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking));
	for (cudaEvent_t& e : h->copy_ev)
		if (!e) CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
	const uint64_t chunk = bkm::round_up64((s.n + bkm_handle_s::UPLOAD_CHUNKS - 1) / bkm_handle_s::UPLOAD_CHUNKS, 4096);
	bkm::FusedAcc fa{h->ws.acc, h->ws.counts, h->ws.replicas, bkm::acc_replica_stride(s.k, s.dim), h->ws.tm.center};
	bool fused = false, early_pass = false;
	// the copies must not overtake the clearing of the workspace and of what the previous use left in the planes' consumers
	CUDA_TRY(cudaEventRecord(h->copy_ev[0], h->stream));
	CUDA_TRY(cudaStreamWaitEvent(h->copy_stream, h->copy_ev[0], 0));
	uint32_t c = 0;
	for (uint64_t p0 = 0; p0 < s.n; p0 += chunk, ++c) {
		const uint64_t p1 = std::min<uint64_t>(p0 + chunk, s.n), count = p1 - p0;
		if (s.soa)
			CUDA_TRY(cudaMemcpy2DAsync(h->d_points_owned + p0, (size_t)s.n * sizeof(float), host_points + p0, (size_t)s.n * sizeof(float),
				(size_t)count * sizeof(float), s.dim, cudaMemcpyHostToDevice, h->copy_stream));
		else
			CUDA_TRY(cudaMemcpyAsync(h->d_points_owned + (size_t)p0 * s.dim, host_points + (size_t)p0 * s.dim, (size_t)count * s.dim * sizeof(float),
				cudaMemcpyHostToDevice, h->copy_stream));
		CUDA_TRY(cudaEventRecord(h->copy_ev[c], h->copy_stream));
		CUDA_TRY(cudaStreamWaitEvent(h->stream, h->copy_ev[c], 0));
		if (c == 0) {
			CUDA_TRY(bkm::launch_compute_center(h->d_points, s, h->ws.tm.center, h->stream, nullptr, count));
			const int rc = prepare_plan_and_means(h);
			if (rc) return rc;
			// On CTA pairs the fast pass of the first iteration follows the upload chunk by chunk as well
			// (its key constants need the largest |x|^2 of the launch's own points only, and the running
			// maximum covers those); the first bkm_run then starts at the re-check.
			fused = h->fuse_update && fuse_pays(h->assign_variant, h->update_variant, h->plan, fa, s, h->fuse_update >= 2);
			early_pass = bkm::tc_plan_uses_pair(h->plan);
		}
		// the last chunk also takes the padding rows behind the last point
		CUDA_TRY(bkm::launch_split_points(h->d_points, s, h->ws.tp, h->ws.tm.center, h->ws.ctl, h->stream, nullptr,
			p0, p1 == s.n ? h->ws.tp.n_pad : p1));
		if (early_pass)
			CUDA_TRY(bkm::launch_assign_tc(h->plan, h->d_asg, h->ws.ctl, h->slot, h->ws.flag_list, h->margin_scale, h->stream,
				fused ? &fa : nullptr, p0, p1));
	}
	h->first_pass_done = early_pass;
	h->first_pass_fused = fused;
	return BKM_OK;
}

// Forgets a first pass that ran behind the upload (the means or a setting it depended on change):
// its sums and its near-tie list are cleared, the next iteration runs the pass again.
static int drop_first_pass(bkm_handle_t h)
{
	if (!h->first_pass_done) return BKM_OK;
	h->first_pass_done = false;
	CUDA_TRY(cudaMemsetAsync(h->ws.acc, 0, h->ws.acc_bytes, h->stream));
	CUDA_TRY(cudaMemsetAsync(&h->ws.ctl->flag_count, 0, sizeof(uint32_t), h->stream));
	return BKM_OK;
}

int bkm_initialize(bkm_handle_t h, const float* host_points, const float* host_means)
{
	if (!h || !host_points || !host_means) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->shards.empty()) {
		// every GPU gets its contiguous range of points: rows of the row-major array, or the same
		// column range of every dimension of the dimension-major one
		const uint64_t n_total = h->shape.n;
		const uint32_t dim = h->shape.dim;
		for (size_t g = 0; g < h->shards.size(); ++g) {
			bkm_handle_s* c = h->shards[g];
			const uint64_t begin = h->shard_begin[g], count = c->shape.n;
			if (!h->shape.soa) {
				const int rc = bkm_initialize(c, host_points + (size_t)begin * dim, host_means);
				if (rc) return rc;
				continue;
			}
			CUDA_TRY(cudaSetDevice(c->cfg.device));
			if (!c->d_points_owned) CUDA_TRY(cudaMalloc(&c->d_points_owned, (size_t)count * dim * sizeof(float)));
			c->d_points = c->d_points_owned;
			CUDA_TRY(cudaMemcpy2DAsync(c->d_points_owned, (size_t)count * sizeof(float), host_points + begin, (size_t)n_total * sizeof(float),
				(size_t)count * sizeof(float), dim, cudaMemcpyHostToDevice, c->stream));
			const int rc = initialize_common(c, host_means, cudaMemcpyHostToDevice);
			if (rc) return rc;
		}
		h->initialized = true;
		return BKM_OK;
	}
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	const size_t bytes = (size_t)h->shape.n * h->shape.dim * sizeof(float);
	if (!h->d_points_owned) CUDA_TRY(cudaMalloc(&h->d_points_owned, bytes));
	h->d_points = h->d_points_owned;
	if (h->assign_variant == BKM_ASSIGN_TC && bytes >= ((size_t)32 << 20)) {
		int rc = initialize_begin(h, host_means, cudaMemcpyHostToDevice);
		if (!rc) rc = upload_and_split(h, host_points);
		if (rc) h->first_pass_done = false;
		return rc ? rc : initialize_finish(h, true);
	}
	CUDA_TRY(cudaMemcpyAsync(h->d_points_owned, host_points, bytes, cudaMemcpyHostToDevice, h->stream));
	return initialize_common(h, host_means, cudaMemcpyHostToDevice);
}

int bkm_initialize_device(bkm_handle_t h, const float* dev_points, const float* dev_means)
{
	if (!h || !dev_points || !dev_means) return fail(BKM_ERR_INVALID, "null argument");
	NOT_FOR_GROUPS(h, "bkm_initialize_device (the points of a shard must lie on its own GPU)");
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	h->d_points = dev_points;
	return initialize_common(h, dev_means, cudaMemcpyDeviceToDevice);
}

int bkm_set_means(bkm_handle_t h, const float* host_means)
{
	if (!h || !host_means) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->initialized) return fail(BKM_ERR_STATE, "set_means before initialize");
	if (!h->shards.empty()) {
		for (bkm_handle_s* c : h->shards) { const int rc = bkm_set_means(c, host_means); if (rc) return rc; }
		return BKM_OK;
	}
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	const bkm::Shape& s = h->shape;
	cudaStream_t st = h->stream;
	{ const int rc = drop_first_pass(h); if (rc) return rc; }
	CUDA_TRY(cudaMemcpyAsync(h->d_means[h->cur], host_means, (size_t)s.k * s.dim * sizeof(float), cudaMemcpyHostToDevice, st));
	// the preparation fills cmax2[slot] with atomicMax, so the slot starts from zero
	CUDA_TRY(cudaMemsetAsync(&h->ws.ctl->cmax2[h->slot], 0, sizeof(float), st));
	bkm::launch_prepare_means(h->d_means[h->cur], s,
		h->assign_variant == BKM_ASSIGN_SIMT ? &h->ws.sm : nullptr,
		h->assign_variant == BKM_ASSIGN_TC ? &h->ws.tm : nullptr, h->ws.ctl, h->slot, st);
	CUDA_TRY(cudaGetLastError());
	CUDA_TRY(cudaStreamSynchronize(st));
	return BKM_OK;
}

// Enqueues one iteration on the handle's stream; `ev` (6 events) brackets the phases when given.
static int enqueue_iteration(bkm_handle_t h, cudaEvent_t* ev)
{
	const bkm::Shape& s = h->shape;
	cudaStream_t st = h->stream;
	const size_t kd = (size_t)s.k * s.dim;
	const int next = h->cur ^ 1;
	if (ev) CUDA_TRY(cudaEventRecord(ev[0], st));
	// The CTA-pair tensor-core pass and the CUDA-core pass can add every point to its cluster's sum on
	// the way (the accumulators are zero between iterations: the finalize pass clears what it has read).
	bkm::FusedAcc fa{h->ws.acc, h->ws.counts, h->ws.replicas, bkm::acc_replica_stride(s.k, s.dim), h->ws.tm.center};
	const bool fused = h->fuse_update && fuse_pays(h->assign_variant, h->update_variant, h->plan, fa, s, h->fuse_update >= 2);
	h->last_fused = fused;
	h->launches_per_iter = (h->assign_variant == BKM_ASSIGN_EXACT ? 1u : 2u) + (fused ? 0u : 1u) + 1u;
	bool fast_pass_done = false;
	if (h->first_pass_done) {
		// usable if nothing has happened since bkm_initialize and the sums went where this iteration expects them
		if (h->iters_done == 0 && h->cur == 0 && h->slot == 0 && h->assign_variant == BKM_ASSIGN_TC && fused == h->first_pass_fused) {
			fast_pass_done = true;
			h->first_pass_done = false;
		} else {
			const int rc0 = drop_first_pass(h);
			if (rc0) return rc0;
		}
	}
	int rc = enqueue_assign(h->assign_variant, h->d_points, h->d_means[h->cur], h->d_asg, s, h->ws, h->slot,
		h->plan, h->margin_scale, h->sm_count, st, ev ? ev[1] : nullptr, fused ? &fa : nullptr, fast_pass_done);
	if (rc) return rc;
	if (ev) CUDA_TRY(cudaEventRecord(ev[2], st));
	if (!fused)
		bkm::launch_update(h->d_points, h->d_asg, h->ws.acc, h->ws.counts, h->ws.replicas, s, h->update_variant, h->ws.ctl, h->sm_count, st);
	if (ev) CUDA_TRY(cudaEventRecord(ev[3], st));
	if (h->peer_on) {
		// one kernel: publish this rank's sums, read the peers', add in rank order, divide, next operands
		++h->epoch;
		CUDA_TRY(bkm::launch_exchange_finalize(h->ws.acc, h->ws.counts, h->ws.replicas, h->peer_base, (uint32_t)h->peer_world,
			(uint32_t)h->rank, h->epoch, h->exchange_wait_ns, h->d_means[next], h->d_sizes, s,
			h->assign_variant == BKM_ASSIGN_SIMT ? &h->ws.sm : nullptr,
			h->assign_variant == BKM_ASSIGN_TC ? &h->ws.tm : nullptr, h->ws.ctl, h->slot ^ 1, st));
		if (ev) { CUDA_TRY(cudaEventRecord(ev[4], st)); CUDA_TRY(cudaEventRecord(ev[5], st)); }
		h->cur = next;
		h->slot ^= 1;
		++h->iters_done;
		return BKM_OK;
	}
	if (h->comm) {
		bkm::launch_merge_replicas(h->ws.acc, h->ws.counts, h->ws.replicas, s, st);
		Nccl* nc = nccl();
		NCCL_TRY(nc->GroupStart());
		NCCL_TRY(nc->AllReduce(h->ws.acc, h->ws.acc, kd, NCCL_FLOAT32, NCCL_SUM, h->comm, st));
		NCCL_TRY(nc->AllReduce(h->ws.counts, h->ws.counts, s.k, NCCL_UINT32, NCCL_SUM, h->comm, st));
		NCCL_TRY(nc->GroupEnd());
	}
	if (ev) CUDA_TRY(cudaEventRecord(ev[4], st));
	bkm::launch_finalize(h->ws.acc, h->ws.counts, h->comm ? 1u : h->ws.replicas, h->d_means[next], h->d_sizes, s,
		h->assign_variant == BKM_ASSIGN_SIMT ? &h->ws.sm : nullptr,
		h->assign_variant == BKM_ASSIGN_TC ? &h->ws.tm : nullptr, h->ws.ctl, h->slot ^ 1, st);
	if (ev) CUDA_TRY(cudaEventRecord(ev[5], st));
	CUDA_TRY(cudaGetLastError());
	h->cur = next;
	h->slot ^= 1;
	++h->iters_done;
	return BKM_OK;
}

static void drop_graph(bkm_handle_t h)
{
	if (h->graph_exec) { cudaGraphExecDestroy(h->graph_exec); h->graph_exec = nullptr; }
}

// Small problems are bound by launch latency: two iterations (after which the double-buffered
// means and the cmax2 slot are back where they started) are captured once into a CUDA graph and
// replayed.  The graph is rebuilt when the starting buffers differ from the captured ones.
static bool graph_wanted(bkm_handle_t h, uint32_t iters)
{
	if (h->comm || h->peer_on || iters < 4) return false;
	if (h->use_graph == 0) return false;
	// the legacy default stream (what bkm_set_stream(h, NULL) selects) and the per-thread default
	// stream cannot be captured: plain launches there
	if (h->stream == nullptr || h->stream == cudaStreamLegacy || h->stream == cudaStreamPerThread) return false;
	if (h->use_graph == 1) return true;
	return (double)h->shape.n * h->shape.k * h->shape.dim <= 1.0e8;     // auto: launch-bound sizes only
}

int bkm_run_async(bkm_handle_t h, uint32_t iters)
{
	if (!h) return fail(BKM_ERR_INVALID, "null handle");
	if (!h->initialized) return fail(BKM_ERR_STATE, "run before initialize");
	if (!h->shards.empty()) {
		// iteration by iteration over all GPUs, so that no device runs far ahead of the one whose
		// kernels this thread has not enqueued yet (their exchange kernels wait for each other)
		for (bkm_handle_s* c : h->shards) c->ev_count = 0;
		for (uint32_t it = 0; it < iters; ++it)
			for (bkm_handle_s* c : h->shards) {
				CUDA_TRY(cudaSetDevice(c->cfg.device));
				const bool timed = c->phase_timing && (iters - it) <= (uint32_t)bkm_handle_s::EV_RING;
				const int rc = enqueue_iteration(c, timed ? c->ev[c->ev_count] : nullptr);
				if (rc) return rc;
				if (timed) ++c->ev_count;
			}
		return BKM_OK;
	}
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	cudaStream_t st = h->stream;
	h->ev_count = 0;
	h->launches_per_iter = (h->assign_variant == BKM_ASSIGN_EXACT ? 1u : 2u) + 2u;
	uint32_t it = 0;
	if (graph_wanted(h, iters)) {
		// a replayed graph must hold whole iterations: a fast pass that ran behind the upload is not used
		{ const int rc0 = drop_first_pass(h); if (rc0) return rc0; }
		if (!h->graph_exec || h->graph_cur != h->cur || h->graph_slot != h->slot || h->graph_stream != st) {
			drop_graph(h);
			const int cur0 = h->cur, slot0 = h->slot;
			const uint64_t done0 = h->iters_done;
			cudaGraph_t graph = nullptr;
			CUDA_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed));
			int rc = enqueue_iteration(h, nullptr);
			if (rc == BKM_OK) rc = enqueue_iteration(h, nullptr);
			cudaError_t e = cudaStreamEndCapture(st, &graph);
			h->cur = cur0; h->slot = slot0; h->iters_done = done0;     // capturing ran nothing
			if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
			if (e != cudaSuccess) return fail(BKM_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
			e = cudaGraphInstantiate(&h->graph_exec, graph, 0);
			cudaGraphDestroy(graph);
			if (e != cudaSuccess) { h->graph_exec = nullptr; return fail(BKM_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
			h->graph_cur = cur0; h->graph_slot = slot0; h->graph_stream = st;
		}
		// the last few iterations run as plain launches so that their phases can be timed
		const uint32_t tail = h->phase_timing ? 2u : 0u;
		if (h->phase_timing) CUDA_TRY(cudaEventRecord(h->ev_run[0], st));
		for (; it + 2 + tail <= iters; it += 2) {
			CUDA_TRY(cudaGraphLaunch(h->graph_exec, st));
			h->iters_done += 2;
		}
	}
	for (; it < iters; ++it) {
		const bool timed = h->phase_timing && (iters - it) <= (uint32_t)bkm_handle_s::EV_RING;
		int rc = enqueue_iteration(h, timed ? h->ev[h->ev_count] : nullptr);
		if (rc) return rc;
		if (timed) ++h->ev_count;
	}
	return BKM_OK;
}

int bkm_synchronize(bkm_handle_t h)
{
	if (!h) return fail(BKM_ERR_INVALID, "null handle");
	if (!h->shards.empty()) {
		int first = BKM_OK;
		std::string msg;
		for (bkm_handle_s* c : h->shards) {
			const int rc = bkm_synchronize(c);
			if (rc && !first) { first = rc; msg = g_error; }
		}
		if (first) g_error = msg;
		return first;
	}
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	bkm::Control c;
	CUDA_TRY(cudaMemcpy(&c, h->ws.ctl, sizeof(c), cudaMemcpyDeviceToHost));
	if (c.status) {
		cudaMemset(&h->ws.ctl->status, 0, sizeof(uint32_t));
		return fail(BKM_ERR_DEVICE, "kernel status 0x%x (1=wait timeout, 2=assignment out of range, 4=list overflow)", c.status);
	}
	return BKM_OK;
}

int bkm_run(bkm_handle_t h, uint32_t iters)
{
	int rc = bkm_run_async(h, iters);
	if (rc) return rc;
	return bkm_synchronize(h);
}

int bkm_get_means(bkm_handle_t h, float* host_means)
{
	if (!h || !host_means) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->initialized) return fail(BKM_ERR_STATE, "no results before initialize");
	if (!h->shards.empty()) return bkm_get_means(h->shards[0], host_means);      // identical on every GPU
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaMemcpyAsync(host_means, h->d_means[h->cur], (size_t)h->shape.k * h->shape.dim * sizeof(float), cudaMemcpyDeviceToHost, h->stream));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	return BKM_OK;
}

int bkm_get_assignment(bkm_handle_t h, uint32_t* host_assignment)
{
	if (!h || !host_assignment) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->initialized) return fail(BKM_ERR_STATE, "no results before initialize");
	if (!h->shards.empty()) {
		for (size_t g = 0; g < h->shards.size(); ++g) {
			const int rc = bkm_get_assignment(h->shards[g], host_assignment + h->shard_begin[g]);
			if (rc) return rc;
		}
		return BKM_OK;
	}
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaMemcpyAsync(host_assignment, h->d_asg, h->shape.n * sizeof(uint32_t), cudaMemcpyDeviceToHost, h->stream));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	return BKM_OK;
}

int bkm_get_sizes(bkm_handle_t h, uint32_t* host_sizes)
{
	if (!h || !host_sizes) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->initialized) return fail(BKM_ERR_STATE, "no results before initialize");
	if (!h->shards.empty()) return bkm_get_sizes(h->shards[0], host_sizes);
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaMemcpyAsync(host_sizes, h->d_sizes, (size_t)h->shape.k * sizeof(uint32_t), cudaMemcpyDeviceToHost, h->stream));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	return BKM_OK;
}

int bkm_device_means(bkm_handle_t h, const float** dev_means)
{
	if (!h || !dev_means) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->shards.empty()) return bkm_device_means(h->shards[0], dev_means);
	*dev_means = h->d_means[h->cur];
	return BKM_OK;
}

int bkm_device_assignment(bkm_handle_t h, const uint32_t** dev_assignment)
{
	if (!h || !dev_assignment) return fail(BKM_ERR_INVALID, "null argument");
	NOT_FOR_GROUPS(h, "bkm_device_assignment (the assignment is spread over the GPUs)");
	*dev_assignment = h->d_asg;
	return BKM_OK;
}

int bkm_iterations_done(bkm_handle_t h, uint64_t* out)
{
	if (!h || !out) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->shards.empty()) return bkm_iterations_done(h->shards[0], out);
	*out = h->iters_done;
	return BKM_OK;
}

int bkm_phase_ms(bkm_handle_t h, float out[6])
{
	if (!h || !out) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->shards.empty()) return bkm_phase_ms(h->shards[0], out);
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	for (int p = 0; p < 6; ++p) out[p] = 0.0f;
	if (h->ev_count == 0) return BKM_OK;
	for (uint32_t i = 0; i < h->ev_count; ++i) {
		float ms = 0.0f;
		for (int p = 0; p < 5; ++p) {
			CUDA_TRY(cudaEventElapsedTime(&ms, h->ev[i][p], h->ev[i][p + 1]));
			out[p] += ms;
		}
		CUDA_TRY(cudaEventElapsedTime(&ms, h->ev[i][0], h->ev[i][5]));
		out[5] += ms;
	}
	for (int p = 0; p < 6; ++p) out[p] /= (float)h->ev_count;
	return BKM_OK;
}

int bkm_counters(bkm_handle_t h, uint64_t out[4])
{
	if (!h || !out) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->shards.empty()) {
		// kernels and variants of the first GPU; the re-checked points of all
		uint64_t total = 0;
		for (bkm_handle_s* c : h->shards) { const int rc = bkm_counters(c, out); if (rc) return rc; total += out[0]; }
		const int rc = bkm_counters(h->shards[0], out);
		out[0] = total;
		return rc;
	}
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	bkm::Control c;
	CUDA_TRY(cudaMemcpy(&c, h->ws.ctl, sizeof(c), cudaMemcpyDeviceToHost));
	out[0] = c.last_flag_count;
	out[1] = h->launches_per_iter;
	out[2] = (uint64_t)h->assign_variant;
	out[3] = h->last_fused ? (uint64_t)BKM_UPDATE_FUSED : (uint64_t)h->update_variant;
	return BKM_OK;
}

int bkm_assign_plan(bkm_handle_t h, uint32_t out[4])
{
	if (!h || !out) return fail(BKM_ERR_INVALID, "null argument");
	if (!h->shards.empty()) return bkm_assign_plan(h->shards[0], out);
	out[0] = out[1] = out[2] = out[3] = 0;
	if (h->assign_variant == BKM_ASSIGN_EXACT) out[0] = BKM_PLAN_EXACT;
	else if (h->assign_variant == BKM_ASSIGN_SIMT) out[0] = BKM_PLAN_SIMT;
	else {
		if (!h->plan) return fail(BKM_ERR_STATE, "the tensor-core plan exists after initialize only");
		bkm::tc_plan_describe(h->plan, out);
	}
	out[3] = h->last_fused ? 1u : 0u;
	return BKM_OK;
}

// ---- multi-GPU ----------------------------------------------------------------------------------

int bkm_comm_unique_id(void* id, size_t id_bytes)
{
	if (!id || id_bytes < sizeof(nccl_unique_id)) return fail(BKM_ERR_INVALID, "id buffer must hold 128 bytes");
	Nccl* nc = nccl();
	if (!nc->ok) return fail(BKM_ERR_NCCL, "libnccl.so.2 not found");
	nccl_unique_id uid;
	NCCL_TRY(nc->GetUniqueId(&uid));
	memcpy(id, &uid, sizeof(uid));
	return BKM_OK;
}

int bkm_comm_init(bkm_handle_t h, const void* id, size_t id_bytes, int world_size, int rank)
{
	if (!h || !id || id_bytes < sizeof(nccl_unique_id)) return fail(BKM_ERR_INVALID, "bad argument");
	if (world_size < 1 || rank < 0 || rank >= world_size) return fail(BKM_ERR_INVALID, "bad world_size/rank");
	NOT_FOR_GROUPS(h, "bkm_comm_init");
	if (h->comm) return fail(BKM_ERR_STATE, "communicator already initialised");
	Nccl* nc = nccl();
	if (!nc->ok) return fail(BKM_ERR_NCCL, "libnccl.so.2 not found");
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	nccl_unique_id uid;
	memcpy(&uid, id, sizeof(uid));
	NCCL_TRY(nc->CommInitRank(&h->comm, world_size, uid, rank));
	h->world = world_size;
	h->rank = rank;
	return BKM_OK;
}

// ---- peer-memory exchange -------------------------------------------------------------------------

namespace {

struct PeerBlob {                 // what one rank tells the others about its exchange buffer
	cudaIpcMemHandle_t handle;    // 64 bytes
	uint32_t k, dim;
	uint64_t bytes;
	uint32_t magic;
	uint32_t pad[11];
};
static_assert(sizeof(PeerBlob) == BKM_PEER_BLOB_BYTES, "blob size is part of the ABI");
constexpr uint32_t PEER_MAGIC = 0x626b6d78u;

int own_exchange_buffer(bkm_handle_t h)
{
	NOT_FOR_GROUPS(h, "the peer exchange of a single shard");
	if (h->d_xbuf) return BKM_OK;
	if ((uint64_t)h->shape.k * h->shape.dim + h->shape.k > bkm::EXCHANGE_MAX_WORDS)
		return fail(BKM_ERR_UNSUPPORTED, "k*dim + k = %llu exceeds the %llu words the peer exchange is meant for (use the NCCL all-reduce)",
			(unsigned long long)h->shape.k * h->shape.dim + h->shape.k, (unsigned long long)bkm::EXCHANGE_MAX_WORDS);
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	const size_t bytes = bkm::exchange_buffer_bytes(h->shape.k, h->shape.dim);
	CUDA_TRY(cudaMalloc(&h->d_xbuf, bytes));
	CUDA_TRY(cudaMemset(h->d_xbuf, 0, bytes));
	return BKM_OK;
}

} // namespace

int bkm_peer_layout(uint32_t k, uint32_t dim, uint64_t out[4])
{
	if (!out || k == 0 || dim == 0) return fail(BKM_ERR_INVALID, "bad argument");
	out[0] = bkm::exchange_buffer_bytes(k, dim);
	out[1] = bkm::exchange_slot_words(k, dim);                          // packets per sender
	out[2] = bkm::EXCHANGE_MAX_RANKS;                                    // senders per slot
	out[3] = (uint64_t)bkm::EXCHANGE_MAX_RANKS * bkm::exchange_slot_words(k, dim) * sizeof(uint64_t);   // bytes per slot
	return BKM_OK;
}

int bkm_peer_buffer(bkm_handle_t h, void** base, size_t* bytes)
{
	if (!h || !base) return fail(BKM_ERR_INVALID, "null argument");
	int rc = own_exchange_buffer(h);
	if (rc) return rc;
	*base = h->d_xbuf;
	if (bytes) *bytes = bkm::exchange_buffer_bytes(h->shape.k, h->shape.dim);
	return BKM_OK;
}

int bkm_peer_export(bkm_handle_t h, void* blob, size_t blob_bytes)
{
	if (!h || !blob || blob_bytes < sizeof(PeerBlob)) return fail(BKM_ERR_INVALID, "blob buffer must hold %d bytes", (int)BKM_PEER_BLOB_BYTES);
	int rc = own_exchange_buffer(h);
	if (rc) return rc;
	PeerBlob b;
	memset(&b, 0, sizeof(b));
	CUDA_TRY(cudaIpcGetMemHandle(&b.handle, h->d_xbuf));
	b.k = h->shape.k; b.dim = h->shape.dim;
	b.bytes = bkm::exchange_buffer_bytes(h->shape.k, h->shape.dim);
	b.magic = PEER_MAGIC;
	memcpy(blob, &b, sizeof(b));
	return BKM_OK;
}

static int peer_world_check(bkm_handle_t h, int world_size, int rank)
{
	if (world_size < 2 || world_size > (int)bkm::EXCHANGE_MAX_RANKS || rank < 0 || rank >= world_size)
		return fail(BKM_ERR_UNSUPPORTED, "the peer exchange handles 2..%d ranks (world_size=%d rank=%d)", (int)bkm::EXCHANGE_MAX_RANKS, world_size, rank);
	if (h->comm && (h->world != world_size || h->rank != rank))
		return fail(BKM_ERR_INVALID, "world_size/rank differ from the NCCL communicator's");
	if (h->peer_world) return fail(BKM_ERR_STATE, "peer buffers already attached");
	return BKM_OK;
}

int bkm_peer_open(bkm_handle_t h, const void* blobs, size_t blob_bytes, int world_size, int rank)
{
	if (!h || !blobs || blob_bytes != sizeof(PeerBlob)) return fail(BKM_ERR_INVALID, "bad argument");
	int rc = peer_world_check(h, world_size, rank);
	if (rc) return rc;
	if ((rc = own_exchange_buffer(h))) return rc;
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	const char* p = static_cast<const char*>(blobs);
	for (int r = 0; r < world_size; ++r) {
		PeerBlob b;
		memcpy(&b, p + (size_t)r * sizeof(PeerBlob), sizeof(b));
		if (b.magic != PEER_MAGIC || b.k != h->shape.k || b.dim != h->shape.dim)
			return fail(BKM_ERR_INVALID, "rank %d exports an exchange buffer for another problem (k=%u dim=%u)", r, b.k, b.dim);
		if (r == rank) { h->peer_base[r] = h->d_xbuf; continue; }
		void* ptr = nullptr;
		cudaError_t e = cudaIpcOpenMemHandle(&ptr, b.handle, cudaIpcMemLazyEnablePeerAccess);
		if (e != cudaSuccess) {
			cudaGetLastError();
			for (int q = 0; q < r; ++q) if (h->peer_ipc[q]) { cudaIpcCloseMemHandle(h->peer_base[q]); h->peer_ipc[q] = false; h->peer_base[q] = nullptr; }
			return fail(BKM_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d: %s", r, cudaGetErrorString(e));
		}
		h->peer_base[r] = ptr;
		h->peer_ipc[r] = true;
	}
	h->peer_world = world_size;
	h->world = world_size;
	h->rank = rank;
	return BKM_OK;
}

int bkm_peer_attach(bkm_handle_t h, void* const* bases, int world_size, int rank)
{
	if (!h || !bases) return fail(BKM_ERR_INVALID, "null argument");
	int rc = peer_world_check(h, world_size, rank);
	if (rc) return rc;
	if ((rc = own_exchange_buffer(h))) return rc;
	for (int r = 0; r < world_size; ++r) {
		if (r != rank && !bases[r]) return fail(BKM_ERR_INVALID, "buffer of rank %d is null", r);
		h->peer_base[r] = r == rank ? h->d_xbuf : bases[r];
	}
	h->peer_world = world_size;
	h->world = world_size;
	h->rank = rank;
	return BKM_OK;
}

int bkm_peer_enable(bkm_handle_t h, int enable)
{
	if (!h) return fail(BKM_ERR_INVALID, "null handle");
	NOT_FOR_GROUPS(h, "bkm_peer_enable");
	if (enable && !h->peer_world) return fail(BKM_ERR_STATE, "no peer buffers attached (bkm_peer_open / bkm_peer_attach first)");
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	h->peer_on = enable != 0;
	drop_graph(h);
	return BKM_OK;
}

int bkm_run_ready(bkm_handle_t h)
{
	if (!h) return fail(BKM_ERR_INVALID, "null handle");
	if (!h->initialized) return fail(BKM_ERR_STATE, "not initialized");
	if (!h->shards.empty()) {
		for (bkm_handle_s* c : h->shards) { const int rc = bkm_run_ready(c); if (rc) return rc; }
		return BKM_OK;
	}
	if (h->assign_variant == BKM_ASSIGN_TC && !h->plan) return fail(BKM_ERR_STATE, "the tensor-core plan is missing");
	CUDA_TRY(cudaSetDevice(h->cfg.device));
	bkm::Control c;
	CUDA_TRY(cudaStreamSynchronize(h->stream));
	CUDA_TRY(cudaMemcpy(&c, h->ws.ctl, sizeof(c), cudaMemcpyDeviceToHost));
	if (c.status) return fail(BKM_ERR_DEVICE, "kernel status 0x%x is pending", c.status);
	return BKM_OK;
}

// ---- host-buffer convenience ----------------------------------------------------------------------

int bkm_kmeans_host_f32(const float* host_points, float* means, uint32_t* assignment,
	uint64_t n, uint32_t k, uint32_t dim, uint32_t iters, int layout, int layout_means, int device)
{
	if (!host_points || !means || !assignment) return fail(BKM_ERR_INVALID, "null argument");
	bkm_config_t cfg{};
	cfg.n = n; cfg.k = k; cfg.dim = dim; cfg.layout = layout; cfg.layout_means = layout_means; cfg.device = device;
	bkm_handle_t h = nullptr;
	int rc = bkm_create(&cfg, &h);
	if (rc) return rc;
	if ((rc = bkm_initialize(h, host_points, means)) == BKM_OK &&
		(rc = bkm_run(h, iters)) == BKM_OK &&
		(rc = bkm_get_means(h, means)) == BKM_OK)
		rc = bkm_get_assignment(h, assignment);
	std::string keep = g_error;
	bkm_destroy(h);
	g_error = keep;
	return rc;
}

} // extern "C"
