// Internal launch interface between the host driver (api.cu) and the kernel files.
#pragma once

#include "common.cuh"

namespace bkm {

struct Shape {
	uint64_t n;     // local points
	uint32_t k;
	uint32_t dim;
	int soa;        // points layout is SoA
	int soa_means;  // means layout is SoA
};

// Operands of the tensor-core assignment derived from the means (rewritten every iteration).
struct TcMeans {
	float* b_hi;     // [k_pad][d_pad] tf32 high part of -2*mean, K-major
	float* b_lo;     // [k_pad][d_pad] tf32 low part
	float* cnorm;    // [k_pad] |mean|^2, +inf for padding rows
	float* b_aug;    // [k_pad x 8] one K step (aug_offset layout): columns 0,1 = tf32 (hi, lo) of |mean|^2,
	                 // columns 2,3 = 1 (they meet the kernel's offset constant), rest 0; padding rows 0,0,1,1
	float* center;   // [d_pad] vector subtracted from points and means alike before the split (distances do
	                 // not change; the norms, and with them the cancellation of the GEMM form, shrink)
	uint32_t k_pad;  // k rounded up to the centroid tile
	uint32_t d_pad;  // dim rounded up to TC_KCHUNK
};

// Operand of the CUDA-core fast pass derived from the means (rewritten every iteration).
struct SimtMeans {
	float* rows;          // [simt_rows(k)][simt_row_stride(dim)]: |c - centre|^2, -2(c - centre), zero padding; +inf marks a padding row
	const float* center;  // [dim] the vector subtracted from points and means alike (as for the tensor-core operands)
};

// Operands derived from the points (written once per initialize).
struct TcPoints {
	float* a_hi;     // [n_pad][d_pad]
	float* a_lo;     // [n_pad][d_pad]
	float* xnorm;    // [n_pad] |x|^2
	uint64_t n_pad;  // n rounded up to TC_MTILE
	uint32_t d_pad;
	uint32_t* partial; // K loop only (d_pad > 32): [TC_JSPLIT][3][n_pad] partial arg-min keys, else null
};
constexpr uint32_t TC_JSPLIT = 2;   // CTAs that can share the mean tiles of one point block in the K loop

// SM count of the current device (cached per device ordinal; 1 if the query fails).
int current_sm_count();

// ---- means preparation + divide (update.cu) ----

// means (given layout) -> CUDA-core rows and/or tensor-core operands; cmax2 -> ctl slot.
// `sm` / `tc` may be null.  Also clears flag_count.
// `slot` is the cmax2 slot to fill (it must be zero on entry).
void launch_prepare_means(const float* means, const Shape& s, const SimtMeans* sm, const TcMeans* tc,
	Control* ctl, int slot, cudaStream_t stream);

// acc/counts -> means_out (given layout), sizes_out, then the same preparation as above from
// the fresh means; clears acc, counts and flag_count for the next iteration.
void launch_finalize(float* acc, uint32_t* counts, uint32_t replicas, float* means_out, uint32_t* sizes_out, const Shape& s,
	const SimtMeans* sm, const TcMeans* tc, Control* ctl, int slot, cudaStream_t stream);

// ---- exchange between ranks (update.cu) ----
// Every rank owns a receive buffer of exchange_buffer_bytes(k, dim) that all ranks can write: two
// slots x EXCHANGE_MAX_RANKS senders x exchange_slot_words 8-byte packets (k*dim float sums, then
// k sizes; value in the low half of a packet, iteration count in the high half).
constexpr uint32_t EXCHANGE_MAX_RANKS = 8;
constexpr uint64_t EXCHANGE_MAX_WORDS = 1ull << 19;     // larger sum sets are a bandwidth problem: NCCL's job
__host__ __device__ __forceinline__ size_t exchange_slot_words(uint32_t k, uint32_t dim) { return ((size_t)k * dim + k + 63) / 64 * 64; }
size_t exchange_buffer_bytes(uint32_t k, uint32_t dim);
// One kernel instead of merge + all-reduce + finalize: sends this rank's sums and sizes to every
// rank's receive buffer, waits (at most wait_limit_ns) for all senders' packets in its own, adds
// them in rank order, divides and prepares the next operands.  `peer_bases[r]` = receive buffer of
// rank r as addressable from this device (own buffer at [rank]); `epoch` grows by one per call on
// every rank, starting at 1.
cudaError_t launch_exchange_finalize(float* acc, uint32_t* counts, uint32_t replicas, void* const* peer_bases, uint32_t world,
	uint32_t rank, uint32_t epoch, uint64_t wait_limit_ns, float* means_out, uint32_t* sizes_out, const Shape& s,
	const SimtMeans* sm, const TcMeans* tc, Control* ctl, int slot, cudaStream_t stream);

// acc/counts -> sums_out in the means layout of `s`, NOT divided (the bucketing study's result); clears acc and counts.
void launch_finalize_sums(float* acc, uint32_t* counts, uint32_t replicas, float* sums_out, const Shape& s, Control* ctl, cudaStream_t stream);
// Write-only atomic-add probe: n*dim additions of 0.1 into result[(i / dim) % k][i % dim] (result layout `soa`).
cudaError_t launch_probe_atomics(float* result, uint64_t n, uint32_t k, uint32_t dim, int soa, bool shared_cache, uint32_t items_per_thread,
	cudaStream_t stream);

// ---- recognising the point set of a stateless call (update.cu) ----
// Adds a fingerprint of the points (every 16th 128-byte line and the last one; order-independent
// sum of mixed (value, position) words) to key->fp_new, which must be zero on entry.
cudaError_t launch_points_fingerprint(const float* pts, uint64_t words, PointsKey* key, int sm_count, cudaStream_t stream);
// Sets key->valid (same address, shape, variant and fingerprint as remembered) and remembers the
// current call's; when the points are new it also clears ctl->xmax2, which their preprocessing refills.
cudaError_t launch_points_key_decide(PointsKey* key, const float* pts, const Shape& s, int variant, Control* ctl, cudaStream_t stream);

// ---- update (update.cu) ----
// variant: BKM_UPDATE_SHARED or BKM_UPDATE_GLOBAL (already resolved).  acc/counts must be zero.
// Returns false when the shared variant cannot hold k*dim in shared memory.
bool update_shared_fits(const Shape& s, int device);
bool update_sorted_supported(const Shape& s);
void launch_update(const float* pts, const uint32_t* asg, float* acc, uint32_t* counts, uint32_t replicas, const Shape& s,
	int variant, Control* ctl, int sm_count, cudaStream_t stream);
// Folds accumulator replicas 1.. into replica 0 (before an all-reduce of replica 0).
void launch_merge_replicas(float* acc, uint32_t* counts, uint32_t replicas, const Shape& s, cudaStream_t stream);

// ---- assignment on CUDA cores (assign_simt.cu) ----
// Exact reference arithmetic.  With list != null only the points list[0..*list_count) are done.
// With `fix` set (list form only) the kernel also moves every point whose cluster changed from
// its old cluster's sum and size to the new one's - the correction that goes with an assignment
// pass which has already accumulated the update sums (FusedAcc below).
struct FusedAcc {
	float* acc;           // [replicas][k*dim sums | k sizes], replica stride in 32-bit words
	uint32_t* counts;
	uint32_t replicas;
	size_t rep_stride;
	const float* center;  // the vector the split operands were centred by
};
// `split_scratch` (optional): list_split_scratch_bytes() of zeroed device memory, 8-byte aligned,
// through which the blocks share the groups of a short list; the kernel leaves it zeroed.
size_t list_split_scratch_bytes();
cudaError_t launch_assign_exact(const float* pts, const float* means, uint32_t* asg, const Shape& s,
	const uint32_t* list, const uint32_t* list_count, int sm_count, cudaStream_t stream, const FusedAcc* fix = nullptr,
	void* split_scratch = nullptr);

// Small-d fast pass (dim <= 8): approximate distances, near-ties appended to flag_list.
bool assign_simt_supported(const Shape& s);
// max |x - center|^2 over the points -> ctl->xmax2 (zero on entry); once per data set.
// `skip_if` (optional, device): the kernels of the one-off preprocessing return at once when *skip_if != 0.
cudaError_t launch_points_norm_max(const float* pts, const Shape& s, const float* center, Control* ctl, int sm_count, cudaStream_t stream,
	const uint32_t* skip_if = nullptr);
// With `fused` set (allowed when assign_simt_can_fuse) the kernel also adds every point to the sum and
// the size of the cluster it picked; points that the exact re-check moves afterwards are corrected there.
bool assign_simt_can_fuse(const Shape& s, const FusedAcc& f);
cudaError_t launch_assign_simt(const float* pts, const SimtMeans& sm, uint32_t* asg, const Shape& s,
	Control* ctl, int slot, uint32_t* flag_list, float margin_scale, int sm_count, cudaStream_t stream, const FusedAcc* fused = nullptr);

// ---- assignment on tensor cores (assign_tc.cu) ----
bool assign_tc_supported(const Shape& s);
uint32_t tc_kpad(uint32_t k);
// One-off split of the points into tf32 hi/lo K-major planes + |x|^2.
// `p_begin`, `p_end` (multiples of 32; 0, 0 = all): only these rows of the planes, so that a host upload
// can be split chunk by chunk while the next chunk is on its way.
cudaError_t launch_split_points(const float* pts, const Shape& s, const TcPoints& tp, const float* center, Control* ctl, cudaStream_t stream,
	const uint32_t* skip_if = nullptr, uint64_t p_begin = 0, uint64_t p_end = 0);
// center[j] = mean of dimension j over a strided sample of the points (any vector would do; the
// sample mean keeps the shifted norms small).
// `n_sampled` (0 = all): the sample is taken from the first n_sampled points only.
cudaError_t launch_compute_center(const float* pts, const Shape& s, float* center, cudaStream_t stream, const uint32_t* skip_if = nullptr,
	uint64_t n_sampled = 0);
// Opaque per-handle state (tensor maps).  Created once the operand buffers exist.
struct TcPlan;
TcPlan* tc_plan_create(const Shape& s, const TcPoints& tp, const TcMeans& tm, int device, const char** err);
void tc_plan_destroy(TcPlan* plan);
// The CTA-pair kernel (means resident in shared memory) is used where it applies unless disallowed.
void tc_plan_allow_pair(TcPlan* plan, bool allow);
bool tc_plan_uses_pair(const TcPlan* plan);
// With `fused` set (allowed when tc_plan_can_fuse) the kernel also adds every point to the sum and
// the size of the cluster it picked, so that no separate update pass is needed; points that the
// exact re-check moves afterwards are corrected there.
bool tc_plan_can_fuse(const TcPlan* plan, const FusedAcc& f);
// out[0] = BKM_PLAN_* code of the kernel the plan launches, out[1] = mean tiles, out[2] = CTAs that
// share one point block (1 = no split; > 1 implies the partial-result merge kernel).
void tc_plan_describe(const TcPlan* plan, uint32_t out[4]);
// `p_begin`, `p_end` (0, 0 = all; CTA-pair plans only; p_begin a multiple of 256, p_end too unless it is
// the last point): only these points, so that the pass can follow a host upload chunk by chunk.
cudaError_t launch_assign_tc(TcPlan* plan, uint32_t* asg, Control* ctl, int slot, uint32_t* flag_list,
	float margin_scale, cudaStream_t stream, const FusedAcc* fused = nullptr, uint64_t p_begin = 0, uint64_t p_end = 0);

// A wait that is made to run out (nothing ever arrives): sets STATUS_WAIT_TIMEOUT in `ctl` after `limit_ns`.
cudaError_t launch_wait_timeout_selftest(Control* ctl, uint64_t limit_ns, cudaStream_t stream);

} // namespace bkm
