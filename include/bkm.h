/*
 * bkm.h - C ABI of the B200 k-means iteration library (libbkm.so).
 *
 * The library implements one Lloyd iteration (nearest-centroid assignment + bucketed
 * sum/count update + divide) and the fixed-iteration loop around it, in fp32, on NVIDIA
 * B200 (sm_100a).  It is the drop-in for the per-iteration hot path of
 * krulis-martin/cuda-kmeans; each entry point names the reference interface it replaces
 * (paths relative to experimental/k-means/k-means/ of that project).
 *
 * Conventions
 *   - Every function returns BKM_OK (0) or an error code; bkm_last_error() then returns a
 *     thread-local, human-readable message.  No exception crosses this boundary.
 *   - Layout codes follow the reference's layout policies with ALIGN = 1
 *     (headers/layout_policies.hpp:16-36, 40-60):
 *       BKM_LAYOUT_AOS: element (item i, dimension j) at  p[i*dim + j]
 *       BKM_LAYOUT_SOA: element (item i, dimension j) at  p[j*items + i]
 *     where items = n for points and items = k for means.
 *   - Nearest means the smallest Euclidean distance as the reference's serial code computes
 *     it (headers/serial.hpp:21-35): the lowest index wins exact ties.
 *   - An empty cluster gets the all-zero mean (headers/serial.hpp:49-54, 66-67).
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails with
 *     BKM_ERR_CUDA.
 */
#ifndef BKM_H
#define BKM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BKM_OK 0
#define BKM_ERR_INVALID 1      /* bad argument (null pointer, zero size, unknown code) */
#define BKM_ERR_CUDA 2         /* a CUDA runtime/driver call failed, or no device */
#define BKM_ERR_NCCL 3         /* NCCL missing or a NCCL call failed */
#define BKM_ERR_UNSUPPORTED 4  /* shape outside what the selected variant handles */
#define BKM_ERR_STATE 5        /* call order violated (e.g. run before initialize) */
#define BKM_ERR_DEVICE 6       /* a kernel reported an internal error (bounded wait ran out) */

#define BKM_LAYOUT_AOS 0
#define BKM_LAYOUT_SOA 1

/* Assignment variants (the counterpart of choosing ASGN_KERNEL in headers/cuda.hpp:15-19). */
#define BKM_ASSIGN_AUTO 0   /* pick by shape */
#define BKM_ASSIGN_EXACT 1  /* CUDA cores, reference arithmetic for every point (any shape) */
#define BKM_ASSIGN_SIMT 2   /* CUDA cores, small-d fast path (dim <= 8), near-ties re-checked exactly */
#define BKM_ASSIGN_TC 3     /* tcgen05 tensor cores, split-TF32 GEMM form, near-ties re-checked exactly */

/* Update variants (the counterpart of choosing UPDATE_KERNEL). */
#define BKM_UPDATE_AUTO 0
#define BKM_UPDATE_SHARED 1  /* shared-memory privatised buckets + one global merge */
#define BKM_UPDATE_GLOBAL 2  /* global atomics only (any k*dim) */
#define BKM_UPDATE_ROWS 3    /* one coalesced 128-byte global reduction per point and 32 dimensions */
#define BKM_UPDATE_FUSED 4   /* reported by bkm_counters only: the assignment pass accumulated the sums itself */
#define BKM_UPDATE_SORTED 5  /* block-local counting sort by cluster, one reduction per cluster and 2048 points (k <= 1024) */

const char* bkm_last_error(void);

/* Library version: major*10000 + minor*100 + patch. */
int bkm_version(void);

/* Number of visible CUDA devices (0 without a GPU; never fails). */
int bkm_device_count(void);

/* ------------------------------------------------------------------------------------------
 * Kernel-runner entry points: device pointers in, device pointers out, stream-ordered, no
 * device allocation.  `workspace` is device scratch of at least bkm_workspace_bytes(n,k,dim)
 * bytes, 256-byte aligned, owned by the caller; it may hold anything on the first call.
 * `stream` is a cudaStream_t (NULL = legacy default stream, which is what the reference's
 * runners launch on, kernels/kernels.cu:201-207).
 *
 * The reference's drivers call their runners once per iteration on the same, immutable points
 * (headers/cuda.hpp:70-88).  bkm_assign_f32 and bkm_iterate_f32 therefore leave what they derive
 * from the points alone (a centre vector, the largest norm, tf32 operand planes) in the
 * workspace, and a later call on the same workspace skips that work when it finds the same
 * points: same address, shape and variant, and the same fingerprint of a sample of the values
 * (every 16th 128-byte line and the last).  New data at the same address is therefore noticed;
 * a caller that rewrites single coordinates in place, or scribbles over the workspace while
 * keeping its first 256 bytes, must clear those 256 bytes before the next call.
 * ------------------------------------------------------------------------------------------ */

/* Scratch size for the three calls below (0 on overflow or bad arguments). */
size_t bkm_workspace_bytes(uint64_t n, uint32_t k, uint32_t dim);

/* assignment[i] = index of the mean nearest to point i.
 * Replaces ASGN_KERNEL::run(const AssignmentProblemInstance<F,IDX_T>&, CudaExecParameters&)
 * (headers/kernels.cuh:8-20, 81-93; runners kernels/kernels.cu:201-207, 297-319, 688-717). */
int bkm_assign_f32(const float* points, const float* means, uint32_t* assignment,
                   uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means,
                   int variant, void* workspace, size_t workspace_bytes, void* stream);

/* means[c][:] = average of the points with assignment c, sizes[c] = their number.  The
 * outputs are fully overwritten (the caller need not zero them, and may).
 * Replaces UPDATE_KERNEL::run(const UpdateProblemInstance<F,IDX_T>&, CudaExecParameters&)
 * including its trailing merge and divide (headers/kernels.cuh:24-36, 96-105; runners
 * kernels/kernels.cu:746-761, 794-809, 861-878). */
int bkm_update_f32(const float* points, const uint32_t* assignment, float* means, uint32_t* sizes,
                   uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means,
                   int variant, void* workspace, size_t workspace_bytes, void* stream);

/* The update step of the reference's separate bucketing study: sums[c][:] = SUM of the points with
 * index c - no sizes, no divide - with `sums` in the same layout as the points (items = k) and
 * fully overwritten.  Replaces KERNEL::run(const ProblemInstance<F>&, CudaExecParameters&) there
 * (experimental/bucketing-cuda/bucketing-cuda/headers/kernels.cuh; runners kernels/kernels.cu:
 * 180-186, 214-226, 254-266, 296-308, 357-372, 425-444 incl. their trailing reducePrivCopies).
 * `variant` is a BKM_UPDATE_* code, workspace as above. */
int bkm_bucket_sums_f32(const float* points, const uint32_t* indices, float* sums,
                        uint64_t n, uint32_t k, uint32_t dim, int layout, int variant,
                        void* workspace, size_t workspace_bytes, void* stream);

/* Write-only probe of the atomic-add throughput: n*dim additions of the constant 0.1, value i going
 * to result[(i / dim) % k][i % dim], nothing read; `result` (k*dim floats in `layout`) is added to,
 * not cleared.  shared_cache != 0 keeps the first buckets (as many as fit 96 KiB) in shared memory
 * and flushes them per block.  Replaces AtomicFakeKernel::run / AtomicShmFakeKernel::run of the
 * bucketing study (kernels/kernels.cu:455-486, 496-549); items_per_thread as in their runners. */
int bkm_probe_atomics_f32(float* result, uint64_t n, uint32_t k, uint32_t dim, int layout,
                          int shared_cache, uint32_t items_per_thread, void* stream);

/* One whole iteration: means_out/sizes from means_in.  `assignment` may be NULL when the
 * caller does not want it, as in the reference's fused runners.  The points are read once, as in
 * those runners, where the assignment pass can add up the sums itself (dim <= 8 with at most 1024
 * means; 257..1024 means of 17..32 dimensions, dim % 4 == 0, dimension-major points); elsewhere
 * the assignment pass is followed by the update pass.
 * Replaces KERNEL::run(const FusedProblemInstance<F,IDX_T>&, CudaExecParameters&)
 * (headers/kernels.cuh:40-52, 108-116; runners kernels/kernels.cu:951-998, 1146-1190). */
int bkm_iterate_f32(const float* points, const float* means_in, float* means_out, uint32_t* sizes,
                    uint32_t* assignment, uint64_t n, uint32_t k, uint32_t dim, int layout,
                    int layout_means, int variant_assign, int variant_update,
                    void* workspace, size_t workspace_bytes, void* stream);

/* The update step without any scratch from the caller and without any allocation inside.
 * (No counterpart in the reference: its update runners get their extra copies from the
 * algorithm class that owns all buffers, headers/cuda.hpp:25-28, 161.)
 *
 * Who needs it: a runner plugged into the reference's harness is handed only the problem
 * instance - data, assignment, means, clusterSizes - with no room for a workspace pointer, and
 * it runs inside the timed iteration loop, where a cudaMalloc would stall the whole device;
 * likewise an application that has already given all device memory to its own pool, or that
 * has filled the GPU with point data, has nothing left for cudaMalloc to return.  For such
 * callers the accumulators of this entry point live in a fixed array inside the library
 * image: BKM_NOALLOC_SCRATCH_WORDS 32-bit words (2 MiB) on every GPU that loads the library,
 * held until the process exits whether or not the call is ever used.
 *
 * Limit: k*dim + k <= BKM_NOALLOC_MAX_WORDS, otherwise BKM_ERR_UNSUPPORTED (use
 * bkm_update_f32 with a workspace of your own).  Results are those of bkm_update_f32.
 *
 * The first call on each device looks up the device address of the array (a host-side
 * set-up step, done with that device current); make that first call outside any stream
 * capture.  All calls on a device share the one array and each call clears what it
 * accumulates into, so two calls whose kernels overlap on the GPU (different streams, or
 * different host threads on different streams) race on it: keep calls on one device ordered.
 * Nothing else of the library touches the array. */
#define BKM_NOALLOC_SCRATCH_WORDS (512u * 1024u)
#define BKM_NOALLOC_MAX_WORDS (BKM_NOALLOC_SCRATCH_WORDS - 128u)
int bkm_update_noalloc_f32(const float* points, const uint32_t* assignment, float* means, uint32_t* sizes,
                           uint64_t n, uint32_t k, uint32_t dim, int layout, int layout_means, void* stream);

/* The bkm_workspace_check of bkm_update_noalloc_f32 (likewise without a counterpart in the
 * reference): waits for `stream` and returns BKM_ERR_DEVICE if the last such call on the current
 * device met an assignment value >= k (the point is then left out of sums and sizes).  Allocates
 * nothing; reads the status word at the head of the built-in array. */
int bkm_noalloc_check(void* stream);

/* Waits for `stream` and returns BKM_ERR_DEVICE if a kernel of the calls issued on this
 * workspace since its last check recorded an error (a bounded wait that ran out, an assignment
 * value >= k fed to the update).  The counterpart of the reference's CUCH(cudaGetLastError())
 * after each runner (headers/cuda.hpp:76, 83). */
int bkm_workspace_check(const void* workspace, void* stream);

/* Self-test of the kernels' bounded waits (no counterpart in the reference, whose kernels have no
 * waits): enqueues a one-thread kernel that waits limit_ms (1..1000) milliseconds for a barrier
 * nobody arrives on, gives up, and records the "wait timeout" status bit in the control block at
 * the start of `workspace` (at least 256 bytes of device memory) - the path an assignment kernel
 * takes when a pipeline stage never delivers.  Nothing hangs and the context stays usable;
 * bkm_workspace_check then reports BKM_ERR_DEVICE.  Clear the first 32 bytes of the workspace (or
 * pass it to a stateless call, which does) before reusing it. */
int bkm_selftest_wait_timeout(void* workspace, uint32_t limit_ms, void* stream);

/* ------------------------------------------------------------------------------------------
 * Fixed-iteration driver.  Replaces CudaKMeansAlgorithm (headers/cuda.hpp:19-112) behind the
 * IKMeansAlgorithm call sequence initialize / run / getMeans / getAssignment / cleanup
 * (headers/interface.hpp:8-49).  One handle drives one GPU, or (config.num_gpus) several from one
 * process; with one process per GPU (bkm_comm_init) every rank holds a contiguous shard of the
 * points and the per-iteration sums and sizes are exchanged between the ranks before the divide.
 * ------------------------------------------------------------------------------------------ */

typedef struct bkm_handle_s* bkm_handle_t;

typedef struct bkm_config_s {
	uint64_t n;            /* points held by THIS handle (the local shard) */
	uint32_t k;            /* clusters */
	uint32_t dim;          /* dimensions */
	int32_t layout;        /* BKM_LAYOUT_* of the points (local shard: items = n) */
	int32_t layout_means;  /* BKM_LAYOUT_* of the means */
	int32_t device;        /* CUDA device ordinal */
	int32_t variant_assign;/* BKM_ASSIGN_* */
	int32_t variant_update;/* BKM_UPDATE_* */
	int32_t num_gpus;      /* 0 or 1: this handle drives GPU `device`.  G = 2..8: ONE process drives the GPUs
	                          device .. device+G-1 through this handle: n is then the TOTAL number of points,
	                          split into contiguous shards (bkm_shard_range), and every iteration's sums and
	                          sizes cross between the GPUs through the peer-memory exchange (all pairs of the
	                          devices must have peer access, k*dim + k <= 2^19).  bkm_initialize takes the
	                          whole host array; results come back whole.  Not available on such a handle:
	                          bkm_initialize_device, bkm_set_stream, bkm_device_assignment, bkm_comm_init.
	                          The reference drives device 0 only (headers/cuda.hpp:53). */
} bkm_config_t;

/* Allocates the device state for the configuration (no data yet). */
int bkm_create(const bkm_config_t* config, bkm_handle_t* out);

/* Frees everything the handle owns (cleanup(), headers/cuda.hpp:102-111). */
int bkm_destroy(bkm_handle_t h);

/* Makes all work of the handle run on `stream` (a cudaStream_t of the handle's device)
 * instead of the non-blocking stream the handle created for itself.  NULL selects the legacy
 * default stream, the one the reference's drivers use (headers/cuda.hpp:70-88). */
int bkm_set_stream(bkm_handle_t h, void* stream);

/* Tunables: "margin_scale" (multiplier on the near-tie band, default 1), "phase_timing"
 * (0/1: record per-phase CUDA events for the last 8 iterations of a run, default 1; they cost
 * 2-5 % of those iterations), "use_graph" (0 never, 1 always, 2 = default:
 * replay a CUDA graph of two iterations when the problem is small enough to be bound by launch
 * latency; single GPU only), "tc_pair" (0/1, default 1: let the tensor-core assignment run on CTA
 * pairs with all means resident in shared memory where the shape allows, i.e. 257..1024 means
 * of 17..32 dimensions), "fuse_update" (0 never, 1 = default: where it pays, 2 wherever possible:
 * let the fast assignment pass add every point to the sum of the cluster it picks, which replaces
 * the update pass of bkm_run; possible on CTA pairs with dim % 4 == 0 and in the CUDA-core pass
 * for dim <= 8 and at most 1024 means; by default the latter only for launch-bound sizes),
 * "exchange_wait_ms" (1..600000, default 2000: how long the peer-memory exchange waits for a peer).
 * Unknown names fail with BKM_ERR_INVALID. */
int bkm_set_option(bkm_handle_t h, const char* name, double value);

/* initialize(): copies points and initial means from HOST memory, runs the one-off
 * preprocessing of the immutable points, resets the iteration state
 * (headers/cuda.hpp:45-68).  Synchronous.  Points of 32 MB and more on the tensor-core path
 * travel in eight chunks (fastest from pinned memory); each chunk is preprocessed while the
 * next is on its way, and where the assignment runs on CTA pairs the fast pass of the first
 * iteration follows the chunks as well, so that the first bkm_run starts at its re-check
 * (bkm_set_means or a changed option before that run discards the early pass). */
int bkm_initialize(bkm_handle_t h, const float* host_points, const float* host_means);

/* Same with DEVICE pointers.  The points are borrowed, not copied: they must stay valid and
 * unchanged until the next initialize or destroy.  The means are copied. */
int bkm_initialize_device(bkm_handle_t h, const float* dev_points, const float* dev_means);

/* run(): `iters` iterations of assign -> update (-> all-reduce) -> divide, then one
 * synchronisation, like headers/cuda.hpp:70-88.  Iterations continue from the current
 * means, so run(a) followed by run(b) equals run(a+b). */
int bkm_run(bkm_handle_t h, uint32_t iters);

/* As bkm_run without the final synchronisation (enqueue only). */
int bkm_run_async(bkm_handle_t h, uint32_t iters);

/* Waits for the handle's stream and reports any error a kernel recorded. */
int bkm_synchronize(bkm_handle_t h);

/* getMeans()/getAssignment(): results of the last completed iteration to HOST memory
 * (headers/cuda.hpp:90-100).  The assignment is the one computed in the last iteration,
 * i.e. against the means of the iteration before.  Sizes are the (global) cluster sizes. */
int bkm_get_means(bkm_handle_t h, float* host_means);
int bkm_get_assignment(bkm_handle_t h, uint32_t* host_assignment);
int bkm_get_sizes(bkm_handle_t h, uint32_t* host_sizes);

/* Device pointers of the same results (valid until the next run/initialize/destroy). */
int bkm_device_means(bkm_handle_t h, const float** dev_means);
int bkm_device_assignment(bkm_handle_t h, const uint32_t** dev_assignment);

/* Replaces the current means from HOST memory (resume from saved centroids). */
int bkm_set_means(bkm_handle_t h, const float* host_means);

/* Iterations completed since the last initialize. */
int bkm_iterations_done(bkm_handle_t h, uint64_t* out);

/* Device time per phase, averaged over the iterations of the most recent run (at most the
 * last 8), in milliseconds: out[0]=assignment pass, out[1]=exact re-check of near-ties,
 * out[2]=update, out[3]=all-reduce, out[4]=divide + operand preparation, out[5]=whole
 * iteration.  Taken with CUDA events on the handle's stream. */
int bkm_phase_ms(bkm_handle_t h, float out[6]);

/* Counters of the most recent iteration: out[0]=points re-checked exactly,
 * out[1]=kernels launched per iteration, out[2]=assignment variant used,
 * out[3]=update variant used. */
int bkm_counters(bkm_handle_t h, uint64_t out[4]);

/* Which assignment kernel the handle launches and how (for tests and tuning; no counterpart in the
 * reference, whose runner is fixed by the ASGN_KERNEL template argument): out[0] = BKM_PLAN_* code,
 * out[1] = tiles of up to 256 means the tensor-core kernels walk (0 otherwise), out[2] = CTAs that
 * share one block of points and split its mean tiles between them (1 = none; > 1 means the partial
 * results are combined by a small merge kernel), out[3] = 1 when the last iteration's assignment
 * pass also accumulated the update sums.  Valid after bkm_initialize. */
#define BKM_PLAN_EXACT 0        /* CUDA cores, reference arithmetic */
#define BKM_PLAN_SIMT 1         /* CUDA cores, small-dim fast pass */
#define BKM_PLAN_TC_RESIDENT 2  /* tcgen05, one CTA per SM, point tiles resident (dim <= 32) */
#define BKM_PLAN_TC_KLOOP 3     /* tcgen05, one CTA per SM, both operands stream in slices (dim > 32) */
#define BKM_PLAN_TC_PAIR 4      /* tcgen05 on CTA pairs, all means resident in shared memory */
int bkm_assign_plan(bkm_handle_t h, uint32_t out[4]);

/* ---- multi-GPU (one process per GPU) ------------------------------------------------------ */

/* Fills `id` (128 bytes) with a fresh NCCL unique id; rank 0 calls it and hands the bytes
 * to the other ranks by whatever means the launcher offers. */
int bkm_comm_unique_id(void* id, size_t id_bytes);

/* Joins the handle to a communicator of `world_size` ranks.  Collective: every rank calls it
 * with the same id.  After it, every bkm_run all-reduces sums and sizes over the ranks. */
int bkm_comm_init(bkm_handle_t h, const void* id, size_t id_bytes, int world_size, int rank);

/* [begin, begin+count) of the points rank `rank` of `world_size` holds when `n_total` points
 * are split into contiguous, near-equal shards (pure host arithmetic, no GPU needed). */
int bkm_shard_range(uint64_t n_total, int world_size, int rank, uint64_t* begin, uint64_t* count);

/* ---- exchange through peer memory (instead of the NCCL all-reduce) ---------------------------
 * The sums and sizes of one iteration are k*dim + k words: a latency problem, not a bandwidth
 * problem.  With this exchange every rank owns a small receive buffer that the other ranks map
 * into their address space, and ONE kernel per iteration stores this rank's totals, each tagged
 * with the iteration count in the same 8-byte store, into the buffers of all ranks over NVLink,
 * polls its own buffer until every sender's packets of this iteration are there (bounded), adds
 * all ranks' values in rank order (bit-identical means everywhere), divides and prepares the next
 * operands - in place of merge + grouped all-reduce + finalize.  2..8 ranks, k*dim + k <= 2^19
 * (beyond that the exchange is bandwidth-bound and stays with NCCL); no counterpart in the
 * reference.  All ranks must make the same sequence of bkm_run calls (the packets carry the
 * iteration count).
 *
 * Several processes: every rank calls bkm_peer_export, the launcher gathers the blobs of all
 * ranks in rank order, every rank calls bkm_peer_open with the concatenation, the launcher makes
 * sure that ALL ranks succeeded (otherwise stay with NCCL), then every rank calls
 * bkm_peer_enable(h, 1).  One process driving several GPUs: bkm_peer_buffer of every handle,
 * bkm_peer_attach with the raw pointers (peer access enabled by the caller), bkm_peer_enable.
 * A wait that runs out ("exchange_wait_ms" option, default 2000) sets the status word, and the
 * remaining iterations of that run do not wait again: the run returns BKM_ERR_DEVICE within about
 * the limit, instead of hanging, when a rank has died or made a different call. */
#define BKM_PEER_BLOB_BYTES 128
int bkm_peer_export(bkm_handle_t h, void* blob, size_t blob_bytes);
int bkm_peer_open(bkm_handle_t h, const void* blobs, size_t blob_bytes_each, int world_size, int rank);
int bkm_peer_buffer(bkm_handle_t h, void** base, size_t* bytes);
int bkm_peer_attach(bkm_handle_t h, void* const* bases, int world_size, int rank);
int bkm_peer_enable(bkm_handle_t h, int enable);
/* Layout of a receive buffer (for tests and for hosts that inspect it): out[0] = bytes, out[1] =
 * 8-byte packets per sender (k*dim sums in row-major cluster order, then k sizes, padded), out[2] =
 * senders per slot, out[3] = bytes per slot.  The packet of word w from sender r in iteration t
 * (t = 1 for the first bkm_run iteration after bkm_create) lies at byte
 * (t & 1) * out[3] + (r * out[1] + w) * 8 and holds t in its high and the value in its low 32 bits.
 * Pure host arithmetic. */
int bkm_peer_layout(uint32_t k, uint32_t dim, uint64_t out[4]);

/* BKM_OK when the handle could start an iteration now (initialized, kernels set up, no error
 * pending).  For multi-rank launchers: reduce the codes of all ranks on the host BEFORE calling
 * bkm_run, and skip the run everywhere when any rank is not ready - a rank that fails before its
 * collective would otherwise leave its peers waiting for it. */
int bkm_run_ready(bkm_handle_t h);

/* ---- host-buffer convenience --------------------------------------------------------------
 * The whole job with HOST buffers in one call: create, initialize (host->device), run,
 * fetch results (device->host), destroy - the sequence the reference harness performs in
 * run_kmeans (k-means.cpp:118-189).  `means` holds the initial means on entry and the final
 * means on return. */
int bkm_kmeans_host_f32(const float* host_points, float* means, uint32_t* assignment,
                        uint64_t n, uint32_t k, uint32_t dim, uint32_t iters,
                        int layout, int layout_means, int device);

/* The same whole job in fp64, for the reference executable's --double mode (k-means.cpp:313-315,
 * 340-345: every algorithm there is instantiated for double as well).  Not the tuned path: one plain
 * kernel per step with the reference's arithmetic in double, so the assignment equals the serial
 * algorithm's (headers/serial.hpp:21-35 with F = double) bit for bit for the same means; sums are
 * accumulated with double atomics (means agree with the serial loop to rounding). */
int bkm_kmeans_host_f64(const double* host_points, double* means, uint32_t* assignment,
                        uint64_t n, uint32_t k, uint32_t dim, uint32_t iters,
                        int layout, int layout_means, int device);

#ifdef __cplusplus
}
#endif

#endif /* BKM_H */
