// Assignment on CUDA cores.
//
//  * assign_exact_kernel: one warp per point, lanes over the means, the reference's arithmetic
//    (sequential subtract / multiply / add without fusing, square root, strictly-smaller
//    comparison in ascending index order).  Used for every point by the EXACT variant and
//    for the queued near-ties of the fast passes.  Replaces baseAssignmentKernel
//    (kernels/kernels.cu:182-199 of the reference) and follows serial.hpp:21-35.
//
//  * assign_simt_kernel<D, SOA, P>: small-d fast pass (see the comment above the kernel): the
//    means staged into shared memory with a bulk TMA copy, P points per thread in registers,
//    |c|^2 - 2 x.c on the FMA pipe, arg-min on integer keys, near-ties queued for the exact
//    kernel.  Covers the shape range of cachedFixedAssignmentKernel (kernels/kernels.cu:218-273)
//    and cachedAllMeansAssignmentKernel (:330-374).
#include "kernels.cuh"
#include "ptx.cuh"
#include "keys.cuh"

#include <cmath>

namespace bkm {

// ------------------------------------------------------------------------------------------
// exact kernel
// ------------------------------------------------------------------------------------------

template<bool SOA, bool SOAM>
__global__ void __launch_bounds__(256) assign_exact_kernel(const float* __restrict__ pts,
	const float* __restrict__ means, uint32_t* __restrict__ asg, uint64_t n, uint32_t k, uint32_t d,
	const uint32_t* __restrict__ list, const uint32_t* __restrict__ list_count)
{
	extern __shared__ float sx[];
	const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
	float* x = sx + (size_t)warp * d;
	uint64_t total = n;
	if (list != nullptr) {
		uint64_t c = *list_count;
		total = c < n ? c : n;
	}
	for (uint64_t w = (uint64_t)blockIdx.x * wpb + warp; w < total; w += (uint64_t)gridDim.x * wpb) {
		const uint64_t i = list ? (uint64_t)list[w] : w;
		__syncwarp();
		for (uint32_t j = lane; j < d; j += 32) x[j] = pts[at<SOA>(i, j, n, d)];
		__syncwarp();
		float best = INFINITY;
		uint32_t bidx = 0xffffffffu;
		for (uint32_t m = lane; m < k; m += 32) {
			float sum = 0.0f;
			for (uint32_t j = 0; j < d; ++j) {
				float diff = __fsub_rn(x[j], means[at<SOAM>(m, j, k, d)]);
				sum = __fadd_rn(sum, __fmul_rn(diff, diff));
			}
			float dist = __fsqrt_rn(sum);
			if (dist < best || bidx == 0xffffffffu) { best = dist; bidx = m; }
		}
		// lowest (distance, index) pair over the warp = what the sequential scan would keep
		#pragma unroll
		for (int off = 16; off > 0; off >>= 1) {
			float ob = __shfl_xor_sync(0xffffffffu, best, off);
			uint32_t oi = __shfl_xor_sync(0xffffffffu, bidx, off);
			if (oi != 0xffffffffu && (bidx == 0xffffffffu || ob < best || (ob == best && oi < bidx))) { best = ob; bidx = oi; }
		}
		if (lane == 0) asg[i] = bidx;
	}
}


// Four consecutive dimensions of one mean against the LIST_PB staged points: each point's four
// coordinates come with one 128-bit shared load (the same address for the whole warp), and the
// squares are added in dimension order, one rounding per operation, as in the scalar loop.
template<int PB>
__device__ __forceinline__ void add_four_dims(float (&sum)[PB], const float* sx, uint32_t dpad, uint32_t j,
	float c0, float c1, float c2, float c3)
{
	#pragma unroll
	for (int p = 0; p < PB; ++p) {
		const float4 x = *reinterpret_cast<const float4*>(sx + p * dpad + j);
		const float d0 = __fsub_rn(x.x, c0), d1 = __fsub_rn(x.y, c1), d2 = __fsub_rn(x.z, c2), d3 = __fsub_rn(x.w, c3);
		sum[p] = __fadd_rn(sum[p], __fmul_rn(d0, d0));
		sum[p] = __fadd_rn(sum[p], __fmul_rn(d1, d1));
		sum[p] = __fadd_rn(sum[p], __fmul_rn(d2, d2));
		sum[p] = __fadd_rn(sum[p], __fmul_rn(d3, d3));
	}
}

// The same arithmetic for a list of queued points: one block per PB points, one mean per
// thread at a time, so that a short list still fills the machine and every mean that is
// fetched serves PB points (4, or 16 for long rows and many means, where the re-reads of the means
// for every group of points are what the kernel spends its time on).  Each distance is still summed in dimension order by a single
// thread.  AoS means are staged through a shared tile (32 dimensions of 256 means at a time,
// loaded along the dimensions) so that the global loads stay coalesced; SoA means are read
// directly (consecutive threads = consecutive means).
constexpr int LIST_THREADS = 256;
constexpr int LIST_PB = 4;          // points per block (the default)
constexpr int LIST_PB_WIDE = 16;    // ... when every fetched mean should serve more points (long rows, many means)
constexpr uint32_t LIST_SPLIT_MAX_BLOCKS = 2048;   // grid size up to which a short list is shared between blocks

template<bool SOA, bool SOAM, int PB>
__global__ void __launch_bounds__(LIST_THREADS, PB > LIST_PB ? 2 : 3) assign_exact_list_kernel(const float* __restrict__ pts,
	const float* __restrict__ means, uint32_t* __restrict__ asg, uint64_t n, uint32_t k, uint32_t d,
	const uint32_t* __restrict__ list, const uint32_t* __restrict__ list_count,
	float* __restrict__ fix_acc, uint32_t* __restrict__ fix_counts, uint32_t resident_ok,
	unsigned long long* __restrict__ split_keys, uint32_t* __restrict__ split_arrive)
{
	extern __shared__ __align__(16) float sx[];         // PB points (dpad floats each), then the means tile
	__shared__ uint32_t smoved[PB][2];             // (old, new) cluster of a point that changed, else old == new
	__shared__ uint32_t s_last;                         // this block is the last of its group's blocks to finish
	const uint32_t dpad = (d + 3) & ~3u;
	float (*tile)[33] = reinterpret_cast<float (*)[33]>(sx + (size_t)PB * dpad);
	__shared__ float sbest[PB][LIST_THREADS / 32];
	__shared__ uint32_t sidx[PB][LIST_THREADS / 32];
	const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
	uint64_t total = *list_count;
	if (total > n) total = n;
	// A long list and few means: every block copies all means to shared memory once (rows of an
	// odd number of floats, one mean per thread -> conflict-free) instead of fetching them again
	// for every group of points.
	const uint32_t ds = d | 1u;
	float* mres = sx + (size_t)PB * dpad;
	const bool resident = resident_ok != 0 && total >= (uint64_t)gridDim.x * PB * 4;
	if (resident) {
		for (uint32_t e = tid; e < k * d; e += LIST_THREADS) {
			// e walks the means array in memory order (coalesced)
			const uint32_t m = SOAM ? e % k : e / d, j = SOAM ? e / k : e % d;
			mres[m * ds + j] = means[e];
		}
	}
	// Staging of a group's points: two dependent global reads (the list entry, then the coordinate)
	// for each of the PB * d floats, all of them in flight together.  With few dimensions
	// (at most two floats per thread) a thread fetches the NEXT group's floats into registers
	// while the block works on the current group, which takes both reads off the block's
	// critical path.  Unused slots of the last group repeat its first point.
	const uint32_t pe = PB * d;
	const bool prefetch = pe <= 2 * LIST_THREADS;
	uint32_t pf_p[2], pf_j[2];
	float pf[2] = {0.0f, 0.0f};
	#pragma unroll
	for (uint32_t r = 0; r < 2; ++r) {
		const uint32_t e = tid + r * LIST_THREADS;
		pf_p[r] = e / d;
		pf_j[r] = e - pf_p[r] * d;
	}
	auto fetch = [&](uint64_t g0) {
		#pragma unroll
		for (uint32_t r = 0; r < 2; ++r) {
			if (tid + r * LIST_THREADS < pe) {
				const uint64_t idx = g0 + pf_p[r] < total ? g0 + pf_p[r] : g0;
				pf[r] = pts[at<SOA>((uint64_t)list[idx], pf_j[r], n, d)];
			}
		}
	};
	// A short list (fewer groups than blocks) would leave most of the machine idle while a few
	// blocks walk all k means one after another.  The blocks then share the groups: `splits`
	// blocks take one group, each a contiguous range of the means, and combine their results in
	// global memory (see below); every block has at most one piece of work.
	const uint64_t groups = (total + PB - 1) / PB;
	const uint32_t mchunks = (k + LIST_THREADS - 1) / LIST_THREADS;
	uint32_t splits = 1;
	if (split_keys != nullptr && groups > 0 && groups < gridDim.x && gridDim.x <= LIST_SPLIT_MAX_BLOCKS && mchunks > 1) {
		splits = gridDim.x / (uint32_t)groups;
		if (splits > mchunks) splits = mchunks;
	}
	const uint32_t split_group = blockIdx.x / splits, split_part = blockIdx.x - split_group * splits;
	const uint32_t m_begin = splits > 1 ? (split_part * mchunks / splits) * LIST_THREADS : 0u;
	const uint32_t m_end = splits > 1 ? min(k, ((split_part + 1) * mchunks / splits) * LIST_THREADS) : k;
	const uint32_t n_chunks = (m_end - m_begin + LIST_THREADS - 1) / LIST_THREADS;
	const uint32_t chunk_rot = (splits > 1 ? split_group : blockIdx.x) % n_chunks;
	const uint64_t stride = (uint64_t)gridDim.x * PB;        // with splits > 1 one step leaves the list
	const uint64_t w_first = (uint64_t)(splits > 1 ? split_group : blockIdx.x) * PB;
	if (prefetch && w_first < total) fetch(w_first);
	for (uint64_t w0 = w_first; w0 < total; w0 += stride) {
		const uint32_t np = total - w0 < PB ? (uint32_t)(total - w0) : PB;
		__syncthreads();
		if (prefetch) {
			#pragma unroll
			for (uint32_t r = 0; r < 2; ++r)
				if (tid + r * LIST_THREADS < pe) sx[pf_p[r] * dpad + pf_j[r]] = pf[r];
		} else {
			for (uint32_t e = tid; e < pe; e += LIST_THREADS) {
				const uint32_t p = e / d, j = e - p * d;
				const uint64_t idx = w0 + p < total ? w0 + p : w0;
				sx[p * dpad + j] = pts[at<SOA>((uint64_t)list[idx], j, n, d)];
			}
		}
		__syncthreads();
		if (prefetch && w0 + stride < total) fetch(w0 + stride);
		float best[PB];
		uint32_t bidx[PB];
		#pragma unroll
		for (int p = 0; p < PB; ++p) { best[p] = INFINITY; bidx[p] = 0xffffffffu; }
		// The blocks walk their chunks of 256 means starting at different chunks, so that blocks
		// working at the same time do not all ask the L2 for the same rows at once.
		for (uint32_t c = 0; c < n_chunks; ++c) {
			const uint32_t m0 = m_begin + (c + chunk_rot < n_chunks ? c + chunk_rot : c + chunk_rot - n_chunks) * LIST_THREADS;
			const uint32_t m = m0 + tid;
			float sum[PB];
			#pragma unroll
			for (int p = 0; p < PB; ++p) sum[p] = 0.0f;
			if (resident) {
				if (m < k) {
					const float* cm = mres + m * ds;
					uint32_t j = 0;
					for (; j + 4 <= d; j += 4) add_four_dims<PB>(sum, sx, dpad, j, cm[j], cm[j + 1], cm[j + 2], cm[j + 3]);
					for (; j < d; ++j) {
						const float c = cm[j];
						#pragma unroll
						for (int p = 0; p < PB; ++p) {
							const float diff = __fsub_rn(sx[p * dpad + j], c);
							sum[p] = __fadd_rn(sum[p], __fmul_rn(diff, diff));
						}
					}
				}
			} else if (SOAM) {
				if (m < k) {
					const float* cm = means + m;
					uint32_t j = 0;
					for (; j + 4 <= d; j += 4)
						add_four_dims<PB>(sum, sx, dpad, j, cm[(size_t)j * k], cm[(size_t)(j + 1) * k], cm[(size_t)(j + 2) * k], cm[(size_t)(j + 3) * k]);
					for (; j < d; ++j) {
						const float c = cm[(size_t)j * k];
						#pragma unroll
						for (int p = 0; p < PB; ++p) {
							const float diff = __fsub_rn(sx[p * dpad + j], c);
							sum[p] = __fadd_rn(sum[p], __fmul_rn(diff, diff));
						}
					}
				}
			} else {
				// 32 dimensions of the chunk's 256 means at a time go through the shared tile (read along
				// the rows, used along the means).  The next slab's row segments are fetched into registers
				// while the current slab is evaluated, so their latency does not sit between two barriers.
				float seg[32];
				auto fetch_slab = [&](uint32_t j0) {
					#pragma unroll
					for (uint32_t r = 0; r < 32; ++r) {
						const uint32_t row = warp * 32 + r;
						seg[r] = (m0 + row < k && j0 + lane < d) ? means[(size_t)(m0 + row) * d + j0 + lane] : 0.0f;
					}
				};
				fetch_slab(0);
				for (uint32_t j0 = 0; j0 < d; j0 += 32) {
					__syncthreads();                    // the previous slab has been read by everyone
					#pragma unroll
					for (uint32_t r = 0; r < 32; ++r) tile[warp * 32 + r][lane] = seg[r];
					__syncthreads();
					if (j0 + 32 < d) fetch_slab(j0 + 32);
					const uint32_t jn = d - j0 < 32 ? d - j0 : 32;
					uint32_t jj = 0;
					for (; jj + 4 <= jn; jj += 4)
						add_four_dims<PB>(sum, sx, dpad, j0 + jj, tile[tid][jj], tile[tid][jj + 1], tile[tid][jj + 2], tile[tid][jj + 3]);
					for (; jj < jn; ++jj) {
						const float c = tile[tid][jj];
						#pragma unroll
						for (int p = 0; p < PB; ++p) {
							const float diff = __fsub_rn(sx[p * dpad + j0 + jj], c);
							sum[p] = __fadd_rn(sum[p], __fmul_rn(diff, diff));
						}
					}
				}
			}
			if (m < k) {
				#pragma unroll
				for (int p = 0; p < PB; ++p) {
					const float dist = __fsqrt_rn(sum[p]);
					// (the chunks come in rotated order: the lower index wins a tie explicitly)
					if (bidx[p] == 0xffffffffu || dist < best[p] || (dist == best[p] && m < bidx[p])) { best[p] = dist; bidx[p] = m; }
				}
			}
		}
		#pragma unroll
		for (int p = 0; p < PB; ++p) {
			// Distances are >= +0, so their bit patterns order like the values: the warp's smallest
			// distance, then the lowest index among the means that have it (a thread without a mean
			// holds infinity and the index 0xffffffff).
			const uint32_t bits = __float_as_uint(best[p]);
			const uint32_t mn = __reduce_min_sync(0xffffffffu, bits);
			const uint32_t mi = __reduce_min_sync(0xffffffffu, bits == mn ? bidx[p] : 0xffffffffu);
			if (lane == 0) { sbest[p][warp] = __uint_as_float(mn); sidx[p][warp] = mi; }
		}
		__syncthreads();
		if (tid < np) {
			float b = sbest[tid][0];
			uint32_t bi = sidx[tid][0];
			for (uint32_t v = 1; v < LIST_THREADS / 32; ++v) {
				const float ob = sbest[tid][v];
				const uint32_t oi = sidx[tid][v];
				if (oi != 0xffffffffu && (bi == 0xffffffffu || ob < b || (ob == b && oi < bi))) { b = ob; bi = oi; }
			}
			if (splits > 1) {
				// (distance, index) as one 64-bit key whose minimum is the smallest distance and, among
				// equal distances, the lowest index; stored inverted so that zero means "nothing yet"
				const unsigned long long key = ((unsigned long long)__float_as_uint(b) << 32) | bi;
				atomicMax(&split_keys[w0 + tid], ~key);
			} else {
				const uint32_t i = list[w0 + tid];
				smoved[tid][0] = fix_acc ? asg[i] : bi;
				smoved[tid][1] = bi;
				asg[i] = bi;
			}
		}
		if (splits > 1) {
			// The block that arrives last for its group finds all partial results in place; it
			// writes the assignment and leaves keys and counter zeroed for the next launch.
			__threadfence();
			__syncthreads();
			if (tid == 0) s_last = atomicAdd(&split_arrive[split_group], 1u) == splits - 1 ? 1u : 0u;
			__syncthreads();
			if (s_last == 0) break;
			__threadfence();
			if (tid < np) {
				const unsigned long long key = ~atomicExch(&split_keys[w0 + tid], 0ull);
				const uint32_t bi = (uint32_t)key;
				const uint32_t i = list[w0 + tid];
				smoved[tid][0] = fix_acc ? asg[i] : bi;
				smoved[tid][1] = bi;
				asg[i] = bi;
			}
			if (tid == 0) split_arrive[split_group] = 0;
		}
		if (fix_acc) {
			// the fast pass has already added these points to the sums of the clusters it picked
			__syncthreads();
			for (uint32_t p = 0; p < np; ++p) {
				const uint32_t from = smoved[p][0], to = smoved[p][1];
				if (from == to || from >= k) continue;
				for (uint32_t j = tid; j < d; j += LIST_THREADS) {
					const float x = sx[p * dpad + j];
					atomicAdd(&fix_acc[(size_t)from * d + j], -x);
					atomicAdd(&fix_acc[(size_t)to * d + j], x);
				}
				if (tid == 0) { atomicSub(&fix_counts[from], 1u); atomicAdd(&fix_counts[to], 1u); }
			}
		}
	}
}

// The same arithmetic with one THREAD per queued point and all means in shared memory, for mean sets
// of a few thousand floats and at most 16 dimensions: there a block per four points spends its time
// in barriers and reductions, while a thread walks the whole set in microseconds and a long list
// fills the machine by itself.
constexpr uint32_t LIST_SMALL_MAX_FLOATS = 4096;
constexpr uint32_t LIST_SMALL_MAX_DIM = 16;

template<int D, bool SOA, bool SOAM>
__global__ void __launch_bounds__(256) assign_exact_list_small_kernel(const float* __restrict__ pts, const float* __restrict__ means,
	uint32_t* __restrict__ asg, uint64_t n, uint32_t k, const uint32_t* __restrict__ list, const uint32_t* __restrict__ list_count,
	float* __restrict__ fix_acc, uint32_t* __restrict__ fix_counts)
{
	__shared__ __align__(16) float sm[LIST_SMALL_MAX_FLOATS];          // [mean][dimension]
	uint64_t total = *list_count;
	if (total > n) total = n;
	if ((uint64_t)blockIdx.x * blockDim.x >= total) return;            // the grid is sized for long lists: most blocks of a short one have nothing to do
	for (uint32_t e = threadIdx.x; e < k * D; e += blockDim.x) {
		const uint32_t m = e / D, j = e - m * D;
		sm[e] = means[at<SOAM>(m, j, k, D)];
	}
	__syncthreads();
	for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (uint64_t)gridDim.x * blockDim.x) {
		const uint64_t i = list[w];
		float x[D];
		#pragma unroll
		for (int j = 0; j < D; ++j) x[j] = pts[at<SOA>(i, j, n, D)];
		float best = 0.0f, best_sum = 0.0f;
		uint32_t bidx = 0;
		for (uint32_t m = 0; m < k; ++m) {
			float c[D];
			if (D % 4 == 0) {
				// whole rows as 128-bit loads (the same address for all threads: broadcast)
				#pragma unroll
				for (int q = 0; q < D / 4; ++q) {
					const float4 v = reinterpret_cast<const float4*>(sm + m * D)[q];
					c[4 * q] = v.x; c[4 * q + 1] = v.y; c[4 * q + 2] = v.z; c[4 * q + 3] = v.w;
				}
			} else {
				#pragma unroll
				for (int j = 0; j < D; ++j) c[j] = sm[m * D + j];
			}
			float sum = 0.0f;
			#pragma unroll
			for (int j = 0; j < D; ++j) {
				const float diff = __fsub_rn(x[j], c[j]);
				sum = __fadd_rn(sum, __fmul_rn(diff, diff));
			}
			// The reference compares square roots.  The correctly rounded square root never decreases
			// with its argument, so a sum that is not below the best sum cannot give a smaller root:
			// only the few candidates that are below it need the root itself (equal roots of different
			// sums keep the earlier mean, as the reference's strict comparison does).
			if (m == 0) {
				best_sum = sum;
				best = __fsqrt_rn(sum);
			} else if (sum < best_sum) {
				const float dist = __fsqrt_rn(sum);
				if (dist < best) { best = dist; best_sum = sum; bidx = m; }
			}
		}
		if (fix_acc) {
			// the fast pass has already added this point to the sum of the cluster it picked
			const uint32_t from = asg[i];
			if (from != bidx && from < k) {
				#pragma unroll
				for (int j = 0; j < D; ++j) {
					atomicAdd(&fix_acc[(size_t)from * D + j], -x[j]);
					atomicAdd(&fix_acc[(size_t)bidx * D + j], x[j]);
				}
				atomicSub(&fix_counts[from], 1u);
				atomicAdd(&fix_counts[bidx], 1u);
			}
		}
		asg[i] = bidx;
	}
}

template<int D>
static cudaError_t launch_list_small(const float* pts, const float* means, uint32_t* asg, const Shape& s,
	const uint32_t* list, const uint32_t* list_count, int sm_count, cudaStream_t stream, const FusedAcc* fix)
{
	// a thread's point is a dependent gather behind its list entry: many threads in flight hide that,
	// so a long list gets one or two points per thread rather than a loop
	const uint32_t grid = (uint32_t)sm_count * 16;
	float* fa = fix ? fix->acc : nullptr;
	uint32_t* fc = fix ? fix->counts : nullptr;
	if (s.soa && s.soa_means) assign_exact_list_small_kernel<D, true, true><<<grid, 256, 0, stream>>>(pts, means, asg, s.n, s.k, list, list_count, fa, fc);
	else if (s.soa) assign_exact_list_small_kernel<D, true, false><<<grid, 256, 0, stream>>>(pts, means, asg, s.n, s.k, list, list_count, fa, fc);
	else if (s.soa_means) assign_exact_list_small_kernel<D, false, true><<<grid, 256, 0, stream>>>(pts, means, asg, s.n, s.k, list, list_count, fa, fc);
	else assign_exact_list_small_kernel<D, false, false><<<grid, 256, 0, stream>>>(pts, means, asg, s.n, s.k, list, list_count, fa, fc);
	return cudaGetLastError();
}

size_t list_split_scratch_bytes()
{
	return (size_t)LIST_SPLIT_MAX_BLOCKS * LIST_PB_WIDE * sizeof(unsigned long long) + (size_t)LIST_SPLIT_MAX_BLOCKS * sizeof(uint32_t);
}

cudaError_t launch_assign_exact(const float* pts, const float* means, uint32_t* asg, const Shape& s,
	const uint32_t* list, const uint32_t* list_count, int sm_count, cudaStream_t stream, const FusedAcc* fix, void* split_scratch)
{
	unsigned long long* split_keys = reinterpret_cast<unsigned long long*>(split_scratch);
	uint32_t* split_arrive = split_scratch ? reinterpret_cast<uint32_t*>(split_keys + (size_t)LIST_SPLIT_MAX_BLOCKS * LIST_PB_WIDE) : nullptr;
	if (fix != nullptr && (list == nullptr || (size_t)s.dim * sizeof(float) * LIST_PB > 120 * 1024)) return cudaErrorInvalidValue;
	if (list != nullptr && s.dim <= LIST_SMALL_MAX_DIM && (uint64_t)s.k * s.dim <= LIST_SMALL_MAX_FLOATS) {
		switch (s.dim) {
		case 1: return launch_list_small<1>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 2: return launch_list_small<2>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 3: return launch_list_small<3>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 4: return launch_list_small<4>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 5: return launch_list_small<5>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 6: return launch_list_small<6>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 7: return launch_list_small<7>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 8: return launch_list_small<8>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 9: return launch_list_small<9>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 10: return launch_list_small<10>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 11: return launch_list_small<11>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 12: return launch_list_small<12>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 13: return launch_list_small<13>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 14: return launch_list_small<14>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		case 15: return launch_list_small<15>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		default: return launch_list_small<16>(pts, means, asg, s, list, list_count, sm_count, stream, fix);
		}
	}
	if (list != nullptr && (size_t)s.dim * sizeof(float) * LIST_PB <= 120 * 1024) {
		// Every group of points walks all means: with long rows and many means (megabytes of them) the
		// re-reads through L2 dominate, and sixteen points per group cut them fourfold.
		const bool wide = fix == nullptr && (size_t)s.k * s.dim * sizeof(float) >= (1u << 20) &&
			(size_t)LIST_PB_WIDE * ((s.dim + 3) & ~3u) * sizeof(float) <= 64 * 1024;
		const int pb = wide ? LIST_PB_WIDE : LIST_PB;
		const size_t points_bytes = (size_t)pb * ((s.dim + 3) & ~3u) * sizeof(float);
		size_t lsmem = points_bytes + (s.soa_means ? 0 : (size_t)LIST_THREADS * 33 * sizeof(float));
		// room for all means (the kernel uses it when the list is long): at most 64 KiB, so that
		// several blocks still share an SM
		const size_t resident_bytes = points_bytes + (size_t)s.k * (s.dim | 1u) * sizeof(float);
		const uint32_t resident_ok = resident_bytes <= 64 * 1024 ? 1u : 0u;
		if (resident_ok && resident_bytes > lsmem) lsmem = resident_bytes;
		const uint32_t lgrid = (uint32_t)sm_count * 8;
#define BKM_LAUNCH_LIST_PB(SOA, SOAM, PBV) do { \
		auto kern = assign_exact_list_kernel<SOA, SOAM, PBV>; \
		if (lsmem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lsmem); if (e != cudaSuccess) return e; } \
		kern<<<lgrid, LIST_THREADS, lsmem, stream>>>(pts, means, asg, s.n, s.k, s.dim, list, list_count, \
			fix ? fix->acc : nullptr, fix ? fix->counts : nullptr, resident_ok, split_keys, split_arrive); \
	} while (0)
#define BKM_LAUNCH_LIST(SOA, SOAM) do { if (wide) BKM_LAUNCH_LIST_PB(SOA, SOAM, LIST_PB_WIDE); else BKM_LAUNCH_LIST_PB(SOA, SOAM, LIST_PB); } while (0)
		if (s.soa && s.soa_means) BKM_LAUNCH_LIST(true, true);
		else if (s.soa && !s.soa_means) BKM_LAUNCH_LIST(true, false);
		else if (!s.soa && s.soa_means) BKM_LAUNCH_LIST(false, true);
		else BKM_LAUNCH_LIST(false, false);
#undef BKM_LAUNCH_LIST_PB
#undef BKM_LAUNCH_LIST
		return cudaGetLastError();
	}

	// shared memory: one copy of the point per warp
	uint32_t warps = 8;
	while (warps > 1 && (size_t)warps * s.dim * sizeof(float) > 96 * 1024) warps >>= 1;
	size_t smem = (size_t)warps * s.dim * sizeof(float);
	if (smem > 200 * 1024) return cudaErrorInvalidValue;
	uint64_t want = list ? (uint64_t)sm_count * 8 : (s.n + warps - 1) / warps;
	uint32_t grid = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(want, 1), (uint64_t)sm_count * 16);
	dim3 block(warps * 32);
#define BKM_LAUNCH_EXACT(SOA, SOAM) do { \
		auto kern = assign_exact_kernel<SOA, SOAM>; \
		if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; } \
		kern<<<grid, block, smem, stream>>>(pts, means, asg, s.n, s.k, s.dim, list, list_count); \
	} while (0)
	if (s.soa && s.soa_means) BKM_LAUNCH_EXACT(true, true);
	else if (s.soa && !s.soa_means) BKM_LAUNCH_EXACT(true, false);
	else if (!s.soa && s.soa_means) BKM_LAUNCH_EXACT(false, true);
	else BKM_LAUNCH_EXACT(false, false);
#undef BKM_LAUNCH_EXACT
	return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// small-d fast pass
// ------------------------------------------------------------------------------------------
//
// Every thread keeps P points in registers (shifted by the common centre vector) and walks the
// means in chunks of 32.  A mean's row in shared memory is [ |c|^2 + C, -2c_0 .. -2c_{D-1} ], so a
// point's value |c|^2 - 2 x.c + C costs D fused multiply-adds per mean; the constant C (from the
// largest |x|^2 and |c|^2, see make_key_consts) puts all values into one binade, where their bit
// patterns order like the values.  The 32 values of a chunk become integer keys (bits * M + column)
// and are reduced to the smallest and second smallest with plain integer minima (chunk_update):
// about 1.75 integer instructions per point and mean where a (best, second, index) tournament on
// floats takes five, and D instead of 2D arithmetic instructions.  The form cancels where the
// difference form does not, so a point whose best and second-best keys are closer than the
// rounding band of the pass (and of the reference's own sum and square root) is queued for the
// exact kernel; the final assignment is the reference's for every point.

constexpr int SIMT_THREADS = 256;
constexpr int SIMT_TILE_ROWS = 1024; // means per shared-memory tile (a multiple of the 32-mean chunk)

// Fused update sums (FUSE): every WARP sorts the 32 * P points it has just assigned by cluster, in
// shared memory of its own (counters whose atomic also yields the rank, prefix sum over the counters,
// scatter of the centred coordinates to the sorted position).  A lane then walks P neighbouring
// sorted positions, adds rows while the cluster stays the same and sends one row of reductions when
// it changes (with the centre added back, once per point of the run); the sizes are counted per
// block and sent at the end.  Nothing here waits for another warp, and no separate update pass reads
// the points again.  (Measured alternatives on 2^24 two-dimensional points, 64 clusters, where the
// plain pass takes 0.32 ms and a separate sorted update 0.10 ms: this form 0.43 ms; the same sort per
// block with five block-wide barriers 0.48 ms; match.any groups added by the warp's integer
// reduction 1.53 ms - both instructions are replayed once per distinct cluster in the warp.)
constexpr uint32_t SIMT_FUSE_MAX_K = 1024;

// sum[0..D) + len * cen[0..D) onto the row `dst` of the accumulators, as vector reductions where the row allows
template<int D>
__device__ __forceinline__ void send_row(float* dst, const float (&sum)[D], float len, const float (&cen)[D])
{
	float v[D];
	#pragma unroll
	for (int j = 0; j < D; ++j) v[j] = fmaf(len, cen[j], sum[j]);
	if (D % 4 == 0) {
		#pragma unroll
		for (int q = 0; q < D / 4; ++q)
			asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(dst + 4 * q), "f"(v[4 * q]), "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3]) : "memory");
	} else if (D % 2 == 0) {
		#pragma unroll
		for (int q = 0; q < D / 2; ++q)
			asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" :: "l"(dst + 2 * q), "f"(v[2 * q]), "f"(v[2 * q + 1]) : "memory");
	} else {
		#pragma unroll
		for (int j = 0; j < D; ++j) atomicAdd(dst + j, v[j]);
	}
}

template<int D, bool SOA, int P, bool FUSE>
__global__ void __launch_bounds__(SIMT_THREADS) assign_simt_kernel(const float* __restrict__ pts,
	const float* __restrict__ cprep, const float* __restrict__ center, uint32_t* __restrict__ asg, uint64_t n, uint32_t rows,
	Control* __restrict__ ctl, int slot, uint32_t* __restrict__ flag_list, float margin_ulps, int vec_ok,
	uint32_t k, float* __restrict__ fuse_acc, uint32_t* __restrict__ fuse_counts)
{
	constexpr int RS = (D + 1 + 3) / 4 * 4;
	extern __shared__ __align__(128) float tile[];
	__shared__ __align__(8) uint64_t bar;
	// fused update sums: see above
	__shared__ uint32_t s_hist[FUSE ? SIMT_THREADS / 32 : 1][FUSE ? (SIMT_FUSE_MAX_K + 2) / 2 : 1];   // per warp: points per cluster, 16 bits each
	__shared__ uint32_t s_cnt[FUSE ? SIMT_FUSE_MAX_K : 1];                  // sizes counted by this block
	__shared__ __align__(16) float s_x[FUSE ? SIMT_THREADS * P * D : 1];    // per warp: sorted position -> centred coordinates
	__shared__ __align__(8) uint16_t s_cl[FUSE ? SIMT_THREADS * P : 4];     // per warp: sorted position -> cluster
	float* fuse_acc_rep = fuse_acc;
	if (FUSE) {
		fuse_acc_rep += (blockIdx.x % acc_replicas(k, D)) * acc_replica_stride(k, D);
		for (uint32_t c = threadIdx.x; c < SIMT_FUSE_MAX_K; c += SIMT_THREADS) s_cnt[c] = 0;
	}
	__shared__ uint32_t flag_bufs[SIMT_THREADS / 32][FLAG_BUFFER];     // per warp: near-ties on their way to the list
	uint32_t* flag_buf = flag_bufs[threadIdx.x >> 5];
	uint32_t flag_cnt = 0;

	const uint32_t tid = threadIdx.x;
	const uint32_t ntiles = (rows + SIMT_TILE_ROWS - 1) / SIMT_TILE_ROWS;
	const uint64_t per_block = (uint64_t)SIMT_THREADS * P;
	const uint64_t nblocks = (n + per_block - 1) / per_block;
	const KeyConsts kc = make_key_consts(ctl->xmax2, ctl->cmax2[slot]);
	const uint32_t key_mult = kc.key_mult, key_base = kc.key_base, key_magic = kc.key_magic;
	const float pad_value = kc.pow2 * (2.0f - 1.0f / 32.0f);     // padding rows: above every real value, inside [P, 2P)
	uint32_t phase = 0;
	bool ok = true;
	float cen[D];
	#pragma unroll
	for (int j = 0; j < D; ++j) cen[j] = center[j];

	if (tid == 0) {
		ptx::mbar_init(&bar, 1);
		ptx::fence_mbar_init();
	}
	__syncthreads();

	// Brings tile t of the prepared means into shared memory and adds the offset constant to its
	// |c|^2 column (padding rows, marked by +inf there, get the top of the value band).
	auto load_tile = [&](uint32_t t) -> uint32_t {
		uint32_t trows = rows - t * SIMT_TILE_ROWS;
		if (trows > SIMT_TILE_ROWS) trows = SIMT_TILE_ROWS;
		if (tid == 0) {
			const uint32_t bytes = trows * RS * (uint32_t)sizeof(float);
			ptx::mbar_arrive_expect_tx(&bar, bytes);
			ptx::bulk_g2s(tile, cprep + (size_t)t * SIMT_TILE_ROWS * RS, bytes, &bar);
		}
		ok = ptx::mbar_wait(&bar, phase) && ok;
		phase ^= 1;
		for (uint32_t r = tid; r < trows; r += SIMT_THREADS) {
			const float c2 = tile[(size_t)r * RS];
			tile[(size_t)r * RS] = c2 > 3.0e38f ? pad_value : c2 + kc.offset_c;
		}
		__syncthreads();
		return trows;
	};

	uint32_t trows0 = 0;
	if (ntiles == 1) trows0 = load_tile(0);

	// The points of a block of work, as they lie in memory (slots behind the last point read as the
	// centre).  The next block's points are fetched while the current block is being evaluated.
	float raw[P][D];
	auto load_points = [&](uint64_t blk) {
		const uint64_t base = blk * per_block;
		if (SOA) {
			#pragma unroll
			for (int p = 0; p < P; ++p) {
				const uint64_t i = base + (uint64_t)p * SIMT_THREADS + tid;
				#pragma unroll
				for (int j = 0; j < D; ++j) raw[p][j] = i < n ? pts[(size_t)j * n + i] : cen[j];
			}
		} else {
			const uint64_t i0 = base + (uint64_t)tid * P;
			if ((P * D) % 4 == 0 && vec_ok && i0 + P - 1 < n) {
				// 128-bit loads: the thread's P points are P*D consecutive floats
				const float4* src = reinterpret_cast<const float4*>(pts + (size_t)i0 * D);
				float buf[P * D];
				#pragma unroll
				for (int q = 0; q < (P * D) / 4; ++q) {
					float4 v = src[q];
					buf[4 * q + 0] = v.x; buf[4 * q + 1] = v.y; buf[4 * q + 2] = v.z; buf[4 * q + 3] = v.w;
				}
				#pragma unroll
				for (int p = 0; p < P; ++p)
					#pragma unroll
					for (int j = 0; j < D; ++j) raw[p][j] = buf[p * D + j];
			} else {
				#pragma unroll
				for (int p = 0; p < P; ++p)
					#pragma unroll
					for (int j = 0; j < D; ++j) raw[p][j] = i0 + p < n ? pts[(size_t)(i0 + p) * D + j] : cen[j];
			}
		}
	};
	if (blockIdx.x < nblocks) load_points(blockIdx.x);

	for (uint64_t blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
		float x[P][D];
		uint64_t idx[P];
		const uint64_t base = blk * per_block;
		#pragma unroll
		for (int p = 0; p < P; ++p) {
			idx[p] = SOA ? base + (uint64_t)p * SIMT_THREADS + tid : base + (uint64_t)tid * P + p;
			#pragma unroll
			for (int j = 0; j < D; ++j) x[p][j] = raw[p][j] - cen[j];
		}
		if (blk + gridDim.x < nblocks) load_points(blk + gridDim.x);

		uint32_t best[P], second[P], bchunk[P];
		#pragma unroll
		for (int p = 0; p < P; ++p) { best[p] = 0xFFFFFFFFu; second[p] = 0xFFFFFFFFu; bchunk[p] = 0; }

		for (uint32_t t = 0; t < ntiles; ++t) {
			uint32_t trows = trows0;
			if (ntiles > 1) {
				__syncthreads();   // everyone is done reading the previous tile
				trows = load_tile(t);
			}
			const uint32_t chunk_base = t * (SIMT_TILE_ROWS / 32);
			#pragma unroll 1
			for (uint32_t ch = 0; ch < trows / 32; ++ch) {
				uint32_t v[P][32];
				const float4* rowp = reinterpret_cast<const float4*>(tile + (size_t)ch * 32 * RS);
				#pragma unroll
				for (int m = 0; m < 32; ++m) {
					float r[RS];
					#pragma unroll
					for (int q = 0; q < RS / 4; ++q) {
						const float4 w = rowp[m * (RS / 4) + q];
						r[4 * q + 0] = w.x; r[4 * q + 1] = w.y; r[4 * q + 2] = w.z; r[4 * q + 3] = w.w;
					}
					#pragma unroll
					for (int p = 0; p < P; ++p) {
						float val = r[0];
						#pragma unroll
						for (int j = 0; j < D; ++j) val = fmaf(x[p][j], r[1 + j], val);
						v[p][m] = __float_as_uint(val);
					}
				}
				#pragma unroll
				for (int p = 0; p < P; ++p) chunk_update<false>(v[p], key_mult, chunk_base + ch, 32, best[p], second[p], bchunk[p]);
			}
		}

		uint32_t cl[P];
		#pragma unroll
		for (int p = 0; p < P; ++p) {
			bool flag = false;
			cl[p] = k;                     // rows behind the last point sort behind every cluster
			if (idx[p] < n) {
				// key - key_base = M * mantissa + column
				const uint32_t bm = div_key(best[p] - key_base, key_magic);
				cl[p] = bchunk[p] * 32u + ((best[p] - key_base) - bm * key_mult);
				asg[idx[p]] = cl[p];
				const float gap = second[p] == 0xFFFFFFFFu ? INFINITY : (float)(div_key(second[p] - key_base, key_magic) - bm);
				flag = gap <= margin_ulps;
			}
			buffered_append(flag, (uint32_t)idx[p], flag_buf, flag_cnt, ctl, flag_list, n);
		}

		if (FUSE) {
			// everything below is private to the warp: its 32 * P points, its counters, its sorted rows
			const uint32_t lane = tid & 31u, warp = tid >> 5;
			uint32_t* hist32 = s_hist[warp];
			uint16_t* hist = reinterpret_cast<uint16_t*>(hist32);      // k + 1 counters, two to a word; the start positions later
			uint16_t* w_cl = s_cl + warp * (32 * P);
			float* w_x = s_x + warp * (32 * P * D);
			const uint32_t nb = k + 1;
			__syncwarp();                  // the walk over the previous block's rows is over
			for (uint32_t w = lane; w < (nb + 1) / 2; w += 32) hist32[w] = 0;
			__syncwarp();
			uint32_t rank[P];
			#pragma unroll
			for (int p = 0; p < P; ++p) {
				if (cl[p] > k) cl[p] = k;  // (cannot happen: padding columns never win)
				const uint32_t sh = (cl[p] & 1u) * 16u;
				rank[p] = (atomicAdd(&hist32[cl[p] >> 1], 1u << sh) >> sh) & 0xffffu;   // the count also hands out the place within the cluster
			}
			__syncwarp();
			// exclusive prefix sum over the counters: a run of them per lane, warp scan of the run totals
			const uint32_t per = (nb + 31) / 32, b0 = min(nb, lane * per), b1 = min(nb, b0 + per);
			uint32_t local = 0;
			for (uint32_t b = b0; b < b1; ++b) {
				const uint32_t v = hist[b];
				local += v;
				if (v != 0 && b < k) atomicAdd(&s_cnt[b], v);          // the sizes, sent once at the end of the kernel
			}
			uint32_t incl = local;
			#pragma unroll
			for (uint32_t off = 1; off < 32; off <<= 1) { const uint32_t o = __shfl_up_sync(0xffffffffu, incl, off); if (lane >= off) incl += o; }
			uint32_t run = incl - local;
			for (uint32_t b = b0; b < b1; ++b) {
				const uint32_t v = hist[b];
				hist[b] = (uint16_t)run;
				run += v;
			}
			__syncwarp();
			#pragma unroll
			for (int p = 0; p < P; ++p) {
				const uint32_t pos = hist[cl[p]] + rank[p];
				w_cl[pos] = (uint16_t)cl[p];
				#pragma unroll
				for (int j = 0; j < D; ++j) w_x[pos * D + j] = x[p][j];
			}
			__syncwarp();
			const uint32_t total = hist[k];    // rows of real points
			float sum[D];
			#pragma unroll
			for (int j = 0; j < D; ++j) sum[j] = 0.0f;
			float len = 0.0f;
			uint32_t cur = 0;
			#pragma unroll
			for (int u = 0; u < P; ++u) {
				const uint32_t sp = lane * P + u;
				if (sp < total) {
					const uint32_t c = w_cl[sp];
					if (u == 0) cur = c;
					if (c != cur) {
						send_row<D>(fuse_acc_rep + (size_t)cur * D, sum, len, cen);
						#pragma unroll
						for (int j = 0; j < D; ++j) sum[j] = 0.0f;
						len = 0.0f;
						cur = c;
					}
					#pragma unroll
					for (int j = 0; j < D; ++j) sum[j] += w_x[sp * D + j];
					len += 1.0f;
				}
			}
			if (len > 0.0f) send_row<D>(fuse_acc_rep + (size_t)cur * D, sum, len, cen);
		}
	}
	if (FUSE) {
		__syncthreads();
		uint32_t* cnt = fuse_counts + (blockIdx.x % acc_replicas(k, D)) * acc_replica_stride(k, D);
		for (uint32_t c = tid; c < k; c += SIMT_THREADS) {
			const uint32_t v = s_cnt[c];
			if (v) atomicAdd(&cnt[c], v);
		}
	}
	flush_flag_buffer(flag_buf, flag_cnt, ctl, flag_list, n);
	if (!ok && tid == 0) atomicOr(&ctl->status, (uint32_t)STATUS_WAIT_TIMEOUT);
}

bool assign_simt_supported(const Shape& s)
{
	return s.dim >= 1 && s.dim <= 8 && s.n < (1ull << 32);
}

bool assign_simt_can_fuse(const Shape& s, const FusedAcc& f)
{
	// one tile of means (so that a block meets its points once), vector reductions need aligned rows
	return assign_simt_supported(s) && s.k <= SIMT_FUSE_MAX_K && simt_rows(s.k) <= (uint32_t)SIMT_TILE_ROWS && f.acc != nullptr && f.counts != nullptr &&
		(reinterpret_cast<uintptr_t>(f.acc) & 15u) == 0 && (f.rep_stride * sizeof(float)) % 16 == 0;
}

template<int D, int P>
static cudaError_t launch_simt_d(const float* pts, const float* cprep, const float* center, uint32_t* asg, const Shape& s,
	Control* ctl, int slot, uint32_t* flag_list, float margin_scale, int sm_count, cudaStream_t stream, const FusedAcc* fused)
{
	constexpr int RS = (D + 1 + 3) / 4 * 4;
	const uint32_t rows = simt_rows(s.k);
	const uint32_t trows = rows < (uint32_t)SIMT_TILE_ROWS ? rows : (uint32_t)SIMT_TILE_ROWS;
	const size_t smem = (size_t)trows * RS * sizeof(float);
	const uint64_t per_block = (uint64_t)SIMT_THREADS * P;
	const uint64_t nblocks = (s.n + per_block - 1) / per_block;
	// persistent grid: a whole number of resident blocks per SM
	int per_sm = 1;
	// Near-tie band in value spacings (ulps of the common binade): roundings of this pass (|c|^2,
	// the offset, D fused steps, the centring of both operands), doubled for a difference of two
	// values, plus the reference's own sum and the collapse of its square root.
	const float margin_ulps = margin_scale * (float)(4 * D + 16);
	const int vec_ok = ((reinterpret_cast<uintptr_t>(pts) & 15u) == 0) ? 1 : 0;
#define BKM_LAUNCH_SIMT(SOA, FUSE) do { \
		auto kern = assign_simt_kernel<D, SOA, P, FUSE>; \
		cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
		if (e != cudaSuccess) return e; \
		e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, SIMT_THREADS, smem); \
		if (e != cudaSuccess) return e; \
		if (per_sm < 1) per_sm = 1; \
		uint32_t grid = (uint32_t)std::min<uint64_t>(nblocks, (uint64_t)sm_count * per_sm); \
		if (grid < 1) grid = 1; \
		kern<<<grid, SIMT_THREADS, smem, stream>>>(pts, cprep, center, asg, s.n, rows, ctl, slot, flag_list, margin_ulps, vec_ok, \
			s.k, fused ? fused->acc : nullptr, fused ? fused->counts : nullptr); \
	} while (0)
	if (fused && !assign_simt_can_fuse(s, *fused)) return cudaErrorInvalidValue;
	if (fused) { if (s.soa) BKM_LAUNCH_SIMT(true, true); else BKM_LAUNCH_SIMT(false, true); }
	else { if (s.soa) BKM_LAUNCH_SIMT(true, false); else BKM_LAUNCH_SIMT(false, false); }
#undef BKM_LAUNCH_SIMT
	return cudaGetLastError();
}

cudaError_t launch_assign_simt(const float* pts, const SimtMeans& sm, uint32_t* asg, const Shape& s,
	Control* ctl, int slot, uint32_t* flag_list, float margin_scale, int sm_count, cudaStream_t stream, const FusedAcc* fused)
{
	switch (s.dim) {
	case 1: return launch_simt_d<1, 4>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	case 2: return launch_simt_d<2, 4>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	case 3: return launch_simt_d<3, 2>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	case 4: return launch_simt_d<4, 2>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	case 5: return launch_simt_d<5, 2>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	case 6: return launch_simt_d<6, 2>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	case 7: return launch_simt_d<7, 2>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	case 8: return launch_simt_d<8, 2>(pts, sm.rows, sm.center, asg, s, ctl, slot, flag_list, margin_scale, sm_count, stream, fused);
	default: return cudaErrorInvalidValue;
	}
}

// max over the points of |x - center|^2 -> ctl->xmax2 (which must start at zero): one pass over
// the points, done once per data set (the key constants of the fast pass need the bound).
template<bool SOA>
__global__ void __launch_bounds__(256) points_norm_max_kernel(const float* __restrict__ pts, const float* __restrict__ center,
	uint64_t n, uint32_t d, Control* __restrict__ ctl, const uint32_t* __restrict__ skip_if)
{
	if (skip_if && *skip_if) return;
	float local = 0.0f;
	for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
		float s = 0.0f;
		for (uint32_t j = 0; j < d; ++j) {
			const float v = pts[at<SOA>(i, j, n, d)] - center[j];
			s = fmaf(v, v, s);
		}
		local = fmaxf(local, s);
	}
	#pragma unroll
	for (int off = 16; off > 0; off >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, off));
	// non-negative floats order like their bit patterns
	if ((threadIdx.x & 31u) == 0) atomicMax(reinterpret_cast<int*>(&ctl->xmax2), __float_as_int(local));
}

cudaError_t launch_points_norm_max(const float* pts, const Shape& s, const float* center, Control* ctl, int sm_count, cudaStream_t stream,
	const uint32_t* skip_if)
{
	const uint32_t grid = (uint32_t)std::min<uint64_t>((s.n + 255) / 256, (uint64_t)sm_count * 8);
	if (s.soa) points_norm_max_kernel<true><<<grid, 256, 0, stream>>>(pts, center, s.n, s.dim, ctl, skip_if);
	else points_norm_max_kernel<false><<<grid, 256, 0, stream>>>(pts, center, s.n, s.dim, ctl, skip_if);
	return cudaGetLastError();
}

} // namespace bkm
