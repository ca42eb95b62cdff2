// Assignment on the 5th-generation tensor cores (tcgen05 + TMEM), GEMM form.
//
//   |x - c|^2 = |x|^2 + ( |c|^2 - 2 x.c )          argmin over c ignores |x|^2
//
// The x.c contraction runs as split-TF32 ("3xTF32"): every fp32 operand is split once into a
// tf32 high part and a tf32 low part (x = xh + xl), and xl*ch + xh*cl + xh*ch is accumulated in
// fp32 in tensor memory, which restores fp32-level accuracy of the products.  |c|^2 and an offset
// constant enter the same accumulator through one more K step whose A operand is a constant
// tile, so the accumulator holds |c|^2 - 2 x.c + C, all values positive with one exponent, and
// the epilogue is a pure arg-min on integer keys.  The N x k distance
// matrix never exists in HBM.  Because the GEMM form cancels, a point whose best and
// second-best values are closer than the error band of this formulation is queued for the
// exact CUDA-core kernel, so the final assignment equals the reference arithmetic
// (headers/serial.hpp:21-35 of krulis-martin/cuda-kmeans) for every point.  The kernel covers
// the shape range of the reference's cachedRegsAssignmentKernel (kernels/kernels.cu:548-661).
//
// Kernel organisation (one persistent CTA per SM, 18 warps):
//   warp 0      : TMA producer.  dim <= 32: point tiles (128 points, hi and lo plane) go through a
//                 ring and stay for all mean tiles; mean tiles (up to 256 means, hi and lo, plus
//                 their |c|^2 K step) stream through a 2-stage ring, or stay when there is only
//                 one.  dim > 32: both operands stream in 32-dimension slices.
//   warp 1      : allocates the 512 TMEM columns and issues the tcgen05.mma instructions
//                 (kind::tf32, M=128, N<=256, K=8) into two accumulators, one per point tile of
//                 a block.  The whole warp walks the loop; one elected lane issues.
//   warps 2..17 : epilogue.  Eight warps per accumulator (TMEM lane quarter x column half), so
//                 that one accumulator is reduced while the other is being multiplied.  A warp
//                 reads its columns with tcgen05.ld two 32-column chunks at a time, hands the
//                 accumulator back after its last load, and reduces each chunk to (best, second)
//                 on integer keys; (best, second, chunk of best) per point stay in registers
//                 across all mean tiles and are merged through shared memory at the end.
// Mean sets of 2..4 tiles of 256 with 17 <= dim <= 32 run on CTA pairs instead, with all means
// resident in shared memory (assign_tc_pair.cu).
// All mbarrier waits are bounded; a wait that runs out sets STATUS_WAIT_TIMEOUT and lets every
// role fall through to the end, where TMEM is released.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "../../include/bkm.h"
#include "kernels.cuh"
#include "ptx.cuh"
#include "tc_common.cuh"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <new>

namespace bkm {

constexpr uint32_t A_PLANE_BYTES = TC_MTILE * TC_KCHUNK * 4;     // 16 KiB: 128 rows x 128 B
constexpr uint32_t B_PLANE_BYTES = TC_NT_MAX * TC_KCHUNK * 4;    // 32 KiB: 256 rows x 128 B
constexpr uint32_t A_TILE_BYTES = 2 * A_PLANE_BYTES;             // hi + lo
constexpr uint32_t B_STAGE_BYTES = 2 * B_PLANE_BYTES;
constexpr uint32_t AUG_BYTES = TC_NT_MAX * 8 * 4;                // 8 KiB: 256 rows x one K step of 8
// K-loop mode (dim > 32): both operands stream in 16-dimension slices (rows of 64 B, 64-byte
// swizzle).  A stage holds the slice of BOTH point tiles of the block and of one mean tile:
// [A0 hi | A0 lo | A1 hi | A1 lo | B hi | B lo], and feeds both accumulators, so every byte of
// the mean tile that crosses from L2 is used for 256 points.  Three stages; the |c|^2 steps of
// the current and the next mean tile sit behind them.
constexpr uint32_t KL_KW = 16;
constexpr uint32_t KL_STAGES = 3;
constexpr uint32_t KL_A_PLANE = TC_MTILE * KL_KW * 4;            // 8 KiB
constexpr uint32_t KL_B_PLANE = TC_NT_MAX * KL_KW * 4;           // 16 KiB
constexpr uint32_t KL_A1_OFF = 2 * KL_A_PLANE, KL_B_OFF = 4 * KL_A_PLANE;
constexpr uint32_t KL_STAGE_BYTES = KL_B_OFF + 2 * KL_B_PLANE;   // 64 KiB
constexpr uint32_t KL_AUG_OFF = KL_STAGES * KL_STAGE_BYTES;      // two |c|^2 steps of 8 KiB
constexpr uint32_t SM_A_OFF = 0;
constexpr uint32_t SM_B_OFF = SM_A_OFF + TC_MA * A_TILE_BYTES;
constexpr uint32_t SM_BAUG_OFF = SM_B_OFF + TC_NB * B_STAGE_BYTES; // |c|^2 K step per stage
constexpr uint32_t SM_AAUG_OFF = SM_BAUG_OFF + TC_NB * AUG_BYTES;  // constant ones tile (128 rows)
constexpr uint32_t SM_MERGE_OFF = SM_AAUG_OFF + TC_MTILE * 8 * 4;
constexpr uint32_t MERGE_BYTES = 2 * 3 * TC_MA * TC_MTILE * 4;   // (best, second, chunk) of the upper column half, two slots
constexpr uint32_t SM_FLAG_OFF = SM_MERGE_OFF + MERGE_BYTES;       // per epilogue warp: near-ties on their way to the list
constexpr uint32_t SM_BAR_OFF = SM_FLAG_OFF + TC_EPI_WARPS * FLAG_BUFFER * 4;
constexpr uint32_t SM_TOTAL = SM_BAR_OFF + 256;
constexpr uint32_t SM_ALLOC = SM_TOTAL + 1024;                   // slack for 1024-byte alignment

uint32_t tc_nt_cols(uint32_t k) { return k >= TC_NT_MAX ? TC_NT_MAX : round_up(k, 32); }
uint32_t tc_kpad(uint32_t k) { return round_up(k, tc_nt_cols(k)); }

bool assign_tc_supported(const Shape& s)
{
	return s.dim <= 4096 && tc_kpad(s.k) <= TC_MAX_KPAD && s.n < (1ull << 32) - 1024;
}

// ------------------------------------------------------------------------------------------
// one-off split of the points
// ------------------------------------------------------------------------------------------

// 32 points x 32 dims per step through a padded shared tile, so that both the read (along
// points for SoA, along dims for AoS) and the write (along dims) are coalesced.
template<bool SOA>
__global__ void __launch_bounds__(256) split_points_kernel(const float* __restrict__ pts, float* __restrict__ a_hi,
	float* __restrict__ a_lo, float* __restrict__ xnorm, uint64_t n, uint64_t p_begin, uint64_t p_end, uint32_t d, uint32_t d_pad,
	const float* __restrict__ center, Control* __restrict__ ctl, const uint32_t* __restrict__ skip_if)
{
	if (skip_if && *skip_if) return;
	float local_max = 0.0f;
	__shared__ float tile[32][33];
	const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
	// rows [p_begin, p_end) of the planes (both multiples of 32); rows at or behind n are padding
	for (uint64_t p0 = p_begin + (uint64_t)blockIdx.x * 32; p0 < p_end; p0 += (uint64_t)gridDim.x * 32) {
		float norm[4] = {0.f, 0.f, 0.f, 0.f};
		for (uint32_t c0 = 0; c0 < d_pad; c0 += 32) {
			__syncthreads();
			#pragma unroll
			for (uint32_t r = 0; r < 4; ++r) {
				const uint32_t rr = ty + r * 8;
				if (SOA) {
					const uint64_t p = p0 + tx;
					const uint32_t j = c0 + rr;
					tile[tx][rr] = (p < n && j < d) ? pts[(size_t)j * n + p] - center[j] : 0.0f;     // tile[point][dim]
				} else {
					const uint64_t p = p0 + rr;
					const uint32_t j = c0 + tx;
					tile[rr][tx] = (p < n && j < d) ? pts[(size_t)p * d + j] - center[j] : 0.0f;
				}
			}
			__syncthreads();
			#pragma unroll
			for (uint32_t r = 0; r < 4; ++r) {
				const uint32_t rr = ty + r * 8;     // point within the group
				const float x = tile[rr][tx];
				const float hi = to_tf32(x);
				const float lo = to_tf32(x - hi);
				const size_t o = (size_t)(p0 + rr) * d_pad + c0 + tx;
				if (c0 + tx < d_pad) {          // rows are shorter than the 32-wide step when d_pad = 16
					a_hi[o] = hi;
					a_lo[o] = lo;
				}
				norm[r] = fmaf(x, x, norm[r]);
			}
		}
		#pragma unroll
		for (uint32_t r = 0; r < 4; ++r) {
			float s = norm[r];
			#pragma unroll
			for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
			if (tx == 0) xnorm[p0 + ty + r * 8] = s;
			local_max = fmaxf(local_max, s);
		}
	}
	// non-negative floats order like their bit patterns
	if (tx == 0) atomicMax(reinterpret_cast<int*>(&ctl->xmax2), __float_as_int(local_max));
}

// One block per dimension: mean of that coordinate over at most 65536 evenly spaced points.
template<bool SOA>
__global__ void __launch_bounds__(256) compute_center_kernel(const float* __restrict__ pts, float* __restrict__ center,
	uint64_t n, uint64_t n_sampled, uint32_t d, const uint32_t* __restrict__ skip_if)
{
	if (skip_if && *skip_if) return;
	__shared__ float part[256];
	const uint32_t j = blockIdx.x;
	// the sample is taken from the first n_sampled points
	const uint64_t samples = n_sampled < 65536 ? n_sampled : 65536;
	const uint64_t stride = n_sampled / samples;
	float sum = 0.0f;
	for (uint64_t t = threadIdx.x; t < samples; t += 256) {
		const uint64_t i = t * stride;
		sum += SOA ? pts[(size_t)j * n + i] : pts[(size_t)i * d + j];
	}
	part[threadIdx.x] = sum;
	__syncthreads();
	for (uint32_t w = 128; w > 0; w >>= 1) {
		if (threadIdx.x < w) part[threadIdx.x] += part[threadIdx.x + w];
		__syncthreads();
	}
	if (threadIdx.x == 0) center[j] = part[0] / (float)samples;
}

cudaError_t launch_compute_center(const float* pts, const Shape& s, float* center, cudaStream_t stream, const uint32_t* skip_if,
	uint64_t n_sampled)
{
	if (n_sampled == 0 || n_sampled > s.n) n_sampled = s.n;
	if (s.soa) compute_center_kernel<true><<<s.dim, 256, 0, stream>>>(pts, center, s.n, n_sampled, s.dim, skip_if);
	else compute_center_kernel<false><<<s.dim, 256, 0, stream>>>(pts, center, s.n, n_sampled, s.dim, skip_if);
	return cudaGetLastError();
}

cudaError_t launch_split_points(const float* pts, const Shape& s, const TcPoints& tp, const float* center, Control* ctl, cudaStream_t stream,
	const uint32_t* skip_if, uint64_t p_begin, uint64_t p_end)
{
	if (p_end == 0 || p_end > tp.n_pad) p_end = tp.n_pad;
	if ((p_begin & 31u) != 0 || (p_end & 31u) != 0 || p_begin >= p_end) return cudaErrorInvalidValue;
	const uint64_t groups = (p_end - p_begin) / 32;
	const uint32_t grid = (uint32_t)std::min<uint64_t>(groups, (uint64_t)current_sm_count() * 16);
	if (s.soa) split_points_kernel<true><<<grid, 256, 0, stream>>>(pts, tp.a_hi, tp.a_lo, tp.xnorm, s.n, p_begin, p_end, s.dim, tp.d_pad, center, ctl, skip_if);
	else split_points_kernel<false><<<grid, 256, 0, stream>>>(pts, tp.a_hi, tp.a_lo, tp.xnorm, s.n, p_begin, p_end, s.dim, tp.d_pad, center, ctl, skip_if);
	return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// the assignment kernel
// ------------------------------------------------------------------------------------------

constexpr uint32_t TC_NA_MAX = 8;        // most point-tile buffers (single resident centroid tile, 16-float rows)

// The 3xTF32 products of one operand-tile pair over KS steps of 8 dimensions: the small cross
// terms lo*hi and hi*lo first, then the dominant hi*hi.  Operands are the low halves of the
// descriptors (+2 in the address field = 32 bytes = one K step), `hi_word` their common high half.
// `acc_first` = accumulate the very first product onto the destination.
template<uint32_t KS>
__device__ __forceinline__ void issue_products(uint32_t d_tmem, uint32_t a_hi, uint32_t a_lo, uint32_t b_hi, uint32_t b_lo,
	uint32_t hi_word, uint32_t idesc, uint32_t acc_first)
{
	ptx::mma_tf32_halves(d_tmem, a_lo, hi_word, b_hi, hi_word, idesc, acc_first);
	#pragma unroll
	for (uint32_t ks = 1; ks < KS; ++ks)
		ptx::mma_tf32_halves(d_tmem, a_lo + 2 * ks, hi_word, b_hi + 2 * ks, hi_word, idesc, 1);
	#pragma unroll
	for (uint32_t ks = 0; ks < KS; ++ks)
		ptx::mma_tf32_halves(d_tmem, a_hi + 2 * ks, hi_word, b_lo + 2 * ks, hi_word, idesc, 1);
	#pragma unroll
	for (uint32_t ks = 0; ks < KS; ++ks)
		ptx::mma_tf32_halves(d_tmem, a_hi + 2 * ks, hi_word, b_hi + 2 * ks, hi_word, idesc, 1);
}

struct TcBars {
	uint64_t a_full[TC_NA_MAX];
	uint64_t a_empty[TC_NA_MAX];
	uint64_t b_full[KL_STAGES];      // TC_NB of them in the resident-points modes
	uint64_t b_empty[KL_STAGES];
	uint64_t aug_full[2];            // K-loop mode: |c|^2 step of a mean tile has landed
	uint64_t aug_empty[2];
	uint64_t acc_full[TC_MA];
	uint64_t acc_empty[TC_MA];
	uint32_t tmem_slot;
	uint32_t abort_flag;
};
static_assert(sizeof(TcBars) <= 256, "barrier block too large");
static_assert(SM_ALLOC <= 227 * 1024, "shared memory budget exceeded");
static_assert(KL_AUG_OFF + 2 * AUG_BYTES <= SM_AAUG_OFF, "K-loop stages overlap the constant tile");

// The end of a point's arg-min: decode the winning key (key - key_base = M * mantissa + column) and
// write the assignment.  Returns whether best and second are closer than `margin`, i.e. whether
// the point has to be queued for the exact kernel (the caller appends, a warp at a time).
__device__ __forceinline__ bool finish_point(uint32_t best, uint32_t second, uint32_t bchunk, uint32_t key_base, uint32_t key_mult, uint32_t key_magic,
	float ulp, float margin, uint64_t p, uint32_t* __restrict__ asg)
{
	const uint32_t bm = div_key(best - key_base, key_magic);
	asg[p] = bchunk * 32u + ((best - key_base) - bm * key_mult);
	// keys are (mantissa * M + column): the difference of the quotients counts value spacings
	const float gap = second == 0xFFFFFFFFu ? INFINITY : (float)(div_key(second - key_base, key_magic) - bm) * ulp;
	return gap <= margin;
}

// Combines the partial arg-min results of the CTAs that shared the mean tiles of a point block.
__global__ void __launch_bounds__(256) merge_partials_kernel(const uint32_t* __restrict__ partial, uint64_t partial_stride, uint32_t parts,
	const float* __restrict__ xnorm, uint32_t* __restrict__ asg, uint64_t n, Control* __restrict__ ctl, int slot,
	uint32_t* __restrict__ flag_list, float margin_coef)
{
	const float c2max = ctl->cmax2[slot];
	const KeyConsts kc = make_key_consts(ctl->xmax2, c2max);
	const float ulp = kc.pow2 * 1.1920929e-07f;
	const uint64_t n32 = (n + 31) & ~(uint64_t)31;      // whole warps walk the loop together (the append is a warp operation)
	for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n32; p += (uint64_t)gridDim.x * blockDim.x) {
		bool flag = false;
		if (p < n) {
			uint32_t best = 0xFFFFFFFFu, second = 0xFFFFFFFFu, bchunk = 0;
			for (uint32_t part = 0; part < parts; ++part) {
				const uint32_t* src = partial + (size_t)part * 3 * partial_stride + p;
				const uint32_t ob = src[0], os = src[partial_stride], oc = src[2 * partial_stride];
				second = umin3(second, os, max(best, ob));
				bchunk = ob < best ? oc : bchunk;
				best = min(best, ob);
			}
			flag = finish_point(best, second, bchunk, kc.key_base, kc.key_mult, kc.key_magic, ulp, margin_coef * (xnorm[p] + c2max) + 4.0f * ulp, p, asg);
		}
		append_flagged(flag, (uint32_t)p, ctl, flag_list, n);
	}
}

// FULL: k is a whole number of mean tiles of 128 or 256 columns, so no accumulator column is padding
// and every warp takes its columns in pairs of 32-column chunks: the epilogue runs without its masked
// path and without the odd-chunk branches.
template<bool FULL>
__global__ void __launch_bounds__(TC_THREADS, 1) assign_tc_kernel(
	const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
	const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
	const float* __restrict__ b_aug, const float* __restrict__ xnorm, uint32_t* __restrict__ asg,
	uint64_t n, uint32_t n_tiles, uint32_t k, uint32_t k_pad, uint32_t nt_cols, uint32_t kw, uint32_t kchunks, uint32_t ksteps, uint32_t idesc,
	Control* __restrict__ ctl, int slot, uint32_t* __restrict__ flag_list, float margin_coef,
	uint32_t jsplit, uint32_t* __restrict__ partial, uint64_t partial_stride)
{
	extern __shared__ uint8_t smem_raw[];
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
	TcBars* bars = reinterpret_cast<TcBars*>(smem + SM_BAR_OFF);
	uint32_t* mg_state = reinterpret_cast<uint32_t*>(smem + SM_MERGE_OFF);
	volatile uint32_t* abort_flag = &bars->abort_flag;

	const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
	const uint32_t n_ctiles = k_pad / nt_cols;
	const uint32_t nblocks = (n_tiles + TC_MA - 1) / TC_MA;
	// With jsplit > 1, `jsplit` neighbouring CTAs work on the same block of points and share the
	// mean tiles among them (K loop with many mean tiles: the point tiles are re-read for every mean
	// tile, and fewer distinct point blocks in flight keep those re-reads in L2).  Each writes its
	// partial arg-min; merge_partials_kernel combines them.
	const uint32_t jpart = blockIdx.x % jsplit, bid = blockIdx.x / jsplit, nbid = gridDim.x / jsplit;
	const uint32_t jper = (n_ctiles + jsplit - 1) / jsplit;
	const uint32_t j_begin = min(n_ctiles, jpart * jper), j_end = min(n_ctiles, j_begin + jper);
	// Resident-points layout (dim <= 32).  With a single centroid tile (k <= 256) that tile is loaded
	// once and stays, and the space of the second stage holds two more point tiles, so that the
	// next block's points arrive while this block is still being multiplied.
	// Rows are kw = 32 floats (128 B) or, for dim <= 16, kw = 16 floats (64 B): half-size tiles.
	const bool b_resident = n_ctiles == 1;
	const uint32_t a_plane = TC_MTILE * kw * 4, a_tile = 2 * a_plane;
	const uint32_t b_plane = TC_NT_MAX * kw * 4, b_stage = 2 * b_plane;
	const uint32_t n_bstage = b_resident ? 1u : TC_NB;
	const uint32_t n_abuf = min(TC_NA_MAX, (SM_AAUG_OFF - n_bstage * (b_stage + AUG_BYTES)) / a_tile);
	const uint32_t sm_b_off = n_abuf * a_tile;
	const uint32_t sm_baug_off = sm_b_off + n_bstage * b_stage;

	if (threadIdx.x == 0) {
		for (uint32_t i = 0; i < TC_NA_MAX; ++i) {
			ptx::mbar_init(&bars->a_full[i], 1);
			ptx::mbar_init(&bars->a_empty[i], 1);
		}
		for (uint32_t i = 0; i < TC_MA; ++i) {
			ptx::mbar_init(&bars->acc_full[i], 1);
			ptx::mbar_init(&bars->acc_empty[i], TC_EPI_WARPS / TC_MA);
		}
		for (uint32_t i = 0; i < KL_STAGES; ++i) {
			ptx::mbar_init(&bars->b_full[i], 1);
			ptx::mbar_init(&bars->b_empty[i], 1);
		}
		for (uint32_t i = 0; i < 2; ++i) {
			ptx::mbar_init(&bars->aug_full[i], 1);
			ptx::mbar_init(&bars->aug_empty[i], 1);
		}
		bars->abort_flag = 0;
		ptx::fence_mbar_init();
	}
	if (warp == 1) {
		ptx::tmem_alloc(&bars->tmem_slot, TC_TMEM_COLS);
		ptx::tmem_relinquish();
	}
	const float x2max = ctl->xmax2, c2max = ctl->cmax2[slot];
	const KeyConsts kc = make_key_consts(x2max, c2max);
	const float pow2 = kc.pow2;
	const uint32_t key_mult = kc.key_mult, key_base = kc.key_base, key_magic = kc.key_magic;
	fill_a_aug(reinterpret_cast<float*>(smem + SM_AAUG_OFF), kc.offset_c, threadIdx.x, TC_THREADS);
	ptx::fence_proxy_async();
	ptx::tc_fence_before();
	__syncthreads();
	ptx::tc_fence_after();
	const uint32_t tmem_base = bars->tmem_slot;

	if (warp == 0) {
		// ---------------- TMA producer ----------------
		if (lane == 0) {
			ptx::prefetch_tmap(&tm_a_hi); ptx::prefetch_tmap(&tm_a_lo);
			ptx::prefetch_tmap(&tm_b_hi); ptx::prefetch_tmap(&tm_b_lo);
			uint32_t a_use[TC_NA_MAX] = {0, 0, 0, 0, 0, 0, 0, 0};
			uint32_t b_count = 0;
			bool ok = true;
			uint32_t aug_count = 0;
			if (kchunks > 1) {
				// K-loop mode: one (block of two point tiles, mean tile, 16-dimension slice) per stage
				for (uint32_t blk = bid; blk < nblocks && ok; blk += nbid) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t j = j_begin; j < j_end && ok; ++j) {
						{
							const uint32_t as = aug_count & 1u, au = aug_count >> 1;
							ok = wait_or_abort<400>(&bars->aug_empty[as], (au & 1u) ^ 1u, abort_flag);
							if (!ok) break;
							ptx::mbar_arrive_expect_tx(&bars->aug_full[as], nt_cols * 8 * 4);
							ptx::bulk_g2s(smem + KL_AUG_OFF + as * AUG_BYTES, b_aug + (size_t)j * nt_cols * 8, nt_cols * 8 * 4, &bars->aug_full[as]);
							++aug_count;
						}
						for (uint32_t kc = 0; kc < kchunks; ++kc) {
							const uint32_t s = b_count % KL_STAGES, u = b_count / KL_STAGES;
							ok = wait_or_abort<400>(&bars->b_empty[s], (u & 1u) ^ 1u, abort_flag);
							if (!ok) break;
							uint8_t* dst = smem + s * KL_STAGE_BYTES;
							const int32_t row = (int32_t)(blk * TC_MA * TC_MTILE), x = (int32_t)(kc * KL_KW);
							ptx::mbar_arrive_expect_tx(&bars->b_full[s], tiles * 2 * KL_A_PLANE + 2 * nt_cols * KL_KW * 4);
							ptx::tma_load_2d(dst, &tm_a_hi, x, row, &bars->b_full[s]);
							ptx::tma_load_2d(dst + KL_A_PLANE, &tm_a_lo, x, row, &bars->b_full[s]);
							if (tiles > 1) {
								ptx::tma_load_2d(dst + KL_A1_OFF, &tm_a_hi, x, row + (int32_t)TC_MTILE, &bars->b_full[s]);
								ptx::tma_load_2d(dst + KL_A1_OFF + KL_A_PLANE, &tm_a_lo, x, row + (int32_t)TC_MTILE, &bars->b_full[s]);
							}
							ptx::tma_load_2d(dst + KL_B_OFF, &tm_b_hi, x, (int32_t)(j * nt_cols), &bars->b_full[s]);
							ptx::tma_load_2d(dst + KL_B_OFF + KL_B_PLANE, &tm_b_lo, x, (int32_t)(j * nt_cols), &bars->b_full[s]);
							++b_count;
						}
					}
				}
			} else {
				uint32_t g = 0;                       // running count of point tiles = position in the A ring
				bool b_loaded = false;
				for (uint32_t blk = bid; blk < nblocks && ok; blk += nbid) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t i = 0; i < tiles && ok; ++i, ++g) {
						const uint32_t buf = g % n_abuf, u = g / n_abuf;
						ok = wait_or_abort<400>(&bars->a_empty[buf], (u & 1u) ^ 1u, abort_flag);
						if (!ok) break;
						uint8_t* dst = smem + SM_A_OFF + buf * a_tile;
						const int32_t row = (int32_t)((blk * TC_MA + i) * TC_MTILE);
						ptx::mbar_arrive_expect_tx(&bars->a_full[buf], a_tile);
						ptx::tma_load_2d(dst, &tm_a_hi, 0, row, &bars->a_full[buf]);
						ptx::tma_load_2d(dst + a_plane, &tm_a_lo, 0, row, &bars->a_full[buf]);
						++a_use[buf];
					}
					for (uint32_t j = j_begin; j < j_end && ok; ++j) {
						if (b_resident && b_loaded) break;
						const uint32_t s = b_count % TC_NB, u = b_count / TC_NB;
						ok = wait_or_abort<400>(&bars->b_empty[s], (u & 1u) ^ 1u, abort_flag);
						if (!ok) break;
						uint8_t* dst = smem + sm_b_off + s * b_stage;
						const uint32_t aug_bytes = nt_cols * 8 * 4;
						ptx::mbar_arrive_expect_tx(&bars->b_full[s], 2 * nt_cols * kw * 4 + aug_bytes);
						ptx::tma_load_2d(dst, &tm_b_hi, 0, (int32_t)(j * nt_cols), &bars->b_full[s]);
						ptx::tma_load_2d(dst + b_plane, &tm_b_lo, 0, (int32_t)(j * nt_cols), &bars->b_full[s]);
						ptx::bulk_g2s(smem + sm_baug_off + s * AUG_BYTES, b_aug + (size_t)j * nt_cols * 8, aug_bytes, &bars->b_full[s]);
						++b_count;
						b_loaded = true;
					}
				}
			}
			// Do not leave while an own copy may still be in flight towards this CTA's shared memory.
			for (uint32_t i = 0; i < TC_NA_MAX; ++i)
				if (a_use[i]) ptx::mbar_wait(&bars->a_full[i], (a_use[i] - 1) & 1u);
			const uint32_t ring = kchunks > 1 ? KL_STAGES : TC_NB;
			for (uint32_t back = 0; back < ring && back < b_count; ++back) {
				const uint32_t c = b_count - 1 - back;
				ptx::mbar_wait(&bars->b_full[c % ring], (c / ring) & 1u);
			}
			for (uint32_t back = 0; back < 2 && back < aug_count; ++back) {
				const uint32_t c = aug_count - 1 - back;
				ptx::mbar_wait(&bars->aug_full[c & 1u], (c >> 1) & 1u);
			}
		}
	} else if (warp == 1) {
		// ---------------- MMA issuer ----------------
		// The whole warp walks the loop (so that the address arithmetic is warp-uniform and stays
		// off the vector ALU, which the epilogue warps of the same scheduler keep busy); one
		// elected lane issues the tensor-core instructions.
		{
			uint32_t acc_use[TC_MA] = {0, 0};
			uint32_t b_count = 0;
			bool ok = true;
			const uint32_t a_aug_lo = desc_lo_aug(ptx::smem_u32(smem + SM_AAUG_OFF));
			const uint32_t desc_hi = kw == 32 ? DESC_HI_SW128 : DESC_HI_SW64;
			if (kchunks > 1) {
				// K-loop mode: both accumulators of the block collect the slices of one mean tile together
				uint32_t aug_count = 0;
				for (uint32_t blk = bid; blk < nblocks && ok; blk += nbid) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t j = j_begin; j < j_end && ok; ++j) {
						for (uint32_t i = 0; i < tiles && ok; ++i) {
							ok = wait_or_abort<200>(&bars->acc_empty[i], (acc_use[i] & 1u) ^ 1u, abort_flag);
							++acc_use[i];
						}
						if (!ok) break;
						ptx::tc_fence_after();
						for (uint32_t kc = 0; kc < kchunks; ++kc) {
							const uint32_t s = b_count % KL_STAGES, u = b_count / KL_STAGES;
							ok = wait_or_abort<100>(&bars->b_full[s], u & 1u, abort_flag);
							if (!ok) break;
							const bool last = kc == kchunks - 1;
							const uint32_t as = aug_count & 1u;
							if (last) {
								ok = wait_or_abort<100>(&bars->aug_full[as], (aug_count >> 1) & 1u, abort_flag);
								if (!ok) break;
							}
							ptx::tc_fence_after();
							const uint32_t base = ptx::smem_u32(smem + s * KL_STAGE_BYTES);
							const uint64_t b_hi = make_desc_kw(base + KL_B_OFF, KL_KW), b_lo = make_desc_kw(base + KL_B_OFF + KL_B_PLANE, KL_KW);
							const uint32_t steps = last ? ksteps : 2u;
							if (ptx::elect_one()) {
								for (uint32_t i = 0; i < tiles; ++i) {
									const uint32_t d_tmem = tmem_base + i * TC_NT_MAX;
									const uint64_t a_hi = make_desc_kw(base + i * KL_A1_OFF, KL_KW), a_lo = make_desc_kw(base + i * KL_A1_OFF + KL_A_PLANE, KL_KW);
									#pragma unroll
									for (uint32_t ks = 0; ks < 2; ++ks)
										if (ks < steps) ptx::mma_tf32(d_tmem, a_lo + 2 * ks, b_hi + 2 * ks, idesc, (kc | ks) > 0);
									#pragma unroll
									for (uint32_t ks = 0; ks < 2; ++ks)
										if (ks < steps) ptx::mma_tf32(d_tmem, a_hi + 2 * ks, b_lo + 2 * ks, idesc, 1);
									#pragma unroll
									for (uint32_t ks = 0; ks < 2; ++ks)
										if (ks < steps) ptx::mma_tf32(d_tmem, a_hi + 2 * ks, b_hi + 2 * ks, idesc, 1);
									if (last) {
										ptx::mma_tf32(d_tmem, make_desc_aug(ptx::smem_u32(smem + SM_AAUG_OFF)), make_desc_aug(ptx::smem_u32(smem + KL_AUG_OFF + as * AUG_BYTES)), idesc, 1);
										ptx::mma_commit(&bars->acc_full[i]);
									}
								}
								ptx::mma_commit(&bars->b_empty[s]);
								if (last) ptx::mma_commit(&bars->aug_empty[as]);
							}
							__syncwarp();
							++b_count;
						}
						++aug_count;
					}
				}
			} else {
				uint32_t g = 0;                       // position of the block's first tile in the A ring
				bool b_ready = false;
				for (uint32_t blk = bid; blk < nblocks && ok; blk += nbid) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t j = j_begin; j < j_end && ok; ++j) {
						const uint32_t s = b_resident ? 0u : b_count % TC_NB, u = b_count / TC_NB;
						if (!(b_resident && b_ready)) {
							ok = wait_or_abort<100>(&bars->b_full[s], u & 1u, abort_flag);
							if (!ok) break;
							b_ready = true;
						}
						const uint32_t b_addr = ptx::smem_u32(smem + sm_b_off + s * b_stage);
						const uint32_t b_hi = desc_lo_sw128(b_addr), b_lo = desc_lo_sw128(b_addr + b_plane);
						const uint32_t b_aug_lo = desc_lo_aug(ptx::smem_u32(smem + sm_baug_off + s * AUG_BYTES));
						for (uint32_t i = 0; i < tiles; ++i) {
							const uint32_t buf = (g + i) % n_abuf, ua = (g + i) / n_abuf;
							if (j == j_begin) {
								ok = wait_or_abort<100>(&bars->a_full[buf], ua & 1u, abort_flag);
								if (!ok) break;
							}
							ok = wait_or_abort<200>(&bars->acc_empty[i], (acc_use[i] & 1u) ^ 1u, abort_flag);
							if (!ok) break;
							ptx::tc_fence_after();
							const uint32_t a_addr = ptx::smem_u32(smem + SM_A_OFF + buf * a_tile);
							const uint32_t a_hi = desc_lo_sw128(a_addr), a_lo = desc_lo_sw128(a_addr + a_plane);
							const uint32_t d_tmem = tmem_base + i * TC_NT_MAX;
							if (ptx::elect_one()) {
								switch (ksteps) {
								case 4: issue_products<4>(d_tmem, a_hi, a_lo, b_hi, b_lo, desc_hi, idesc, 0); break;
								case 3: issue_products<3>(d_tmem, a_hi, a_lo, b_hi, b_lo, desc_hi, idesc, 0); break;
								case 2: issue_products<2>(d_tmem, a_hi, a_lo, b_hi, b_lo, desc_hi, idesc, 0); break;
								default: issue_products<1>(d_tmem, a_hi, a_lo, b_hi, b_lo, desc_hi, idesc, 0); break;
								}
								ptx::mma_tf32_halves(d_tmem, a_aug_lo, DESC_HI_AUG, b_aug_lo, DESC_HI_AUG, idesc, 1);
								ptx::mma_commit(&bars->acc_full[i]);
								if (j == j_end - 1) ptx::mma_commit(&bars->a_empty[buf]);
							}
							__syncwarp();
							++acc_use[i];
						}
						if (!ok) break;
						if (!b_resident) {
							if (ptx::elect_one()) ptx::mma_commit(&bars->b_empty[s]);
							__syncwarp();
							++b_count;
						}
					}
					g += tiles;
				}
			}
		}
	} else {
		// ---------------- epilogue ----------------
		// Warp (q, half, i): TMEM lane quarter q (the only lanes the warp may read), column half
		// `half` of accumulator i.  The eight warps of one accumulator work while the other
		// accumulator is being multiplied, so on every scheduler two warps read tensor memory while
		// the other two keep the integer pipes busy.  A warp takes its columns two 32-column chunks
		// at a time into registers and hands the accumulator back after its last load.
		// The loops are kept rolled on purpose: unrolled, the arg-min code outgrows the instruction
		// cache and the warps starve on instruction fetch.
		const uint32_t q = warp & 3u;
		const uint32_t part = (warp - 2) >> 2;     // 0..3
		const uint32_t i = part >> 1;              // accumulator = point tile within the block
		const uint32_t half = part & 1u;
		const uint32_t row = q * 32 + lane;
		const float ulp = pow2 * 1.1920929e-07f;   // spacing of the values inside [P, 2P)
		const uint32_t chunks_total = nt_cols >> 5;                    // 1..8
		const uint32_t per_half = (chunks_total + 1) / 2;              // 1..4
		const uint32_t first_chunk = half * per_half;
		const uint32_t nchunks = first_chunk >= chunks_total ? 0u : min(per_half, chunks_total - first_chunk);
		const uint32_t bar_id = 1u + i * 4u + q;   // named barrier of the two warps that share these rows
		uint32_t* flag_buf = reinterpret_cast<uint32_t*>(smem + SM_FLAG_OFF) + (warp - 2) * FLAG_BUFFER;
		uint32_t flag_cnt = 0;
		uint32_t acc_use = 0, blk_count = 0;
		bool ok = true;
		for (uint32_t blk = bid; blk < nblocks; blk += nbid, ++blk_count) {
			const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
			if (i >= tiles) continue;              // odd tail: this accumulator is not used in the last block
			uint32_t best = 0xFFFFFFFFu, second = 0xFFFFFFFFu, bchunk = 0;
			const uint64_t p = (uint64_t)(blk * TC_MA + i) * TC_MTILE + row;
			float xn = 0.0f;                       // |x|^2 of this thread's point, needed at the end of the block
			#pragma unroll 1
			for (uint32_t j = j_begin; j < j_end; ++j) {
				// the whole warp polls (one warp instruction either way, and no divergent region around it)
				if (ok) ok = __all_sync(0xffffffffu, wait_or_abort<100>(&bars->acc_full[i], acc_use & 1u, abort_flag)) != 0;
				++acc_use;
				if (ok && nchunks > 0) {
					ptx::tc_fence_after();
					#pragma unroll 1
					for (uint32_t c = 0; c < nchunks; c += 2) {
						const uint32_t colbase = (first_chunk + c) * 32u;
						const uint32_t taddr = tmem_base + ((q * 32u) << 16) + i * TC_NT_MAX + colbase;
						const uint32_t chunk0 = (j * nt_cols + colbase) >> 5;
						const bool two = FULL ? true : c + 1 < nchunks;
						uint32_t v0[32], v1[32];
						const uint32_t col0 = chunk0 * 32u;
						// columns at or behind k are padding
						const uint32_t left = FULL ? 64u : (k > col0 ? k - col0 : 0u);
						const bool plain = FULL || left >= 64 || (!two && left >= 32);
						// the second chunk travels from tensor memory while the first is reduced
						ptx::tmem_ld32(taddr, v0);
						ptx::tmem_ld_wait();
						if (two) ptx::tmem_ld32(taddr + 32, v1);
						if (plain) chunk_update<false>(v0, key_mult, chunk0, 32, best, second, bchunk);
						else if (left > 0) chunk_update<true>(v0, key_mult, chunk0, left, best, second, bchunk);
						ptx::tmem_ld_wait();
						if (c + 2 >= nchunks) {
							// last load: the tensor cores may fill this accumulator again
							ptx::tc_fence_before();
							__syncwarp();
							if (lane == 0) ptx::mbar_arrive(&bars->acc_empty[i]);
							// fetched behind the hand-back of the block's last accumulator: the arithmetic on
							// the chunks just loaded covers the latency
							if (j == j_end - 1 && half == 0 && p < n) xn = xnorm[p];
						}
						if (plain) {
							if (two) chunk_update<false>(v1, key_mult, chunk0 + 1, 32, best, second, bchunk);
						} else if (two && left > 32) {
							chunk_update<true>(v1, key_mult, chunk0 + 1, left - 32, best, second, bchunk);
						}
					}
				} else {
					__syncwarp();
					if (lane == 0) ptx::mbar_arrive(&bars->acc_empty[i]);
				}
			}
			// The upper column half hands its state to the lower one through shared memory.  The slots
			// alternate with the block count, so one barrier per block is enough: a slot is written
			// again only after its reader has passed the barrier of the block in between.
			uint32_t* mg = mg_state + ((blk_count & 1u) * TC_MA + i) * (3 * TC_MTILE);
			if (half == 1) {
				mg[row] = best; mg[TC_MTILE + row] = second; mg[2 * TC_MTILE + row] = bchunk;
			}
			asm volatile("bar.sync %0, 64;" :: "r"(bar_id) : "memory");
			bool flag = false;
			if (half == 0 && p < n && ok) {
				const uint32_t ob = mg[row], os = mg[TC_MTILE + row], oc = mg[2 * TC_MTILE + row];
				second = umin3(second, os, max(best, ob));
				bchunk = ob < best ? oc : bchunk;
				best = min(best, ob);
				if (partial != nullptr) {
					// this CTA saw only its share of the mean tiles: the keys go out as they are
					uint32_t* dst = partial + (size_t)jpart * 3 * partial_stride + p;
					dst[0] = best; dst[partial_stride] = second; dst[2 * partial_stride] = bchunk;
				} else {
					flag = finish_point(best, second, bchunk, key_base, key_mult, key_magic, ulp, margin_coef * (xn + c2max) + 4.0f * ulp, p, asg);
				}
			}
			if (half == 0 && partial == nullptr) buffered_append(flag, (uint32_t)p, flag_buf, flag_cnt, ctl, flag_list, n);
		}
		flush_flag_buffer(flag_buf, flag_cnt, ctl, flag_list, n);
	}

	ptx::tc_fence_before();
	__syncthreads();
	if (warp == 1) {
		__syncwarp();
		ptx::tc_fence_after();
		ptx::tmem_dealloc(tmem_base, TC_TMEM_COLS);
	}
	if (threadIdx.x == 0 && bars->abort_flag) atomicOr(&ctl->status, (uint32_t)STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------------------------------
// self-test of the bounded wait
// ------------------------------------------------------------------------------------------

// One thread waits for a barrier phase that nothing will ever complete, with a short limit, and
// reports through the status word exactly as the assignment kernels do when a wait runs out.
__global__ void wait_timeout_selftest_kernel(Control* ctl, uint64_t limit_ns)
{
	__shared__ uint64_t bar;
	if (threadIdx.x == 0) {
		ptx::mbar_init(&bar, 1);
		ptx::fence_mbar_init();
		if (!ptx::mbar_wait(&bar, 0, limit_ns)) atomicOr(&ctl->status, (uint32_t)STATUS_WAIT_TIMEOUT);
	}
}

cudaError_t launch_wait_timeout_selftest(Control* ctl, uint64_t limit_ns, cudaStream_t stream)
{
	wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(ctl, limit_ns);
	return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------

struct TcPlan {
	CUtensorMap a_hi, a_lo, b_hi, b_lo;
	CUtensorMap bh_hi, bh_lo;       // the means in boxes of 128 rows: one CTA's half of a tile (pair kernel)
	bool pair_ok;                   // the CTA-pair kernel covers this shape
	bool pair_allowed;
	int max_pairs;                  // CTA pairs the device holds at once
	Shape s;
	TcPoints tp;
	TcMeans tm;
	uint32_t nt_cols;
	uint32_t idesc;
	int sm_count;
};

static PFN_cuTensorMapEncodeTiled_v12000 get_encode()
{
	static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
	static bool tried = false;
	if (!tried) {
		tried = true;
		void* p = nullptr;
		cudaDriverEntryPointQueryResult qres;
		if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
			qres == cudaDriverEntryPointSuccess)
			fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
	}
	return fn;
}

// [rows][cols] fp32 row-major, box = box_rows x 32 columns with 128-byte swizzle, or, when the
// rows are only 16 floats long or the K loop runs (rows longer than 32 floats, 16-dimension
// slices), box_rows x 16 columns with 64-byte swizzle.
static bool encode_plane(CUtensorMap* out, const float* base, uint64_t rows, uint32_t cols, uint32_t box_rows)
{
	const uint32_t kw = (cols == 16 || cols > TC_KCHUNK) ? 16u : TC_KCHUNK;
	auto enc = get_encode();
	if (!enc) return false;
	cuuint64_t dims[2] = {cols, rows};
	cuuint64_t strides[1] = {(cuuint64_t)cols * sizeof(float)};
	cuuint32_t box[2] = {kw, box_rows};
	cuuint32_t estr[2] = {1, 1};
	CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
		CU_TENSOR_MAP_INTERLEAVE_NONE, kw == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
		CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	return r == CUDA_SUCCESS;
}

TcPlan* tc_plan_create(const Shape& s, const TcPoints& tp, const TcMeans& tm, int device, const char** err)
{
	static const char* e_sup = "shape not supported by the tensor-core assignment";
	static const char* e_map = "cuTensorMapEncodeTiled failed or is unavailable";
	static const char* e_attr = "cannot set the shared-memory size of the tensor-core kernel";
	if (!assign_tc_supported(s) || tp.d_pad != tm.d_pad || (tp.d_pad != 16 && tp.d_pad % TC_KCHUNK != 0)) { if (err) *err = e_sup; return nullptr; }
	TcPlan* p = new (std::nothrow) TcPlan();
	if (!p) return nullptr;
	p->s = s; p->tp = tp; p->tm = tm;
	p->nt_cols = tc_nt_cols(s.k);
	// c_format = f32 (bit 4), a/b format = tf32 (bits 7.., 10..), K-major both, N>>3 at bit 17, M>>4 at bit 24
	p->idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((p->nt_cols >> 3) << 17) | ((TC_MTILE >> 4) << 24);
	if (cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || p->sm_count < 1) { cudaGetLastError(); if (err) *err = e_attr; delete p; return nullptr; }
	if (!encode_plane(&p->a_hi, tp.a_hi, tp.n_pad, tp.d_pad, TC_MTILE) ||
		!encode_plane(&p->a_lo, tp.a_lo, tp.n_pad, tp.d_pad, TC_MTILE) ||
		!encode_plane(&p->b_hi, tm.b_hi, tm.k_pad, tm.d_pad, p->nt_cols) ||
		!encode_plane(&p->b_lo, tm.b_lo, tm.k_pad, tm.d_pad, p->nt_cols)) {
		if (err) *err = e_map;
		delete p;
		return nullptr;
	}
	if (cudaFuncSetAttribute(assign_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM_ALLOC) != cudaSuccess ||
		cudaFuncSetAttribute(assign_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM_ALLOC) != cudaSuccess) {
		cudaGetLastError();
		if (err) *err = e_attr;
		delete p;
		return nullptr;
	}
	p->pair_allowed = true;
	p->pair_ok = assign_tc_pair_supported(s.k, tm.k_pad, tp.d_pad, p->nt_cols, p->sm_count) &&
		encode_plane(&p->bh_hi, tm.b_hi, tm.k_pad, tm.d_pad, TC_NT_MAX / 2) &&
		encode_plane(&p->bh_lo, tm.b_lo, tm.k_pad, tm.d_pad, TC_NT_MAX / 2);
	p->max_pairs = 0;
	if (p->pair_ok && (assign_tc_pair_prepare(p->sm_count, &p->max_pairs) != cudaSuccess || p->max_pairs < 1)) {
		cudaGetLastError();
		p->pair_ok = false;
	}
	return p;
}

void tc_plan_allow_pair(TcPlan* plan, bool allow) { if (plan) plan->pair_allowed = allow; }
bool tc_plan_uses_pair(const TcPlan* plan) { return plan && plan->pair_ok && plan->pair_allowed; }

void tc_plan_destroy(TcPlan* plan) { delete plan; }

// The pair kernel can accumulate the update sums when a point's row can go out as 128-bit vector
// reductions: dim a multiple of 4 and 16-byte aligned accumulators.
bool tc_plan_can_fuse(const TcPlan* p, const FusedAcc& f)
{
	return tc_plan_uses_pair(p) && p->s.dim % 4 == 0 && f.acc != nullptr && f.counts != nullptr && f.center != nullptr &&
		(reinterpret_cast<uintptr_t>(f.acc) & 15u) == 0 && (f.rep_stride * sizeof(float)) % 16 == 0;
}

// K loop with several mean tiles: pairs of neighbouring CTAs share a point block (see the kernel)
static uint32_t plan_jsplit(const TcPlan* p)
{
	const bool kloop = p->tp.d_pad > TC_KCHUNK;
	const uint32_t n_ctiles = p->tm.k_pad / p->nt_cols;
	return (kloop && n_ctiles >= 2 * TC_JSPLIT && p->tp.partial != nullptr && p->sm_count >= (int)TC_JSPLIT) ? TC_JSPLIT : 1u;
}

void tc_plan_describe(const TcPlan* p, uint32_t out[4])
{
	out[1] = p->tm.k_pad / p->nt_cols;
	out[2] = 1;
	if (tc_plan_uses_pair(p)) { out[0] = BKM_PLAN_TC_PAIR; return; }
	out[0] = p->tp.d_pad > TC_KCHUNK ? BKM_PLAN_TC_KLOOP : BKM_PLAN_TC_RESIDENT;
	out[2] = plan_jsplit(p);
}

cudaError_t launch_assign_tc(TcPlan* p, uint32_t* asg, Control* ctl, int slot, uint32_t* flag_list,
	float margin_scale, cudaStream_t stream, const FusedAcc* fused, uint64_t p_begin, uint64_t p_end)
{
	if (!p) return cudaErrorInvalidValue;
	if (fused && !tc_plan_can_fuse(p, *fused)) return cudaErrorInvalidValue;
	// a range of the points: CTA pairs only, in whole steps of two point tiles
	const bool ranged = p_begin != 0 || p_end != 0;
	if (ranged && (!tc_plan_uses_pair(p) || p_begin % (2 * TC_MTILE) != 0 || (p_end % (2 * TC_MTILE) != 0 && p_end < p->s.n))) return cudaErrorInvalidValue;
	const uint32_t n_tiles = (uint32_t)(p->tp.n_pad / TC_MTILE);
	const uint32_t nblocks = (n_tiles + TC_MA - 1) / TC_MA;
	const uint32_t grid = std::min<uint32_t>(nblocks, (uint32_t)p->sm_count);
	// error band of the split-TF32 GEMM form relative to |x|^2 + max|c|^2
	const float margin_coef = margin_scale * (48.0f + 0.5f * (float)p->tp.d_pad) * 1.1920929e-07f;
	// rows of 16 or 32 floats stay resident whole; longer rows stream in 16-dimension slices, and
	// slices that hold padding only are skipped
	const bool kloop = p->tp.d_pad > TC_KCHUNK;
	const uint32_t kw = (p->tp.d_pad == 16 || kloop) ? 16u : TC_KCHUNK;
	const uint32_t kchunks = kloop ? (p->s.dim + kw - 1) / kw : 1u;
	const uint32_t ksteps_last = (p->s.dim - (kchunks - 1) * kw + 7) / 8;    // K steps of the last slice
	const uint32_t idesc = p->idesc;
	if (tc_plan_uses_pair(p))
		return launch_assign_tc_pair(p->a_hi, p->a_lo, p->bh_hi, p->bh_lo, p->tm.b_aug, p->tp.xnorm, asg, p->s.n, n_tiles,
			p->s.k, p->tm.k_pad, p->tp.d_pad, ksteps_last, p->max_pairs, ctl, slot, flag_list, margin_coef, stream, fused, p->s.dim,
			ranged ? (uint32_t)(p_begin / (2 * TC_MTILE)) : 0u,
			ranged ? (uint32_t)((std::min<uint64_t>(p_end, p->tp.n_pad) + 2 * TC_MTILE - 1) / (2 * TC_MTILE)) : 0u);
	const uint32_t jsplit = plan_jsplit(p);
	const uint32_t grid_j = jsplit * std::min<uint32_t>(nblocks, (uint32_t)p->sm_count / jsplit);
	auto kern = (p->s.k == p->tm.k_pad && p->nt_cols % 128 == 0) ? assign_tc_kernel<true> : assign_tc_kernel<false>;
	kern<<<jsplit > 1 ? grid_j : grid, TC_THREADS, SM_ALLOC, stream>>>(p->a_hi, p->a_lo, p->b_hi, p->b_lo,
		p->tm.b_aug, p->tp.xnorm, asg, p->s.n, n_tiles, p->s.k, p->tm.k_pad, p->nt_cols, kw, kchunks, ksteps_last, idesc,
		ctl, slot, flag_list, margin_coef, jsplit, jsplit > 1 ? p->tp.partial : nullptr, p->tp.n_pad);
	if (jsplit > 1) {
		const uint32_t mgrid = (uint32_t)std::min<uint64_t>((p->s.n + 255) / 256, (uint64_t)p->sm_count * 8);
		merge_partials_kernel<<<mgrid, 256, 0, stream>>>(p->tp.partial, p->tp.n_pad, jsplit, p->tp.xnorm, asg, p->s.n, ctl, slot,
			flag_list, margin_coef);
	}
	return cudaGetLastError();
}

} // namespace bkm
