// Assignment on the 5th-generation tensor cores (tcgen05 + TMEM), GEMM form.
//
//   |x - c|^2 = |x|^2 + ( |c|^2 - 2 x.c )          argmin over c ignores |x|^2
//
// The x.c contraction runs as split-TF32 ("3xTF32"): every fp32 operand is split once into a
// tf32 high part and a tf32 low part (x = xh + xl), and xl*ch + xh*cl + xh*ch is accumulated in
// fp32 in tensor memory, which restores fp32-level accuracy of the products.  |c|^2 enters the
// same accumulator through one more K step whose A operand is a constant tile of ones, so the
// accumulator holds |c|^2 - 2 x.c and the epilogue is a pure arg-min.  The N x k distance
// matrix never exists in HBM.  Because the GEMM form cancels, a point whose best and
// second-best values are closer than the error band of this formulation is queued for the
// exact CUDA-core kernel, so the final assignment equals the reference arithmetic
// (headers/serial.hpp:21-35 of krulis-martin/cuda-kmeans) for every point.  The kernel covers
// the shape range of the reference's cachedRegsAssignmentKernel (kernels/kernels.cu:548-661).
//
// Kernel organisation (one persistent CTA per SM, 10 warps):
//   warp 0     : TMA producer.  Point tiles (128 points x 32 dims, hi and lo plane) are loaded
//                once per block of 4 tiles and stay in shared memory; centroid tiles (up to 128
//                centroids x 32 dims, hi and lo, plus their |c|^2 K step) stream through a
//                2-stage ring.
//   warp 1     : allocates the 512 TMEM columns and issues the tcgen05.mma instructions
//                (kind::tf32, M=128, N<=128, K=8).  Back-to-back MMAs into ONE accumulator are
//                bound by the accumulate latency, not by the tensor work, so the K steps of two
//                accumulators are issued interleaved.
//   warps 2..9 : epilogue.  Two warps per 32-lane TMEM quarter; the pair alternates over the
//                point tiles, so that one computes while the other waits for tensor memory.
//                Each reads its accumulator rows with tcgen05.ld, packs the column position
//                into the low mantissa bits, and reduces 32 columns at a time to (best, second)
//                with a min/max tournament; (best, second, chunk of best) per point stay in
//                registers across all centroid tiles.
// All mbarrier waits are bounded; a wait that runs out sets STATUS_WAIT_TIMEOUT and lets every
// role fall through to the end, where TMEM is released.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "kernels.cuh"
#include "ptx.cuh"

#include <cmath>
#include <cstdlib>
#include <new>

// Optional stage timing for development builds (-DBKM_TC_TIMING): one CTA prints how its MMA warp
// and three of its epilogue warps spent their cycles.
#ifdef BKM_TC_TIMING
#include <cstdio>
#define TC_T(var) const long long var = clock64()
#define TC_ACC(sum, from, to) sum += (to) - (from)
#else
#define TC_T(var)
#define TC_ACC(sum, from, to)
#endif

namespace bkm {

constexpr uint32_t TC_MA = 2;            // point tiles per block (= TMEM accumulators)
constexpr uint32_t TC_NB = 2;            // centroid-tile stages
constexpr uint32_t TC_NT_MAX = 256;      // centroids per tile (the widest MMA: N = 256)
constexpr uint32_t TC_EPI_WARPS = 16;          // four per TMEM lane quarter, each a quarter of the columns
constexpr uint32_t TC_THREADS = (2 + TC_EPI_WARPS) * 32;
constexpr uint32_t TC_MAX_KPAD = 1u << 20;
constexpr uint32_t TC_TMEM_COLS = 512;

constexpr uint32_t A_PLANE_BYTES = TC_MTILE * TC_KCHUNK * 4;     // 16 KiB: 128 rows x 128 B
constexpr uint32_t B_PLANE_BYTES = TC_NT_MAX * TC_KCHUNK * 4;    // 32 KiB: 256 rows x 128 B
constexpr uint32_t A_TILE_BYTES = 2 * A_PLANE_BYTES;             // hi + lo
constexpr uint32_t B_STAGE_BYTES = 2 * B_PLANE_BYTES;
constexpr uint32_t AUG_BYTES = TC_NT_MAX * 8 * 4;                // 8 KiB: 256 rows x one K step of 8
// K-loop mode (dim > 32): both operands stream, one 32-dimension slice per stage:
// [A hi | A lo | B hi | B lo | B's |c|^2 step]; two such stages fill the same bytes as the
// resident-points layout below.
constexpr uint32_t KSTAGE_BYTES = A_TILE_BYTES + B_STAGE_BYTES + AUG_BYTES;
constexpr uint32_t KS_ALO_OFF = A_PLANE_BYTES, KS_BHI_OFF = A_TILE_BYTES, KS_BLO_OFF = A_TILE_BYTES + B_PLANE_BYTES,
	KS_AUG_OFF = A_TILE_BYTES + B_STAGE_BYTES;
constexpr uint32_t SM_A_OFF = 0;
constexpr uint32_t SM_B_OFF = SM_A_OFF + TC_MA * A_TILE_BYTES;
constexpr uint32_t SM_BAUG_OFF = SM_B_OFF + TC_NB * B_STAGE_BYTES; // |c|^2 K step per stage
constexpr uint32_t SM_AAUG_OFF = SM_BAUG_OFF + TC_NB * AUG_BYTES;  // constant ones tile (128 rows)
constexpr uint32_t SM_MERGE_OFF = SM_AAUG_OFF + TC_MTILE * 8 * 4;
constexpr uint32_t MERGE_BYTES = 3 * 3 * TC_MA * TC_MTILE * 4;   // (best, second, chunk) of column parts 1..3
constexpr uint32_t SM_BAR_OFF = SM_MERGE_OFF + MERGE_BYTES;
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

__device__ __forceinline__ float to_tf32(float x)
{
	uint32_t u;
	asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
	return __uint_as_float(u);
}

// 32 points x 32 dims per step through a padded shared tile, so that both the read (along
// points for SoA, along dims for AoS) and the write (along dims) are coalesced.
template<bool SOA>
__global__ void __launch_bounds__(256) split_points_kernel(const float* __restrict__ pts, float* __restrict__ a_hi,
	float* __restrict__ a_lo, float* __restrict__ xnorm, uint64_t n, uint64_t n_pad, uint32_t d, uint32_t d_pad,
	const float* __restrict__ center, Control* __restrict__ ctl)
{
	float local_max = 0.0f;
	__shared__ float tile[32][33];
	const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
	for (uint64_t p0 = (uint64_t)blockIdx.x * 32; p0 < n_pad; p0 += (uint64_t)gridDim.x * 32) {
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
	uint64_t n, uint32_t d)
{
	__shared__ float part[256];
	const uint32_t j = blockIdx.x;
	const uint64_t samples = n < 65536 ? n : 65536;
	const uint64_t stride = n / samples;
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

cudaError_t launch_compute_center(const float* pts, const Shape& s, float* center, cudaStream_t stream)
{
	if (s.soa) compute_center_kernel<true><<<s.dim, 256, 0, stream>>>(pts, center, s.n, s.dim);
	else compute_center_kernel<false><<<s.dim, 256, 0, stream>>>(pts, center, s.n, s.dim);
	return cudaGetLastError();
}

cudaError_t launch_split_points(const float* pts, const Shape& s, const TcPoints& tp, const float* center, Control* ctl, cudaStream_t stream)
{
	const uint64_t groups = tp.n_pad / 32;
	const uint32_t grid = (uint32_t)std::min<uint64_t>(groups, 148 * 16);
	if (s.soa) split_points_kernel<true><<<grid, 256, 0, stream>>>(pts, tp.a_hi, tp.a_lo, tp.xnorm, s.n, tp.n_pad, s.dim, tp.d_pad, center, ctl);
	else split_points_kernel<false><<<grid, 256, 0, stream>>>(pts, tp.a_hi, tp.a_lo, tp.xnorm, s.n, tp.n_pad, s.dim, tp.d_pad, center, ctl);
	return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// the assignment kernel
// ------------------------------------------------------------------------------------------

constexpr uint32_t TC_NA_MAX = 8;        // most point-tile buffers (single resident centroid tile, 16-float rows)

struct TcBars {
	uint64_t a_full[TC_NA_MAX];
	uint64_t a_empty[TC_NA_MAX];
	uint64_t b_full[TC_NB];
	uint64_t b_empty[TC_NB];
	uint64_t acc_full[TC_MA];
	uint64_t acc_empty[TC_MA];
	uint32_t tmem_slot;
	uint32_t abort_flag;
};
static_assert(sizeof(TcBars) <= 256, "barrier block too large");
static_assert(SM_ALLOC <= 227 * 1024, "shared memory budget exceeded");
static_assert(TC_NB * KSTAGE_BYTES <= SM_AAUG_OFF, "K-loop stages overlap the constant tile");

// Bounded wait that also gives up when another role already failed.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag)
{
	if (ptx::mbar_try_wait(bar, parity)) return true;
	const uint64_t t0 = ptx::globaltimer_ns();
	while (true) {
		if (ptx::mbar_try_wait(bar, parity)) return true;
		if (*abort_flag) return false;
		if (ptx::globaltimer_ns() - t0 > ptx::WAIT_LIMIT_NS) break;
	}
	*abort_flag = 1;
	return false;
}

// K-major operand, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr)
{
	return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Same for rows of `kw` floats: kw = 32 as above, kw = 16 -> 64-byte swizzle, rows of 64 B,
// 8-row groups 512 B apart.
__device__ __forceinline__ uint64_t make_desc_kw(uint32_t smem_addr, uint32_t kw)
{
	return kw == 32 ? make_desc(smem_addr)
		: ((uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (32ull << 32) | (1ull << 46) | (4ull << 61));
}

// K-major operand without swizzle, one K step (8 tf32 = two 16-byte chunks) wide: 8x16-byte core
// matrices; the two chunks of a row group are 128 B apart, row groups 256 B apart.
__device__ __forceinline__ uint64_t make_desc_aug(uint32_t smem_addr)
{
	return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (8ull << 16) | (16ull << 32) | (1ull << 46);
}

__device__ __forceinline__ uint32_t umin3(uint32_t a, uint32_t b, uint32_t c) { return __vimin3_u32(a, b, c); }

// Smallest and second-smallest of 32 keys by a tournament: 16 (min,max) pairs, then 15 merges
// (b,s) x (b',s') -> (min(b,b'), min(max(b,b'), s, s')).  77 instructions, log depth.
__device__ __forceinline__ void top2_of_32(const uint32_t (&p)[32], uint32_t& b, uint32_t& s)
{
	uint32_t lo[16], hi[16];
	#pragma unroll
	for (int i = 0; i < 16; ++i) { lo[i] = min(p[2 * i], p[2 * i + 1]); hi[i] = max(p[2 * i], p[2 * i + 1]); }
	#pragma unroll
	for (int n = 16; n > 1; n >>= 1) {
		#pragma unroll
		for (int i = 0; i < n / 2; ++i) {
			const uint32_t nb = min(lo[2 * i], lo[2 * i + 1]);
			const uint32_t ns = umin3(max(lo[2 * i], lo[2 * i + 1]), hi[2 * i], hi[2 * i + 1]);
			lo[i] = nb;
			hi[i] = ns;
		}
	}
	b = lo[0];
	s = hi[0];
}

// One 32-column chunk of an accumulator row.  The kernel adds a constant to every value so that
// all of them are positive floats with the SAME exponent; their bit patterns then order like the
// values, the upper exponent bits carry no information, and bits*32 + column (one integer
// multiply-add, off the min/max pipe) is a key that keeps the full 23-bit mantissa and carries
// the column position.  The keys are reduced to the two smallest and merged into the running
// (best, second, chunk of best).  `nvalid` < 32 masks the padding columns behind the last mean.
template<bool MASKED>
__device__ __forceinline__ void chunk_update(const uint32_t (&v)[32], uint32_t chunk_id, uint32_t nvalid,
	uint32_t& best, uint32_t& second, uint32_t& best_chunk)
{
	uint32_t p[32];
	#pragma unroll
	for (uint32_t t = 0; t < 32; ++t) p[t] = v[t] * 32u + t;
	if (MASKED && nvalid < 32) {
		#pragma unroll
		for (uint32_t t = 0; t < 32; ++t) p[t] = t < nvalid ? p[t] : 0xFFFFFFFFu;
	}
	uint32_t b, s2;
	top2_of_32(p, b, s2);
	second = umin3(second, max(best, b), s2);
	best_chunk = b < best ? chunk_id : best_chunk;
	best = min(best, b);
}

__global__ void __launch_bounds__(TC_THREADS, 1) assign_tc_kernel(
	const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
	const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
	const float* __restrict__ b_aug, const float* __restrict__ xnorm, uint32_t* __restrict__ asg,
	uint64_t n, uint32_t n_tiles, uint32_t k, uint32_t k_pad, uint32_t nt_cols, uint32_t kw, uint32_t kchunks, uint32_t ksteps, uint32_t idesc,
	Control* __restrict__ ctl, int slot, uint32_t* __restrict__ flag_list, float margin_coef)
{
	extern __shared__ uint8_t smem_raw[];
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
	TcBars* bars = reinterpret_cast<TcBars*>(smem + SM_BAR_OFF);
	uint32_t* mg_state = reinterpret_cast<uint32_t*>(smem + SM_MERGE_OFF);
	volatile uint32_t* abort_flag = &bars->abort_flag;

	const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
	const uint32_t n_ctiles = k_pad / nt_cols;
	const uint32_t nblocks = (n_tiles + TC_MA - 1) / TC_MA;
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
			ptx::mbar_init(&bars->acc_empty[i], TC_EPI_WARPS);
		}
		for (uint32_t i = 0; i < TC_NB; ++i) {
			ptx::mbar_init(&bars->b_full[i], 1);
			ptx::mbar_init(&bars->b_empty[i], 1);
		}
		bars->abort_flag = 0;
		ptx::fence_mbar_init();
	}
	if (warp == 1) {
		ptx::tmem_alloc(&bars->tmem_slot, TC_TMEM_COLS);
		ptx::tmem_relinquish();
	}
	// Offset constant: every value |c|^2 - 2 x.c lies in [-X2, X2 + 2*C2] (X2, C2 = largest |x|^2,
	// |c|^2 after centring), an interval of width 2*(X2+C2); with P a power of two >= 1.25 times
	// that width, value + P + X2 + P/32 stays inside [P, 2P) with P/32 of head-room on both
	// sides for the rounding of the pass: one exponent for all values.
	const float x2max = ctl->xmax2, c2max = ctl->cmax2[slot];
	float pow2 = 1.0f;
	{
		const float span = 1.25f * (2.0f * (x2max + c2max)) + 1.0e-30f;
		int e;
		frexpf(span, &e);                       // span = m * 2^e, m in [0.5, 1)
		pow2 = ldexpf(1.0f, e);                 // >= span
	}
	const float offset_c = pow2 + x2max + pow2 * (1.0f / 32.0f);
	{
		// the constant A operand of the extra K step: columns 0 and 1 are one (they meet the high
		// and the low part of |c|^2), columns 2 and 3 hold the offset constant as tf32 hi/lo
		// (they meet ones on the B side), the rest is zero
		const float c_hi = to_tf32(offset_c), c_lo = to_tf32(offset_c - c_hi);
		float* a_aug = reinterpret_cast<float*>(smem + SM_AAUG_OFF);
		for (uint32_t e = threadIdx.x; e < TC_MTILE * 8; e += TC_THREADS) {
			const uint32_t row = e >> 3, kk = e & 7u;
			a_aug[aug_offset(row, kk)] = kk < 2 ? 1.0f : (kk == 2 ? c_hi : (kk == 3 ? c_lo : 0.0f));
		}
		ptx::fence_proxy_async();
	}
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
			if (kchunks > 1) {
				// K-loop mode: one (point tile, centroid tile, 32-dimension slice) per stage
				for (uint32_t blk = blockIdx.x; blk < nblocks && ok; blk += gridDim.x) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t j = 0; j < n_ctiles && ok; ++j)
						for (uint32_t i = 0; i < tiles && ok; ++i)
							for (uint32_t kc = 0; kc < kchunks; ++kc) {
								const uint32_t s = b_count % TC_NB, u = b_count / TC_NB;
								ok = wait_or_abort(&bars->b_empty[s], (u & 1u) ^ 1u, abort_flag);
								if (!ok) break;
								uint8_t* dst = smem + s * KSTAGE_BYTES;
								const bool last = kc == kchunks - 1;
								const uint32_t aug_bytes = last ? nt_cols * 8 * 4 : 0u;
								const int32_t row = (int32_t)((blk * TC_MA + i) * TC_MTILE), x = (int32_t)(kc * TC_KCHUNK);
								ptx::mbar_arrive_expect_tx(&bars->b_full[s], A_TILE_BYTES + 2 * nt_cols * TC_KCHUNK * 4 + aug_bytes);
								ptx::tma_load_2d(dst, &tm_a_hi, x, row, &bars->b_full[s]);
								ptx::tma_load_2d(dst + KS_ALO_OFF, &tm_a_lo, x, row, &bars->b_full[s]);
								ptx::tma_load_2d(dst + KS_BHI_OFF, &tm_b_hi, x, (int32_t)(j * nt_cols), &bars->b_full[s]);
								ptx::tma_load_2d(dst + KS_BLO_OFF, &tm_b_lo, x, (int32_t)(j * nt_cols), &bars->b_full[s]);
								if (last) ptx::bulk_g2s(dst + KS_AUG_OFF, b_aug + (size_t)j * nt_cols * 8, aug_bytes, &bars->b_full[s]);
								++b_count;
							}
				}
			} else {
				uint32_t g = 0;                       // running count of point tiles = position in the A ring
				bool b_loaded = false;
				for (uint32_t blk = blockIdx.x; blk < nblocks && ok; blk += gridDim.x) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t i = 0; i < tiles && ok; ++i, ++g) {
						const uint32_t buf = g % n_abuf, u = g / n_abuf;
						ok = wait_or_abort(&bars->a_empty[buf], (u & 1u) ^ 1u, abort_flag);
						if (!ok) break;
						uint8_t* dst = smem + SM_A_OFF + buf * a_tile;
						const int32_t row = (int32_t)((blk * TC_MA + i) * TC_MTILE);
						ptx::mbar_arrive_expect_tx(&bars->a_full[buf], a_tile);
						ptx::tma_load_2d(dst, &tm_a_hi, 0, row, &bars->a_full[buf]);
						ptx::tma_load_2d(dst + a_plane, &tm_a_lo, 0, row, &bars->a_full[buf]);
						++a_use[buf];
					}
					for (uint32_t j = 0; j < n_ctiles && ok; ++j) {
						if (b_resident && b_loaded) break;
						const uint32_t s = b_count % TC_NB, u = b_count / TC_NB;
						ok = wait_or_abort(&bars->b_empty[s], (u & 1u) ^ 1u, abort_flag);
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
			for (uint32_t back = 0; back < TC_NB && back < b_count; ++back) {
				const uint32_t c = b_count - 1 - back;
				ptx::mbar_wait(&bars->b_full[c % TC_NB], (c / TC_NB) & 1u);
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
			const uint64_t a_aug_desc = make_desc_aug(ptx::smem_u32(smem + SM_AAUG_OFF));
			if (kchunks > 1) {
				// K-loop mode: the accumulator of a (point tile, centroid tile) pair collects all slices
				for (uint32_t blk = blockIdx.x; blk < nblocks && ok; blk += gridDim.x) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t j = 0; j < n_ctiles && ok; ++j)
						for (uint32_t i = 0; i < tiles && ok; ++i) {
							ok = wait_or_abort(&bars->acc_empty[i], (acc_use[i] & 1u) ^ 1u, abort_flag);
							if (!ok) break;
							ptx::tc_fence_after();
							const uint32_t d_tmem = tmem_base + i * TC_NT_MAX;
							for (uint32_t kc = 0; kc < kchunks; ++kc) {
								const uint32_t s = b_count % TC_NB, u = b_count / TC_NB;
								ok = wait_or_abort(&bars->b_full[s], u & 1u, abort_flag);
								if (!ok) break;
								ptx::tc_fence_after();
								const uint32_t base = ptx::smem_u32(smem + s * KSTAGE_BYTES);
								const uint64_t a_hi = make_desc(base), a_lo = make_desc(base + KS_ALO_OFF);
								const uint64_t b_hi = make_desc(base + KS_BHI_OFF), b_lo = make_desc(base + KS_BLO_OFF);
								const bool last = kc == kchunks - 1;
								const uint32_t steps = last ? ksteps : 4u;
								if (ptx::elect_one()) {
									#pragma unroll
									for (uint32_t ks = 0; ks < 4; ++ks)
										if (ks < steps) ptx::mma_tf32(d_tmem, a_lo + 2 * ks, b_hi + 2 * ks, idesc, (kc | ks) > 0);
									#pragma unroll
									for (uint32_t ks = 0; ks < 4; ++ks)
										if (ks < steps) ptx::mma_tf32(d_tmem, a_hi + 2 * ks, b_lo + 2 * ks, idesc, 1);
									#pragma unroll
									for (uint32_t ks = 0; ks < 4; ++ks)
										if (ks < steps) ptx::mma_tf32(d_tmem, a_hi + 2 * ks, b_hi + 2 * ks, idesc, 1);
									if (last) ptx::mma_tf32(d_tmem, a_aug_desc, make_desc_aug(base + KS_AUG_OFF), idesc, 1);
									ptx::mma_commit(&bars->b_empty[s]);
									if (last) ptx::mma_commit(&bars->acc_full[i]);
								}
								__syncwarp();
								++b_count;
							}
							++acc_use[i];
						}
				}
			} else {
#ifdef BKM_TC_TIMING
				long long t_b = 0, t_a = 0, t_acc = 0, t_issue = 0;
				const long long t_start = clock64();
#endif
				uint32_t g = 0;                       // position of the block's first tile in the A ring
				bool b_ready = false;
				for (uint32_t blk = blockIdx.x; blk < nblocks && ok; blk += gridDim.x) {
					const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
					for (uint32_t j = 0; j < n_ctiles && ok; ++j) {
						const uint32_t s = b_resident ? 0u : b_count % TC_NB, u = b_count / TC_NB;
						TC_T(c0);
						if (!(b_resident && b_ready)) {
							ok = wait_or_abort(&bars->b_full[s], u & 1u, abort_flag);
							if (!ok) break;
							b_ready = true;
						}
						TC_T(c1);
						TC_ACC(t_b, c0, c1);
						const uint32_t b_addr = ptx::smem_u32(smem + sm_b_off + s * b_stage);
						const uint64_t b_hi = make_desc_kw(b_addr, kw), b_lo = make_desc_kw(b_addr + b_plane, kw);
						const uint64_t b_aug_desc = make_desc_aug(ptx::smem_u32(smem + sm_baug_off + s * AUG_BYTES));
						for (uint32_t i = 0; i < tiles; ++i) {
							const uint32_t buf = (g + i) % n_abuf, ua = (g + i) / n_abuf;
							TC_T(c2);
							if (j == 0) {
								ok = wait_or_abort(&bars->a_full[buf], ua & 1u, abort_flag);
								if (!ok) break;
							}
							TC_T(c3);
							ok = wait_or_abort(&bars->acc_empty[i], (acc_use[i] & 1u) ^ 1u, abort_flag);
							if (!ok) break;
							TC_T(c4);
							TC_ACC(t_a, c2, c3);
							TC_ACC(t_acc, c3, c4);
							ptx::tc_fence_after();
							const uint32_t a_addr = ptx::smem_u32(smem + SM_A_OFF + buf * a_tile);
							const uint64_t a_hi = make_desc_kw(a_addr, kw), a_lo = make_desc_kw(a_addr + a_plane, kw);
							const uint32_t d_tmem = tmem_base + i * TC_NT_MAX;
							if (ptx::elect_one()) {
								// small cross terms first, then the dominant hi*hi term, then |c|^2;
								// +2 in the descriptor's address field = 32 bytes = one K step
								#pragma unroll
								for (uint32_t ks = 0; ks < 4; ++ks)
									if (ks < ksteps) ptx::mma_tf32(d_tmem, a_lo + 2 * ks, b_hi + 2 * ks, idesc, ks > 0);
								#pragma unroll
								for (uint32_t ks = 0; ks < 4; ++ks)
									if (ks < ksteps) ptx::mma_tf32(d_tmem, a_hi + 2 * ks, b_lo + 2 * ks, idesc, 1);
								#pragma unroll
								for (uint32_t ks = 0; ks < 4; ++ks)
									if (ks < ksteps) ptx::mma_tf32(d_tmem, a_hi + 2 * ks, b_hi + 2 * ks, idesc, 1);
								ptx::mma_tf32(d_tmem, a_aug_desc, b_aug_desc, idesc, 1);
								ptx::mma_commit(&bars->acc_full[i]);
								if (j == n_ctiles - 1) ptx::mma_commit(&bars->a_empty[buf]);
							}
							__syncwarp();
							TC_T(c5);
							TC_ACC(t_issue, c4, c5);
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
#ifdef BKM_TC_TIMING
				if (blockIdx.x == 3 && lane == 0)
					printf("mma warp: total %lld  wait_b %lld  wait_a %lld  wait_acc %lld  issue %lld  (tiles %u)\n",
						clock64() - t_start, t_b, t_a, t_acc, t_issue, g);
#endif
			}
		}
	} else {
		// ---------------- epilogue ----------------
		// The loops over tiles and chunks are kept rolled on purpose: unrolled, the arg-min code
		// of one block outgrows the instruction cache and the warps starve on instruction fetch.
		const uint32_t q = warp & 3u;              // TMEM lane quarter this warp may read
		const uint32_t part = (warp - 2) >> 2;     // which quarter of the tile's columns (0..3)
		const uint32_t row = q * 32 + lane;
		const float ulp = pow2 * 1.1920929e-07f;   // spacing of the values inside [P, 2P)
		const uint32_t chunks_total = nt_cols >> 5;                    // 1..8
		const uint32_t per_part = (chunks_total + 3) / 4;              // 1..2
		const uint32_t first_chunk = part * per_part;
		const uint32_t nchunks = first_chunk >= chunks_total ? 0u : min(per_part, chunks_total - first_chunk);
		const uint32_t colbase = first_chunk * 32;
		uint32_t acc_use[TC_MA] = {0, 0};
		bool ok = true;
#ifdef BKM_TC_TIMING
		long long e_wait = 0, e_ld = 0, e_cmp = 0, e_merge = 0;
		const long long e_start = clock64();
#endif
		for (uint32_t blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
			const uint32_t tiles = min(TC_MA, n_tiles - blk * TC_MA);
			uint32_t best0 = 0xFFFFFFFFu, second0 = 0xFFFFFFFFu, bchunk0 = 0;
			uint32_t best1 = 0xFFFFFFFFu, second1 = 0xFFFFFFFFu, bchunk1 = 0;
			// |x|^2 of this thread's two points is only needed at the end of the block: fetch it now
			float xn0 = 0.0f, xn1 = 0.0f;
			if (part == 0) {
				const uint64_t p0 = (uint64_t)(blk * TC_MA) * TC_MTILE + row;
				if (p0 < n) xn0 = xnorm[p0];
				if (p0 + TC_MTILE < n) xn1 = xnorm[p0 + TC_MTILE];
			}
			for (uint32_t j = 0; j < n_ctiles; ++j) {
				#pragma unroll 1
				for (uint32_t i = 0; i < tiles; ++i) {
					const uint32_t use = i ? acc_use[1] : acc_use[0];
					TC_T(e0);
					if (ok) {
						// one lane polls the barrier, the warp follows
						bool w = true;
						if (lane == 0) w = wait_or_abort(&bars->acc_full[i], use & 1u, abort_flag);
						ok = __shfl_sync(0xffffffffu, (int)w, 0) != 0;
					}
					if (i) ++acc_use[1]; else ++acc_use[0];
					TC_T(e1);
					TC_ACC(e_wait, e0, e1);
					if (ok && nchunks > 0) {
						ptx::tc_fence_after();
						const uint32_t taddr = tmem_base + ((q * 32u) << 16) + i * TC_NT_MAX + colbase;
						const uint32_t chunk0 = (j * nt_cols + colbase) >> 5;
						// This warp's columns go to registers first and the accumulator is handed back
						// to the MMA warp right away; the arg-min then runs from registers while the
						// tensor cores already fill the accumulator again.
						uint32_t v0[32], v1[32];
						ptx::tmem_ld32(taddr, v0);
						if (nchunks > 1) ptx::tmem_ld32(taddr + 32, v1);
						ptx::tmem_ld_wait();
						ptx::tc_fence_before();
						__syncwarp();
						if (lane == 0) ptx::mbar_arrive(&bars->acc_empty[i]);
						TC_T(e2);
						TC_ACC(e_ld, e1, e2);
						uint32_t b = i ? best1 : best0, s2 = i ? second1 : second0, bc = i ? bchunk1 : bchunk0;
						// columns at or behind k are padding
						const uint32_t col0 = chunk0 * 32u;
						const uint32_t left = k > col0 ? k - col0 : 0u;
						if (left >= 64 || (nchunks == 1 && left >= 32)) {
							chunk_update<false>(v0, chunk0, 32, b, s2, bc);
							if (nchunks > 1) chunk_update<false>(v1, chunk0 + 1, 32, b, s2, bc);
						} else {
							if (left > 0) chunk_update<true>(v0, chunk0, left, b, s2, bc);
							if (nchunks > 1 && left > 32) chunk_update<true>(v1, chunk0 + 1, left - 32, b, s2, bc);
						}
						if (i) { best1 = b; second1 = s2; bchunk1 = bc; } else { best0 = b; second0 = s2; bchunk0 = bc; }
						TC_T(e3);
						TC_ACC(e_cmp, e2, e3);
					} else {
						__syncwarp();
						if (lane == 0) ptx::mbar_arrive(&bars->acc_empty[i]);
					}
				}
			}
			// merge the four column parts: parts 1..3 hand their state over through shared memory
			uint32_t* mg = mg_state;
			TC_T(e4);
			if (part > 0) {
				uint32_t* dst = mg + (part - 1) * (3 * TC_MA * TC_MTILE);
				dst[0 * TC_MTILE + row] = best0; dst[1 * TC_MTILE + row] = second0; dst[2 * TC_MTILE + row] = bchunk0;
				dst[3 * TC_MTILE + row] = best1; dst[4 * TC_MTILE + row] = second1; dst[5 * TC_MTILE + row] = bchunk1;
			}
			asm volatile("bar.sync %0, 128;" :: "r"(1u + q) : "memory");   // the four warps that share these 32 rows
			if (part == 0) {
				#pragma unroll
				for (uint32_t i = 0; i < TC_MA; ++i) {
					const uint64_t p = (uint64_t)(blk * TC_MA + i) * TC_MTILE + row;
					if (i < tiles && p < n && ok) {
						uint32_t b = i ? best1 : best0, s2 = i ? second1 : second0, bc = i ? bchunk1 : bchunk0;
						#pragma unroll
						for (uint32_t o = 0; o < 3; ++o) {
							const uint32_t* src = mg + o * (3 * TC_MA * TC_MTILE) + i * 3 * TC_MTILE;
							const uint32_t ob = src[row], os = src[TC_MTILE + row], oc = src[2 * TC_MTILE + row];
							s2 = umin3(s2, os, max(b, ob));
							bc = ob < b ? oc : bc;
							b = min(b, ob);
						}
						asg[p] = bc * 32u + (b & 31u);
						// keys are (mantissa bits << 5 | column): their difference >> 5 counts value spacings
						const float gap = s2 == 0xFFFFFFFFu ? INFINITY : (float)((s2 >> 5) - (b >> 5)) * ulp;
						const float margin = margin_coef * ((i ? xn1 : xn0) + c2max) + 4.0f * ulp;
						if (gap <= margin) {
							const uint32_t pos = atomicAdd(&ctl->flag_count, 1u);
							if ((uint64_t)pos < n) flag_list[pos] = (uint32_t)p;
							else atomicOr(&ctl->status, (uint32_t)STATUS_LIST_OVERFLOW);
						}
					}
				}
			}
			asm volatile("bar.sync %0, 128;" :: "r"(1u + q) : "memory");   // the four warps that share these 32 rows
			TC_T(e5);
			TC_ACC(e_merge, e4, e5);
		}
#ifdef BKM_TC_TIMING
		if (blockIdx.x == 3 && lane == 0 && (warp == 2 || warp == 7 || warp == 17))
			printf("epi warp %u: total %lld  wait %lld  ld %lld  compute %lld  merge %lld\n", warp, clock64() - e_start, e_wait, e_ld, e_cmp, e_merge);
#endif
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
// host side
// ------------------------------------------------------------------------------------------

struct TcPlan {
	CUtensorMap a_hi, a_lo, b_hi, b_lo;
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
// rows are only 16 floats long, box_rows x 16 columns with 64-byte swizzle.
static bool encode_plane(CUtensorMap* out, const float* base, uint64_t rows, uint32_t cols, uint32_t box_rows)
{
	const uint32_t kw = cols == 16 ? 16u : TC_KCHUNK;
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
	if (cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) p->sm_count = 148;
	if (!encode_plane(&p->a_hi, tp.a_hi, tp.n_pad, tp.d_pad, TC_MTILE) ||
		!encode_plane(&p->a_lo, tp.a_lo, tp.n_pad, tp.d_pad, TC_MTILE) ||
		!encode_plane(&p->b_hi, tm.b_hi, tm.k_pad, tm.d_pad, p->nt_cols) ||
		!encode_plane(&p->b_lo, tm.b_lo, tm.k_pad, tm.d_pad, p->nt_cols)) {
		if (err) *err = e_map;
		delete p;
		return nullptr;
	}
	if (cudaFuncSetAttribute(assign_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM_ALLOC) != cudaSuccess) {
		cudaGetLastError();
		if (err) *err = e_attr;
		delete p;
		return nullptr;
	}
	return p;
}

void tc_plan_destroy(TcPlan* plan) { delete plan; }

cudaError_t launch_assign_tc(TcPlan* p, uint32_t* asg, Control* ctl, int slot, uint32_t* flag_list,
	float margin_scale, cudaStream_t stream)
{
	if (!p) return cudaErrorInvalidValue;
	const uint32_t n_tiles = (uint32_t)(p->tp.n_pad / TC_MTILE);
	const uint32_t nblocks = (n_tiles + TC_MA - 1) / TC_MA;
	const uint32_t grid = std::min<uint32_t>(nblocks, (uint32_t)p->sm_count);
	// error band of the split-TF32 GEMM form relative to |x|^2 + max|c|^2
	const float margin_coef = margin_scale * (48.0f + 0.5f * (float)p->tp.d_pad) * 1.1920929e-07f;
	const uint32_t kw = p->tp.d_pad == 16 ? 16u : TC_KCHUNK;
	const uint32_t kchunks = p->tp.d_pad / kw;
	const uint32_t ksteps_last = (p->s.dim - (kchunks - 1) * kw + 7) / 8;    // K steps of the last slice
	const uint32_t idesc = p->idesc;
	assign_tc_kernel<<<grid, TC_THREADS, SM_ALLOC, stream>>>(p->a_hi, p->a_lo, p->b_hi, p->b_lo,
		p->tm.b_aug, p->tp.xnorm, asg, p->s.n, n_tiles, p->s.k, p->tm.k_pad, p->nt_cols, kw, kchunks, ksteps_last, idesc,
		ctl, slot, flag_list, margin_coef);
	return cudaGetLastError();
}

} // namespace bkm
