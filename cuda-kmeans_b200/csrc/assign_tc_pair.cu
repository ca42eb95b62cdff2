// Tensor-core assignment on CTA pairs (tcgen05 cta_group::2) with all means resident in shared
// memory, for mean sets of 2..4 256-column tiles and 17 <= dim <= 32.
//
// The arithmetic is that of assign_tc.cu (split-TF32 GEMM form, |c|^2 and the offset constant
// folded in by one extra K step, integer keys, near-ties queued for the exact kernel).  What
// differs is where the operands live.  One MMA of the pair multiplies 256 points by 256 means:
// each CTA supplies its 128 points (A) and ITS HALF of the 256 means (B), and receives the
// 128 x 256 block of its own points in its tensor memory.  A CTA therefore stores only half of
// every mean tile - 144 KiB for 1024 means of dim 32 instead of 288 KiB - which fits beside a
// ring of point tiles.  The means are loaded once per launch; afterwards only point tiles move,
// and the tensor cores never wait for an operand ring to turn.
//
// Roles per CTA (576 threads): warp 0 loads (its half of the means once, then its point tiles),
// warp 1 of the pair's first CTA issues the MMAs for both, warps 2..17 of each CTA reduce that
// CTA's accumulator rows.  Barriers that pace the pair live in the first CTA: TMA copies of both
// CTAs count their bytes there, the second CTA's epilogue warps arrive there remotely, and the
// issuing thread commits to the barriers of both CTAs.  All waits are bounded.
#include <cuda.h>

#include "kernels.cuh"
#include "ptx.cuh"
#include "tc_common.cuh"

#include <algorithm>
#include <cmath>

namespace bkm {

constexpr uint32_t P2_AAUG_OFF = 208 * 1024;                      // constant ones tile (128 rows x one K step)
constexpr uint32_t P2_MERGE_OFF = P2_AAUG_OFF + TC_MTILE * 8 * 4;
constexpr uint32_t P2_MERGE_BYTES = 2 * 3 * 3 * TC_MTILE * 4      // two slots x column parts 1..3 x (best, second, chunk)
	+ 2 * TC_MTILE * 4;                                            // two slots of final clusters (fused update sums)
constexpr uint32_t P2_BAR_OFF = P2_MERGE_OFF + P2_MERGE_BYTES;
constexpr uint32_t P2_TOTAL = P2_BAR_OFF + 256;
constexpr uint32_t P2_ALLOC = P2_TOTAL + 1024;                    // slack for 1024-byte alignment
constexpr uint32_t P2_NA_MAX = 8;
constexpr uint32_t P2_HALF = TC_NT_MAX / 2;                       // means of a tile held by one CTA
constexpr uint32_t P2_AUG_HALF_BYTES = P2_HALF * 8 * 4;           // 4 KiB
constexpr uint32_t P2_ACCS = 4;                                   // accumulators in flight
constexpr uint32_t P2_UNIT_COLS = TC_TMEM_COLS / P2_ACCS;         // 128 means per accumulator fill ...
constexpr uint32_t P2_UNIT_ROWS = P2_UNIT_COLS / 2;               // ... 64 from each CTA's half of a tile

struct PairBars {
	uint64_t a_full[P2_NA_MAX];      // first CTA: point tiles of both CTAs have landed
	uint64_t a_empty[P2_NA_MAX];     // every CTA: the MMAs that read the buffer are done
	uint64_t b_full;                 // first CTA: all means of both CTAs have landed
	uint64_t acc_full[P2_ACCS];      // every CTA: accumulator complete
	uint64_t acc_empty[P2_ACCS];     // first CTA: the epilogue warps of both CTAs have read it
	uint32_t tmem_slot;
	uint32_t abort_flag;
};
static_assert(sizeof(PairBars) <= 256, "barrier block too large");
static_assert(P2_ALLOC <= 227 * 1024, "shared memory budget exceeded");

// Bytes of means one CTA keeps: per tile two planes of 128 rows x kw floats and one K step of |c|^2.
__host__ __device__ inline uint32_t pair_b_tile_bytes(uint32_t kw) { return 2 * P2_HALF * kw * 4; }

bool assign_tc_pair_supported(uint32_t k, uint32_t k_pad, uint32_t d_pad, uint32_t nt_cols, int sm_count)
{
	// 16-float rows (dim <= 16) halve the tensor work per accumulator and measured faster on the one-CTA kernel
	if (d_pad != TC_KCHUNK || nt_cols != TC_NT_MAX || k_pad % TC_NT_MAX != 0 || k < TC_NT_MAX || sm_count < 2) return false;
	const uint32_t kw = d_pad == 16 ? 16u : TC_KCHUNK;
	const uint32_t n_ctiles = k_pad / TC_NT_MAX;
	if (n_ctiles < 2) return false;                               // a single tile is resident in the one-CTA kernel as well
	const uint32_t a_off = n_ctiles * (pair_b_tile_bytes(kw) + P2_AUG_HALF_BYTES);
	return a_off + 2 * (2 * TC_MTILE * kw * 4) <= P2_AAUG_OFF;
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d)
{
	asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Like wait_or_abort, and a wait that runs out also raises the flag of the other CTA.
template<uint32_t SLEEP_NS = 100>
__device__ __forceinline__ bool pair_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t peer_abort_addr)
{
	if (wait_or_abort<SLEEP_NS, true>(bar, parity, abort_flag)) return true;
	ptx::st_cluster_u32(peer_abort_addr, 1u);
	return false;
}

// KSTEPS = K steps of 8 dimensions per product (3 for dim 17..24, 4 for dim 25..32): a template
// parameter so that the MMA-issuing warp runs a straight line of instructions.
template<uint32_t KSTEPS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1) assign_tc_pair_kernel(
	const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
	const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
	const float* __restrict__ b_aug, const float* __restrict__ xnorm, uint32_t* __restrict__ asg,
	uint64_t n, uint32_t n_tiles, uint32_t k, uint32_t n_ctiles, uint32_t kw, uint32_t ksteps, uint32_t idesc,
	Control* __restrict__ ctl, int slot, uint32_t* __restrict__ flag_list, float margin_coef,
	float* __restrict__ fuse_acc, uint32_t* __restrict__ fuse_counts, const float* __restrict__ center, uint32_t dim,
	uint32_t step_begin, uint32_t step_end)
{
	extern __shared__ uint8_t smem_raw[];
	uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
	PairBars* bars = reinterpret_cast<PairBars*>(smem + P2_BAR_OFF);
	uint32_t* mg_state = reinterpret_cast<uint32_t*>(smem + P2_MERGE_OFF);
	volatile uint32_t* abort_flag = &bars->abort_flag;

	const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
	const uint32_t rank = ptx::cluster_ctarank();
	const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
	// one step = one point tile per CTA; a launch takes steps [step_begin, step_end) (all of them, or the
	// chunk of the points that has just arrived from the host)
	const uint32_t steps_total = min(step_end, (n_tiles + 1) / 2);
	const uint32_t n_units = 2 * n_ctiles;                         // accumulator fills per step
	const uint32_t peer_abort_addr = ptx::map_to_cta(ptx::smem_u32(&bars->abort_flag), rank ^ 1u);

	// shared-memory layout: [means: per tile hi | lo] [|c|^2 steps] [ring of point tiles] ... fixed tail
	const uint32_t b_plane = P2_HALF * kw * 4, b_tile = 2 * b_plane;
	const uint32_t a_plane = TC_MTILE * kw * 4, a_tile = 2 * a_plane;
	const uint32_t baug_off = n_ctiles * b_tile;
	const uint32_t a_off = baug_off + n_ctiles * P2_AUG_HALF_BYTES;
	const uint32_t n_abuf = min(P2_NA_MAX, (P2_AAUG_OFF - a_off) / a_tile);

	if (threadIdx.x == 0) {
		for (uint32_t i = 0; i < P2_NA_MAX; ++i) {
			ptx::mbar_init(&bars->a_full[i], 1);
			// the MMAs that read the tile and, when the update sums are accumulated here, the
			// epilogue warps that read it again at the end of the step
			ptx::mbar_init(&bars->a_empty[i], fuse_acc ? 1 + TC_EPI_WARPS : 1);
		}
		ptx::mbar_init(&bars->b_full, 1);
		for (uint32_t i = 0; i < P2_ACCS; ++i) {
			ptx::mbar_init(&bars->acc_full[i], 1);
			ptx::mbar_init(&bars->acc_empty[i], 2 * 8);          // two warps per TMEM lane quarter in each CTA
		}
		bars->abort_flag = 0;
		ptx::fence_mbar_init();
	}
	if (warp == 1) {
		ptx::tmem_alloc_pair(&bars->tmem_slot, TC_TMEM_COLS);
		ptx::tmem_relinquish_pair();
	}
	if (fuse_acc) {
		// pairs spread over the copies of the accumulators so that fewer reductions meet on a line
		const size_t rep_stride = acc_replica_stride(k, dim);
		const uint32_t rep = pair % acc_replicas(k, dim);
		fuse_acc += rep * rep_stride;
		fuse_counts += rep * rep_stride;
	}
	const float x2max = ctl->xmax2, c2max = ctl->cmax2[slot];
	const KeyConsts kc = make_key_consts(x2max, c2max);
	const uint32_t key_mult = kc.key_mult, key_base = kc.key_base, key_magic = kc.key_magic;
	fill_a_aug(reinterpret_cast<float*>(smem + P2_AAUG_OFF), kc.offset_c, threadIdx.x, TC_THREADS);
	{
		// This CTA's half of every tile's |c|^2 K step: 128 rows = 4 KiB, contiguous in global memory.
		// Rows behind the last mean are padding (their operand rows are zero); they get the |c|^2 that
		// puts their value at 2P - P/32, above every real value (at most 1.83 P) and inside [P, 2P),
		// so that the arg-min needs no column masks.
		float4* dst = reinterpret_cast<float4*>(smem + baug_off);
		const uint32_t per_tile = P2_AUG_HALF_BYTES / 16;
		const float cn_pad = to_tf32(kc.pow2 - x2max - kc.pow2 * (1.0f / 16.0f));
		for (uint32_t e = threadIdx.x; e < n_ctiles * per_tile; e += TC_THREADS) {
			const uint32_t j = e / per_tile, r = e - j * per_tile;
			// float4 r of a tile half: rows (r / 16) * 8 + r % 8, K positions 4 * ((r / 8) % 2) ..
			const uint32_t mean = j * TC_NT_MAX + rank * P2_HALF + (r >> 4) * 8 + (r & 7u);
			float4 v = reinterpret_cast<const float4*>(b_aug + ((size_t)j * TC_NT_MAX + rank * P2_HALF) * 8)[r];
			if (mean >= k && ((r >> 3) & 1u) == 0) v = make_float4(cn_pad, 0.0f, 1.0f, 1.0f);
			dst[e] = v;
		}
	}
	ptx::fence_proxy_async();
	ptx::tc_fence_before();
	ptx::cluster_sync();            // barriers of both CTAs initialised, tensor memory allocated, constant tiles written
	ptx::tc_fence_after();
	const uint32_t tmem_base = bars->tmem_slot;

	if (warp == 0) {
		// ---------------- TMA producer (both CTAs) ----------------
		if (lane == 0) {
			ptx::prefetch_tmap(&tm_a_hi); ptx::prefetch_tmap(&tm_a_lo);
			ptx::prefetch_tmap(&tm_b_hi); ptx::prefetch_tmap(&tm_b_lo);
			const uint32_t b_full_leader = ptx::leader_cta_addr(ptx::smem_u32(&bars->b_full));
			if (rank == 0) ptx::mbar_arrive_expect_tx(&bars->b_full, 2 * n_ctiles * b_tile);
			for (uint32_t j = 0; j < n_ctiles; ++j) {
				const int32_t row = (int32_t)(j * TC_NT_MAX + rank * P2_HALF);
				ptx::tma_load_2d_pair(smem + j * b_tile, &tm_b_hi, 0, row, b_full_leader);
				ptx::tma_load_2d_pair(smem + j * b_tile + b_plane, &tm_b_lo, 0, row, b_full_leader);
			}
			uint32_t it = 0;
			bool ok = true;
			for (uint32_t step = step_begin + pair; step < steps_total && ok; step += n_pairs, ++it) {
				const uint32_t buf = it % n_abuf, u = it / n_abuf;
				ok = pair_wait<400>(&bars->a_empty[buf], (u & 1u) ^ 1u, abort_flag, peer_abort_addr);
				if (!ok) break;
				if (rank == 0) ptx::mbar_arrive_expect_tx(&bars->a_full[buf], 2 * a_tile);
				const uint32_t a_full_leader = ptx::leader_cta_addr(ptx::smem_u32(&bars->a_full[buf]));
				uint8_t* dst = smem + a_off + buf * a_tile;
				const int32_t row = (int32_t)((2 * step + rank) * TC_MTILE);   // rows behind the last tile read as zeros
				ptx::tma_load_2d_pair(dst, &tm_a_hi, 0, row, a_full_leader);
				ptx::tma_load_2d_pair(dst + a_plane, &tm_a_lo, 0, row, a_full_leader);
			}
			if (rank == 0) {
				// Nobody leaves while a copy may still be in flight: the first CTA's barriers count
				// the bytes of both CTAs, and the second CTA stays until the final cluster barrier.
				ptx::mbar_wait(&bars->b_full, 0);
				for (uint32_t back = 0; back < n_abuf && back < it; ++back) {
					const uint32_t c = it - 1 - back;
					ptx::mbar_wait(&bars->a_full[c % n_abuf], (c / n_abuf) & 1u);
				}
			}
		}
	} else if (warp == 1) {
		// ---------------- MMA issuer (first CTA of the pair) ----------------
		// One accumulator fill ("unit") multiplies the pair's 256 points by 128 means: 64 rows of
		// each CTA's half of a mean tile.  Four 128-column accumulators are in flight, which gives
		// the hand-offs between the CTAs (a few hundred cycles each way) room to hide.
		if (rank == 0) {
			const uint32_t a_aug_lo = desc_lo_aug(ptx::smem_u32(smem + P2_AAUG_OFF));
			const uint32_t peer = 1u;
			// barriers are 8 bytes apart, and so are their images in the other CTA
			const uint32_t a_empty_peer_base = ptx::map_to_cta(ptx::smem_u32(&bars->a_empty[0]), peer);
			const uint32_t acc_full_own = ptx::smem_u32(&bars->acc_full[0]);
			const uint32_t acc_full_peer = ptx::map_to_cta(acc_full_own, peer);
			bool ok = pair_wait(&bars->b_full, 0, abort_flag, peer_abort_addr);
			uint32_t it = 0, c = 0;                 // c counts units: accumulator c % 4, use c / 4
			for (uint32_t step = step_begin + pair; step < steps_total && ok; step += n_pairs, ++it) {
				const uint32_t buf = it % n_abuf, ua = it / n_abuf;
				ok = pair_wait(&bars->a_full[buf], ua & 1u, abort_flag, peer_abort_addr);
				if (!ok) break;
				// descriptor halves (see desc_lo_sw128): +2 in the address field = 32 bytes = one K step
				const uint32_t a_addr = ptx::smem_u32(smem + a_off + buf * a_tile);
				const uint32_t a_hi = desc_lo_sw128(a_addr), a_lo = desc_lo_sw128(a_addr + a_plane);
				for (uint32_t u = 0; u < n_units; ++u, ++c) {
					const uint32_t acc = c % P2_ACCS;
					ok = pair_wait<200>(&bars->acc_empty[acc], ((c / P2_ACCS) & 1u) ^ 1u, abort_flag, peer_abort_addr);
					if (!ok) break;
					ptx::tc_fence_after();
					// rows [h*64, h*64+64) of this CTA's (and, at the same offset, the other CTA's) half of tile j
					const uint32_t j = u >> 1, h = u & 1u;
					const uint32_t b_addr = ptx::smem_u32(smem + j * b_tile) + h * (P2_UNIT_ROWS * TC_KCHUNK * 4);
					const uint32_t b_hi = desc_lo_sw128(b_addr), b_lo = desc_lo_sw128(b_addr + b_plane);
					const uint32_t b_aug_lo = desc_lo_aug(ptx::smem_u32(smem + baug_off + j * P2_AUG_HALF_BYTES) + h * (P2_UNIT_ROWS * 8 * 4));
					const uint32_t d_tmem = tmem_base + acc * P2_UNIT_COLS;
					if (ptx::elect_one()) {
						// small cross terms first, then the dominant hi*hi term, then |c|^2
						ptx::mma_tf32_pair_halves<false>(d_tmem, a_lo, DESC_HI_SW128, b_hi, DESC_HI_SW128, idesc);
						#pragma unroll
						for (uint32_t ks = 1; ks < KSTEPS; ++ks)
							ptx::mma_tf32_pair_halves<true>(d_tmem, a_lo + 2 * ks, DESC_HI_SW128, b_hi + 2 * ks, DESC_HI_SW128, idesc);
						#pragma unroll
						for (uint32_t ks = 0; ks < KSTEPS; ++ks)
							ptx::mma_tf32_pair_halves<true>(d_tmem, a_hi + 2 * ks, DESC_HI_SW128, b_lo + 2 * ks, DESC_HI_SW128, idesc);
						#pragma unroll
						for (uint32_t ks = 0; ks < KSTEPS; ++ks)
							ptx::mma_tf32_pair_halves<true>(d_tmem, a_hi + 2 * ks, DESC_HI_SW128, b_hi + 2 * ks, DESC_HI_SW128, idesc);
						ptx::mma_tf32_pair_halves<true>(d_tmem, a_aug_lo, DESC_HI_AUG, b_aug_lo, DESC_HI_AUG, idesc);
						ptx::mma_commit_pair(acc_full_own + acc * 8u);
						ptx::mma_commit_pair(acc_full_peer + acc * 8u);
						if (u == n_units - 1) {
							ptx::mma_commit_pair(ptx::smem_u32(&bars->a_empty[buf]));
							ptx::mma_commit_pair(a_empty_peer_base + buf * 8u);
						}
					}
					__syncwarp();
				}
			}
		}
	} else {
		// ---------------- epilogue (both CTAs, own accumulator rows) ----------------
		// Warp (q, g): TMEM lane quarter q (the only lanes the warp may read); g = 2 * column half +
		// group.  The two groups of eight warps take the accumulator fills alternately; a warp moves
		// its 64 columns to registers with one load, hands the accumulator back at once and reduces
		// from registers, so an accumulator is away from the tensor cores for a load only.
		// The loops are kept rolled (instruction cache).
		const uint32_t q = warp & 3u;
		const uint32_t g = (warp - 2) >> 2;           // 0..3
		const uint32_t row = q * 32 + lane;
		const float ulp = kc.pow2 * 1.1920929e-07f;   // spacing of the values inside [P, 2P)
		const uint32_t merger = 1u;                   // group 1, lower column half (fills per step are even in number)
		const uint32_t acc_empty_base = ptx::map_to_cta(ptx::smem_u32(&bars->acc_empty[0]), 0);
		uint32_t it = 0;
		bool ok = true;
		// Fused update sums.  The 32 points of this quarter stay in the point tile (tf32 hi + lo of
		// the centred coordinates) after their step.  Eight lanes cover one point's row with a
		// 128-bit vector reduction each, so one instruction of a warp sends four full rows; the
		// four warps of the quarter take eight points each.  A warp sends them after its first
		// accumulator of the following step: the warps reach that point one accumulator fill after
		// another, which keeps the SM's reduction path from being hit by all of them at once, and
		// the tile buffer is handed back to the loader when the last of them has read it.
		bool pending = false;
		uint32_t pend_it = 0;
		auto flush_sums = [&]() {
			if (g != merger) asm volatile("bar.sync %0, 128;" :: "r"(9u + q) : "memory");   // the final clusters are written
			const uint32_t* s_mine = mg_state + 2 * 3 * 3 * TC_MTILE + (pend_it & 1u) * TC_MTILE;
			const uint8_t* tile_hi = smem + a_off + (pend_it % n_abuf) * a_tile;
			const uint32_t sub = lane >> 3, c4 = lane & 7u;
			const bool dims_ok = c4 * 4 < dim;
			float4 cen = make_float4(0.f, 0.f, 0.f, 0.f);
			if (dims_ok) cen = reinterpret_cast<const float4*>(center)[c4];
			#pragma unroll
			for (uint32_t r4 = 0; r4 < 2; ++r4) {
				const uint32_t trow = q * 32 + g * 8 + r4 * 4 + sub;
				const uint32_t a = s_mine[trow];
				const uint32_t off = trow * 128u + ((c4 ^ (trow & 7u)) << 4);     // 128-byte swizzle
				if (a != 0xFFFFFFFFu && dims_ok) {
					const float4 hi = *reinterpret_cast<const float4*>(tile_hi + off);
					const float4 lo = *reinterpret_cast<const float4*>(tile_hi + a_plane + off);
					red_add_v4(&fuse_acc[(size_t)a * dim + c4 * 4], (hi.x + lo.x) + cen.x, (hi.y + lo.y) + cen.y,
						(hi.z + lo.z) + cen.z, (hi.w + lo.w) + cen.w);
				}
			}
			__syncwarp();
			if (lane == 0) ptx::mbar_arrive(&bars->a_empty[pend_it % n_abuf]);
			pending = false;
		};
		for (uint32_t step = step_begin + pair; step < steps_total; step += n_pairs, ++it) {
			uint32_t best = 0xFFFFFFFFu, second = 0xFFFFFFFFu, bchunk = 0;
			const uint64_t p = (uint64_t)(2 * step + rank) * TC_MTILE + row;
			float xn = 0.0f;
			if (g == merger && p < n) xn = xnorm[p];      // needed at the end of the step only: fetch early
			// this warp's accumulator fills of the step: every second one, counted across steps; of
			// each it takes 64 columns with one load and hands the accumulator back at once
			const uint32_t c_step = it * n_units;
			const uint32_t grp = g & 1u, colhalf = g >> 1;
			#pragma unroll 1
			for (uint32_t u = (grp - c_step) & 1u; u < n_units; u += 2) {
				const uint32_t c = c_step + u;
				const uint32_t acc = c % P2_ACCS;
				const uint32_t acc_release = acc_empty_base + acc * 8u;
				// the whole warp polls (one warp instruction either way, and no divergent region around it)
				if (ok) ok = __all_sync(0xffffffffu, pair_wait(&bars->acc_full[acc], (c / P2_ACCS) & 1u, abort_flag, peer_abort_addr)) != 0;
				if (ok) {
					ptx::tc_fence_after();
					const uint32_t j = u >> 1, h = u & 1u;
					// columns [colhalf*64, +64) of the accumulator are rows h*64.. of CTA colhalf's half of tile j
					const uint32_t taddr = tmem_base + ((q * 32u) << 16) + acc * P2_UNIT_COLS + colhalf * 64u;
					uint32_t v0[32], v1[32];
					const uint32_t chunk0 = j * 8u + colhalf * 4u + h * 2u;    // in units of 32 means
					// the second half of the columns travels while the first is reduced
					ptx::tmem_ld32(taddr, v0);
					ptx::tmem_ld_wait();
					ptx::tmem_ld32(taddr + 32, v1);
					chunk_update<false>(v0, key_mult, chunk0, 32, best, second, bchunk);
					ptx::tmem_ld_wait();
					ptx::tc_fence_before();
					__syncwarp();
					if (lane == 0) ptx::mbar_arrive_cluster(acc_release);
					chunk_update<false>(v1, key_mult, chunk0 + 1, 32, best, second, bchunk);
				} else {
					__syncwarp();
					if (lane == 0) ptx::mbar_arrive_cluster(acc_release);
				}
				if (pending) flush_sums();
			}
			if (pending) flush_sums();                    // a step without an accumulator for this warp
			// Three warps of a quarter hand their state to the fourth through shared memory and go on
			// without waiting (bar.arrive); the fourth waits for them (bar.sync), merges and writes the
			// results.  Slots and barrier numbers alternate with the step count.  No warp can be a whole
			// step ahead of another: every accumulator fill needs all warps of both groups to have
			// released the fill four before it.  The merging warp belongs to the group that serves the
			// last fill of a step (it is the last to finish anyway) and has the second fill of the next.
			uint32_t* mg = mg_state + (it & 1u) * (3 * 3 * TC_MTILE);
			const uint32_t merge_bar = 1u + (it & 1u) * 4u + q;
			uint32_t mine = 0xFFFFFFFFu;                  // cluster of this thread's point (merging warp)
			if (g != merger) {
				uint32_t* dst = mg + (g < merger ? g : g - 1) * (3 * TC_MTILE);
				dst[row] = best; dst[TC_MTILE + row] = second; dst[2 * TC_MTILE + row] = bchunk;
				asm volatile("bar.arrive %0, 128;" :: "r"(merge_bar) : "memory");
			} else {
				asm volatile("bar.sync %0, 128;" :: "r"(merge_bar) : "memory");
				bool flag = false;
				if (p < n && ok) {
					#pragma unroll
					for (uint32_t o = 0; o < 3; ++o) {
						const uint32_t* src = mg + o * (3 * TC_MTILE);
						const uint32_t ob = src[row], os = src[TC_MTILE + row], oc = src[2 * TC_MTILE + row];
						second = umin3(second, os, max(best, ob));
						bchunk = ob < best ? oc : bchunk;
						best = min(best, ob);
					}
					// key - key_base = M * mantissa + column
					const uint32_t bm = div_key(best - key_base, key_magic);
					mine = bchunk * 32u + ((best - key_base) - bm * key_mult);
					asg[p] = mine;
					const float gap = second == 0xFFFFFFFFu ? INFINITY : (float)(div_key(second - key_base, key_magic) - bm) * ulp;
					const float margin = margin_coef * (xn + c2max) + 4.0f * ulp;
					flag = gap <= margin;
				}
				append_flagged(flag, (uint32_t)p, ctl, flag_list, n);
			}
			if (fuse_acc != nullptr) {
				// Update sums: the final clusters go to shared memory; the reductions themselves are
				// sent later (flush_sums), spread over the next step.
				if (g == merger) {
					uint32_t* s_mine = mg_state + 2 * 3 * 3 * TC_MTILE + (it & 1u) * TC_MTILE;
					s_mine[row] = mine;
					if (mine != 0xFFFFFFFFu) atomicAdd(&fuse_counts[mine], 1u);
					asm volatile("bar.arrive %0, 128;" :: "r"(9u + q) : "memory");
				}
				pending = true;
				pend_it = it;
			}
		}
		if (pending) flush_sums();
	}

	// Both CTAs stay until neither can touch the other's shared memory or barriers any more.
	__syncwarp();
	ptx::tc_fence_before();
	ptx::cluster_sync();
	if (warp == 1) {
		ptx::tc_fence_after();
		ptx::tmem_dealloc_pair(tmem_base, TC_TMEM_COLS);
	}
	if (threadIdx.x == 0 && bars->abort_flag) atomicOr(&ctl->status, (uint32_t)STATUS_WAIT_TIMEOUT);
}

// Sets the kernel up and reports how many CTA pairs the device can hold at once.  The kernel is
// persistent: launching more pairs than are co-resident would make the surplus run as a second
// wave after the first has finished all its work.  Not every SM can be paired (pairs do not span
// GPCs, and a GPC may have an odd number of SMs), so the answer can be less than SMs / 2.
cudaError_t assign_tc_pair_prepare(int sm_count, int* max_pairs)
{
	cudaError_t e = cudaFuncSetAttribute(assign_tc_pair_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_ALLOC);
	if (e != cudaSuccess) return e;
	e = cudaFuncSetAttribute(assign_tc_pair_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P2_ALLOC);
	if (e != cudaSuccess) return e;
	cudaLaunchConfig_t cfg = {};
	cfg.gridDim = dim3(2 * (uint32_t)(sm_count / 2), 1, 1);
	cfg.blockDim = dim3(TC_THREADS, 1, 1);
	cfg.dynamicSmemBytes = P2_ALLOC;
	cudaLaunchAttribute attr;
	attr.id = cudaLaunchAttributeClusterDimension;
	attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
	cfg.attrs = &attr;
	cfg.numAttrs = 1;
	int clusters = 0;
	e = cudaOccupancyMaxActiveClusters(&clusters, assign_tc_pair_kernel<4>, &cfg);
	if (e != cudaSuccess) return e;
	*max_pairs = clusters;
	return cudaSuccess;
}

cudaError_t launch_assign_tc_pair(const CUtensorMap& a_hi, const CUtensorMap& a_lo, const CUtensorMap& b_hi, const CUtensorMap& b_lo,
	const float* b_aug, const float* xnorm, uint32_t* asg, uint64_t n, uint32_t n_tiles, uint32_t k, uint32_t k_pad, uint32_t d_pad,
	uint32_t ksteps, int max_pairs, Control* ctl, int slot, uint32_t* flag_list, float margin_coef, cudaStream_t stream,
	const FusedAcc* fused, uint32_t dim, uint32_t step_begin, uint32_t step_end)
{
	const uint32_t kw = d_pad == 16 ? 16u : TC_KCHUNK;
	const uint32_t n_ctiles = k_pad / TC_NT_MAX;
	const uint32_t steps_all = (n_tiles + 1) / 2;
	if (step_end == 0 || step_end > steps_all) step_end = steps_all;
	if (step_begin >= step_end) return cudaErrorInvalidValue;
	const uint32_t pairs = std::min<uint32_t>(step_end - step_begin, (uint32_t)max_pairs);
	// c_format = f32 (bit 4), a/b format = tf32 (bits 7.., 10..), K-major both, N>>3 at bit 17, M>>4 at bit 24: M = 256 over the pair, N = 128
	const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((P2_UNIT_COLS >> 3) << 17) | (((2 * TC_MTILE) >> 4) << 24);
	if (ksteps == 4)
		assign_tc_pair_kernel<4><<<2 * pairs, TC_THREADS, P2_ALLOC, stream>>>(a_hi, a_lo, b_hi, b_lo, b_aug, xnorm, asg,
			n, n_tiles, k, n_ctiles, kw, ksteps, idesc, ctl, slot, flag_list, margin_coef,
			fused ? fused->acc : nullptr, fused ? fused->counts : nullptr, fused ? fused->center : nullptr, dim, step_begin, step_end);
	else if (ksteps == 3)
		assign_tc_pair_kernel<3><<<2 * pairs, TC_THREADS, P2_ALLOC, stream>>>(a_hi, a_lo, b_hi, b_lo, b_aug, xnorm, asg,
			n, n_tiles, k, n_ctiles, kw, ksteps, idesc, ctl, slot, flag_list, margin_coef,
			fused ? fused->acc : nullptr, fused ? fused->counts : nullptr, fused ? fused->center : nullptr, dim, step_begin, step_end);
	else
		return cudaErrorInvalidValue;       // dim 17..32 only: three or four K steps
	return cudaGetLastError();
}

} // namespace bkm
