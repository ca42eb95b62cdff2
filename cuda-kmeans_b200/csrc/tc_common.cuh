// Device helpers shared by the tensor-core assignment kernels: shared-memory operand descriptors
// for tcgen05.mma, the bounded wait, and the arg-min over accumulator columns on integer keys.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "kernels.cuh"
#include "ptx.cuh"
#include "keys.cuh"

namespace bkm {

constexpr uint32_t TC_MA = 2;            // point tiles per block (= TMEM accumulators)
constexpr uint32_t TC_NB = 2;            // centroid-tile stages
constexpr uint32_t TC_NT_MAX = 256;      // centroids per tile (the widest MMA: N = 256)
constexpr uint32_t TC_EPI_WARPS = 16;          // four per TMEM lane quarter, each a quarter of the columns
constexpr uint32_t TC_THREADS = (2 + TC_EPI_WARPS) * 32;
constexpr uint32_t TC_MAX_KPAD = 1u << 20;
constexpr uint32_t TC_TMEM_COLS = 512;


__device__ __forceinline__ float to_tf32(float x)
{
	uint32_t u;
	asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
	return __uint_as_float(u);
}

// Bounded wait that also gives up when another role already failed.  try_wait suspends the
// thread for a while by itself but comes back early often, so the loop around it decides how
// much the waiting warps take from the warps that work.  SLEEP_NS = 0: look at the abort flag
// and the clock in every round (the clock read is slow and paces the loop).  SLEEP_NS > 0:
// sleep between rounds and look at flag and clock every 256th round only.  LEAN: the 256 rounds
// run as one six-instruction loop (the CTA-pair kernel gained 1.4 % from it, the one-CTA kernel
// lost 2 %: measured, not explained).
template<uint32_t SLEEP_NS = 0, bool LEAN = false>
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag)
{
	if (ptx::mbar_try_wait(bar, parity)) return true;
	if (SLEEP_NS != 0 && LEAN) {
		uint64_t t0 = 0;
		while (true) {
			if (ptx::mbar_poll_round<SLEEP_NS>(bar, parity, 256)) return true;
			if (*abort_flag) return false;
			const uint64_t now = ptx::globaltimer_ns();
			if (t0 == 0) t0 = now;
			else if (now - t0 > ptx::WAIT_LIMIT_NS) break;
		}
	} else if (SLEEP_NS == 0) {
		const uint64_t t0 = ptx::globaltimer_ns();
		while (true) {
			if (ptx::mbar_try_wait(bar, parity)) return true;
			if (*abort_flag) return false;
			if (ptx::globaltimer_ns() - t0 > ptx::WAIT_LIMIT_NS) break;
		}
	} else {
		uint32_t spins = 0;
		uint64_t t0 = 0;
		while (true) {
			if (ptx::mbar_try_wait(bar, parity)) return true;
			__nanosleep(SLEEP_NS);
			if ((++spins & 255u) == 0) {
				if (*abort_flag) return false;
				const uint64_t now = ptx::globaltimer_ns();
				if (t0 == 0) t0 = now;
				else if (now - t0 > ptx::WAIT_LIMIT_NS) break;
			}
		}
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

// The two 32-bit halves of those descriptors: the low half holds the address field (>> 4) and the
// leading byte offset, the high half is a constant of the layout.
constexpr uint32_t DESC_HI_SW128 = 64u | (1u << 14) | (2u << 29);     // 128-byte swizzle, 8-row groups 1024 B apart
constexpr uint32_t DESC_HI_AUG = 16u | (1u << 14);                    // no swizzle, row groups 256 B apart
constexpr uint32_t DESC_HI_SW64 = 32u | (1u << 14) | (4u << 29);      // 64-byte swizzle, 8-row groups 512 B apart
__device__ __forceinline__ uint32_t desc_lo_sw128(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_aug(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (8u << 16); }

// The constant A operand of the extra K step (128 rows, no-swizzle layout): columns 0 and 1 are
// one (they meet the high and the low part of |c|^2), columns 2 and 3 hold the offset constant as
// tf32 hi/lo (they meet ones on the B side), the rest is zero.
__device__ __forceinline__ void fill_a_aug(float* a_aug, float offset_c, uint32_t tid, uint32_t nthreads)
{
	const float c_hi = to_tf32(offset_c), c_lo = to_tf32(offset_c - c_hi);
	for (uint32_t e = tid; e < TC_MTILE * 8; e += nthreads) {
		const uint32_t row = e >> 3, kk = e & 7u;
		a_aug[aug_offset(row, kk)] = kk < 2 ? 1.0f : (kk == 2 ? c_hi : (kk == 3 ? c_lo : 0.0f));
	}
}

// ---- the CTA-pair kernel (assign_tc_pair.cu), used through the plan of assign_tc.cu ----
bool assign_tc_pair_supported(uint32_t k, uint32_t k_pad, uint32_t d_pad, uint32_t nt_cols, int sm_count);
cudaError_t assign_tc_pair_prepare(int sm_count, int* max_pairs);
cudaError_t launch_assign_tc_pair(const CUtensorMap& a_hi, const CUtensorMap& a_lo, const CUtensorMap& b_hi, const CUtensorMap& b_lo,
	const float* b_aug, const float* xnorm, uint32_t* asg, uint64_t n, uint32_t n_tiles, uint32_t k, uint32_t k_pad, uint32_t d_pad,
	uint32_t ksteps, int max_pairs, Control* ctl, int slot, uint32_t* flag_list, float margin_coef, cudaStream_t stream,
	const FusedAcc* fused, uint32_t dim, uint32_t step_begin = 0, uint32_t step_end = 0);

} // namespace bkm
