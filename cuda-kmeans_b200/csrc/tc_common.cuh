// Device helpers shared by the tensor-core assignment kernels: shared-memory operand descriptors
// for tcgen05.mma, the bounded wait, and the arg-min over accumulator columns on integer keys.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "kernels.cuh"
#include "ptx.cuh"

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
// sleep between rounds and look at flag and clock every 256th round only.
template<uint32_t SLEEP_NS = 0>
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag)
{
	if (ptx::mbar_try_wait(bar, parity)) return true;
	if (SLEEP_NS == 0) {
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

__device__ __forceinline__ uint32_t umin3(uint32_t a, uint32_t b, uint32_t c) { return __vimin3_u32(a, b, c); }

// One 32-column chunk of an accumulator row.  The kernel adds a constant to every value so that
// all of them are positive floats with the SAME exponent; their bit patterns then order like the
// values, the upper exponent bits carry no information, and bits * M + column (M odd, > column:
// one integer multiply-add, off the min/max pipe) is a key that keeps the full 23-bit mantissa
// and carries the column position.  The keys are reduced to the two smallest and merged into the running
// (best, second, chunk of best).  `nvalid` < 32 masks the padding columns behind the last mean.
// Smallest of 32 keys with three-input minima (16 instructions).
__device__ __forceinline__ uint32_t min_of_32(const uint32_t (&p)[32])
{
	uint32_t a[12];
	#pragma unroll
	for (int i = 0; i < 10; ++i) a[i] = umin3(p[3 * i], p[3 * i + 1], p[3 * i + 2]);
	a[10] = p[30];
	a[11] = p[31];
	uint32_t c[4];
	#pragma unroll
	for (int i = 0; i < 4; ++i) c[i] = umin3(a[3 * i], a[3 * i + 1], a[3 * i + 2]);
	return min(umin3(c[0], c[1], c[2]), c[3]);
}

template<bool MASKED>
__device__ __forceinline__ void chunk_update(const uint32_t (&v)[32], uint32_t key_mult, uint32_t chunk_id, uint32_t nvalid,
	uint32_t& best, uint32_t& second, uint32_t& best_chunk)
{
	uint32_t p[32];
	#pragma unroll
	for (uint32_t t = 0; t < 32; ++t) p[t] = v[t] * key_mult + t;
	if (MASKED && nvalid < 32) {
		#pragma unroll
		for (uint32_t t = 0; t < 32; ++t) p[t] = t < nvalid ? p[t] : 0xFFFFFFFFu;
	}
	// Two passes of plain minima instead of a (best, second) tournament.  The keys are distinct
	// (they carry the column), so key - (smallest + 1) wraps to the top of the unsigned range for
	// the smallest key only, and the minimum of these differences belongs to the second smallest.
	// The second pass is 32 fused add-and-minimum instructions in four independent chains;
	// 16 + 32 + 8 integer instructions per chunk where a tournament takes 77 + 5.
	const uint32_t b = min_of_32(p);
	const uint32_t nb1 = ~b;                       // -(b + 1)
	uint32_t r0 = 0xFFFFFFFFu, r1 = 0xFFFFFFFFu, r2 = 0xFFFFFFFFu, r3 = 0xFFFFFFFFu;
	#pragma unroll
	for (uint32_t t = 0; t < 32; t += 4) {
		r0 = __viaddmin_u32(p[t], nb1, r0);
		r1 = __viaddmin_u32(p[t + 1], nb1, r1);
		r2 = __viaddmin_u32(p[t + 2], nb1, r2);
		r3 = __viaddmin_u32(p[t + 3], nb1, r3);
	}
	const uint32_t s2 = min(umin3(r0, r1, r2), r3) - nb1;      // + (b + 1); a lone valid key gives 0xFFFFFFFF again
	second = umin3(second, max(best, b), s2);
	best_chunk = b < best ? chunk_id : best_chunk;
	best = min(best, b);
}


// The constants that turn accumulator values into integer keys (see chunk_update).
struct KeyConsts {
	float pow2;          // P: every accumulator value lies in [P, 2P)
	float offset_c;      // constant added to every |c|^2 - 2 x.c by the extra K step
	uint32_t key_mult;   // M
	uint32_t key_base;   // M * (bit pattern of P) mod 2^32
	uint32_t key_magic;  // multiplier of div_key for this M
};

// Offset constant: every value |c|^2 - 2 x.c lies in [-X2, X2 + 2*C2] (X2, C2 = largest |x|^2,
// |c|^2 after centring), an interval of width 2*(X2+C2); with P a power of two >= 1.25 times
// that width, value + P + X2 + P/32 stays inside [P, 2P) with P/32 of head-room on both
// sides for the rounding of the pass: one exponent for all values.
// Key of a value with bit pattern v in column t: v * M + t (mod 2^32) = key_base + M * mantissa + t.
// M is an odd number >= 33 chosen so that the largest key stays below 2^32: keys then order like
// (value, column).  A multiplier that is not a power of two keeps the multiply-add on the FMA
// pipe; the min/max tournament owns the ALU pipe.
__device__ __forceinline__ KeyConsts make_key_consts(float x2max, float c2max)
{
	KeyConsts kc;
	const float span = 1.25f * (2.0f * (x2max + c2max)) + 1.0e-30f;
	int e;
	frexpf(span, &e);                       // span = m * 2^e, m in [0.5, 1)
	kc.pow2 = ldexpf(1.0f, e);              // >= span
	kc.offset_c = kc.pow2 + x2max + kc.pow2 * (1.0f / 32.0f);
	kc.key_mult = 33;
	const uint32_t eb = __float_as_uint(kc.pow2) >> 23;
	while (kc.key_mult < 63 && ((kc.key_mult * eb) & 511u) > 510u - kc.key_mult) kc.key_mult += 2;
	kc.key_base = kc.key_mult * __float_as_uint(kc.pow2);
	kc.key_magic = (uint32_t)((((unsigned long long)(64u - kc.key_mult)) << 32) / kc.key_mult) + 1u;
	return kc;
}

// x / M for the key multipliers (33 <= M <= 63) without the integer-division sequence: with
// magic = floor(2^32 * (64 - M) / M) + 1 and t = high word of magic * x, the quotient is
// (t + (x - t) / 2) / 32, exact for every 32-bit x (division by an invariant, round-up method).
__device__ __forceinline__ uint32_t div_key(uint32_t x, uint32_t magic)
{
	const uint32_t t = __umulhi(magic, x);
	return (t + ((x - t) >> 1)) >> 5;
}

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
	const FusedAcc* fused, uint32_t dim);

} // namespace bkm
