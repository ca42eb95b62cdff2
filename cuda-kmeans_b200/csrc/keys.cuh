// Integer keys for the arg-min over approximate squared distances, shared by the tensor-core and
// the CUDA-core fast passes: values that all lie in one binade are turned into (value, column)
// keys whose unsigned order is the order of (value, column), and chunks of 32 keys are reduced to
// the smallest and the second smallest with plain integer minima.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

#include "common.cuh"

namespace bkm {

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
	// (the chains start from their first keys: an add each instead of a constant and an add-and-minimum)
	uint32_t r0 = p[0] + nb1, r1 = p[1] + nb1, r2 = p[2] + nb1, r3 = p[3] + nb1;
	#pragma unroll
	for (uint32_t t = 4; t < 32; t += 4) {
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

// Appends the points whose `flag` is set to the near-tie list with ONE atomic per warp (a counter
// that every flagged point bumps by itself is a serial bottleneck once a few per cent of the points
// are flagged).  All 32 lanes of the warp must call it together.
__device__ __forceinline__ void append_flagged(bool flag, uint32_t point, Control* __restrict__ ctl, uint32_t* __restrict__ flag_list, uint64_t n)
{
	const uint32_t mask = __ballot_sync(0xffffffffu, flag);
	if (mask == 0) return;
	const uint32_t lane = threadIdx.x & 31u;
	const int leader = __ffs(mask) - 1;
	uint32_t base = 0;
	if ((int)lane == leader) base = atomicAdd(&ctl->flag_count, (uint32_t)__popc(mask));
	base = __shfl_sync(0xffffffffu, base, leader);
	if (flag) {
		const uint32_t pos = base + (uint32_t)__popc(mask & ((1u << lane) - 1u));
		if ((uint64_t)pos < n) flag_list[pos] = point;
		else atomicOr(&ctl->status, (uint32_t)STATUS_LIST_OVERFLOW);
	}
}

// The same through a small buffer in shared memory that belongs to one warp: flagged points collect
// there and go out FLAG_BUFFER entries at a time, so that the round trip of the global counter is
// paid once per buffer instead of once per call (a warp that waits for it does nothing else).
// `cnt` lives in a register and is the same in all lanes.  All 32 lanes call together; the warp
// calls flush_flag_buffer once more when it is done.
constexpr uint32_t FLAG_BUFFER = 64;

__device__ __forceinline__ void flush_flag_buffer(uint32_t* buf, uint32_t& cnt, Control* __restrict__ ctl, uint32_t* __restrict__ flag_list, uint64_t n)
{
	if (cnt == 0) return;
	const uint32_t lane = threadIdx.x & 31u;
	uint32_t base = 0;
	if (lane == 0) base = atomicAdd(&ctl->flag_count, cnt);
	base = __shfl_sync(0xffffffffu, base, 0);
	for (uint32_t e = lane; e < cnt; e += 32) {
		if ((uint64_t)(base + e) < n) flag_list[base + e] = buf[e];
		else atomicOr(&ctl->status, (uint32_t)STATUS_LIST_OVERFLOW);
	}
	__syncwarp();
	cnt = 0;
}

__device__ __forceinline__ void buffered_append(bool flag, uint32_t point, uint32_t* buf, uint32_t& cnt, Control* __restrict__ ctl,
	uint32_t* __restrict__ flag_list, uint64_t n)
{
	const uint32_t mask = __ballot_sync(0xffffffffu, flag);
	if (mask == 0) return;
	const uint32_t m = (uint32_t)__popc(mask);
	if (cnt + m > FLAG_BUFFER) flush_flag_buffer(buf, cnt, ctl, flag_list, n);
	const uint32_t lane = threadIdx.x & 31u;
	if (flag) buf[cnt + (uint32_t)__popc(mask & ((1u << lane) - 1u))] = point;
	cnt += m;
	__syncwarp();
}

} // namespace bkm
