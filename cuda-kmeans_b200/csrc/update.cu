// Update step: per-cluster sums and sizes, merge, divide, and the preparation of the
// assignment operands from the fresh means.
//
//  * update_kernel<SOA, SHARED>: every block owns a contiguous slice of the points and
//    accumulates it with atomics either into shared-memory copies of the k x dim buckets
//    (SHARED; `replicas` copies, picked by warp so that warps hitting the same hot cluster do
//    not contend on one address) followed by one merge into the global accumulators, or
//    straight into the global accumulators when k*dim does not fit.  Replaces
//    updateAtomicPointKernel / updateAtomicFineKernel / updateAtomicShmKernel
//    (kernels/kernels.cu:727-743, 771-791, 818-858 of the reference) and follows the shared
//    privatisation idea of atomicShm2Kernel (bucketing-cuda kernels/kernels.cu:382-422).
//
//  * finalize_prepare_kernel: mean = sum / size (an empty cluster keeps zeros), written in the
//    means layout - the work of reducePrivCopiesKernel + divideMeansKernel
//    (kernels/kernels.cu:116-135, 150-163) - fused with the derivation of the operands the
//    next assignment reads and with clearing the accumulators (fillZeros, :13-17).
#include "kernels.cuh"
#include "../../include/bkm.h"

#include <algorithm>
#include <cmath>

namespace bkm {

__device__ __forceinline__ void red_add_v2(float* addr, float a, float b)
{
	asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" :: "l"(addr), "f"(a), "f"(b) : "memory");
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d)
{
	asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

int current_sm_count()
{
	static int cache[64] = {};
	int dev = 0;
	if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 1; }
	if (dev >= 0 && dev < 64 && cache[dev] > 0) return cache[dev];
	int sms = 0;
	if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) { cudaGetLastError(); return 1; }
	if (dev >= 0 && dev < 64) cache[dev] = sms;
	return sms;
}

constexpr int UPD_THREADS = 512;
constexpr size_t SMEM_LIMIT = 227 * 1024;

__device__ __forceinline__ float tf32_rna(float x)
{
	uint32_t u;
	asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
	return __uint_as_float(u);
}

// ------------------------------------------------------------------------------------------
// finalize / prepare
// ------------------------------------------------------------------------------------------

// Where the rows of the fresh means go: the means themselves (in their layout), the cluster sizes,
// and the operands the next assignment pass reads.
struct RowSinks {
	float* means_out; uint32_t* sizes_out;
	uint32_t k, d; int soa_means;
	float* cprep; uint32_t rs, srows;
	float* b_hi; float* b_lo; float* cnorm; float* b_aug; const float* center; uint32_t k_pad, d_pad;
	Control* ctl; int slot;
	int divide;            // 0: the rows are written as sums (bucketing), 1: as means
};

// One warp finishes row c < k.  `mean_of(j)` yields coordinate j of the mean (lane-strided calls).
template<class MEAN>
__device__ __forceinline__ void finish_row(const RowSinks& o, uint32_t c, uint32_t lane, bool write_means, uint32_t cnt, MEAN mean_of)
{
	float s2 = 0.0f;
	for (uint32_t j = lane; j < o.d; j += 32) {
		const float mean = mean_of(j);
		if (write_means) o.means_out[at_rt(o.soa_means, c, j, o.k, o.d)] = mean;
		// the tensor-core operands and the norms use the mean relative to the common centre
		const float shifted = o.center ? mean - o.center[j] : mean;
		s2 = fmaf(shifted, shifted, s2);
		const float b = -2.0f * shifted;
		if (o.cprep) o.cprep[(size_t)c * o.rs + 1 + j] = b;
		if (o.b_hi) {
			const float hi = tf32_rna(b);
			const float lo = tf32_rna(b - hi);
			o.b_hi[(size_t)c * o.d_pad + j] = hi;
			o.b_lo[(size_t)c * o.d_pad + j] = lo;
		}
	}
	#pragma unroll
	for (int off = 16; off > 0; off >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, off);
	__syncwarp();
	if (lane == 0) {
		if (o.cprep) o.cprep[(size_t)c * o.rs] = s2;
		if (o.cnorm) o.cnorm[c] = s2;
		if (o.b_aug) {
			const float hi = tf32_rna(s2);
			const float lo = tf32_rna(s2 - hi);
			float4* dst = reinterpret_cast<float4*>(o.b_aug + aug_offset(c, 0));
			dst[0] = make_float4(hi, lo, 1.0f, 1.0f);
			dst[8] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);    // columns 4..7 sit 32 floats further
		}
		atomicMax(reinterpret_cast<int*>(&o.ctl->cmax2[o.slot]), __float_as_int(s2));
		if (write_means && o.sizes_out) o.sizes_out[c] = cnt;
	}
}

// Rows behind the last mean: padding that can never win (their additive term is +inf, the coordinates stay zero).
__device__ __forceinline__ void finish_padding_row(const RowSinks& o, uint32_t c)
{
	if (o.cprep && c < o.srows) o.cprep[(size_t)c * o.rs] = INFINITY;
	if (o.cnorm && c < o.k_pad) o.cnorm[c] = INFINITY;
	if (o.b_aug && c < o.k_pad) {
		float4* dst = reinterpret_cast<float4*>(o.b_aug + aug_offset(c, 0));
		dst[0] = make_float4(0.0f, 0.0f, 1.0f, 1.0f);
		dst[8] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
	}
}

__device__ __forceinline__ void finish_control(Control* ctl, int slot)
{
	ctl->last_flag_count = ctl->flag_count;
	ctl->flag_count = 0;
	ctl->cmax2[slot ^ 1] = 0.0f;
}

__device__ __forceinline__ uint32_t rows_to_finish(const RowSinks& o)
{
	uint32_t rows_total = o.k;
	if (o.cprep && o.srows > rows_total) rows_total = o.srows;
	if (o.cnorm && o.k_pad > rows_total) rows_total = o.k_pad;
	return rows_total;
}

// Sum over the `replicas` copies of one accumulator word (copies `rep_stride` words apart), clearing them.
__device__ __forceinline__ float sum_and_clear(float* src, uint32_t replicas, size_t rep_stride)
{
	float sum = 0.0f;
	uint32_t r = 0;
	for (; r + 4 <= replicas; r += 4) {
		// four independent loads in flight
		const float s0 = src[(r + 0) * rep_stride], s1 = src[(r + 1) * rep_stride];
		const float s2b = src[(r + 2) * rep_stride], s3 = src[(r + 3) * rep_stride];
		src[(r + 0) * rep_stride] = 0.0f; src[(r + 1) * rep_stride] = 0.0f;
		src[(r + 2) * rep_stride] = 0.0f; src[(r + 3) * rep_stride] = 0.0f;
		sum += (s0 + s1) + (s2b + s3);
	}
	for (; r < replicas; ++r) { sum += src[r * rep_stride]; src[r * rep_stride] = 0.0f; }
	return sum;
}

// `replicas` copies of (sums, sizes) lie `rep_stride` 32-bit words apart; all are added up and cleared.
template<bool FINALIZE>
__global__ void __launch_bounds__(256) finalize_prepare_kernel(float* __restrict__ acc, uint32_t* __restrict__ counts,
	uint32_t replicas, size_t rep_stride, const float* __restrict__ means_in, RowSinks o)
{
	const uint32_t lane = threadIdx.x & 31u;
	const uint32_t wpb = blockDim.x >> 5;
	const uint32_t rows_total = rows_to_finish(o);
	for (uint32_t c = blockIdx.x * wpb + (threadIdx.x >> 5); c < rows_total; c += gridDim.x * wpb) {
		if (c < o.k) {
			if (FINALIZE) {
				uint32_t cnt = 0;
				for (uint32_t r = 0; r < replicas; ++r) cnt += counts[c + r * rep_stride];
				const float divisor = (float)cnt;
				finish_row(o, c, lane, true, cnt, [&](uint32_t j) {
					const float sum = sum_and_clear(acc + (size_t)c * o.d + j, replicas, rep_stride);
					if (!o.divide) return sum;
					return cnt ? __fdiv_rn(sum, divisor) : 0.0f;
				});
				__syncwarp();
				if (lane == 0) for (uint32_t r = 0; r < replicas; ++r) counts[c + r * rep_stride] = 0;
			} else {
				finish_row(o, c, lane, false, 0u, [&](uint32_t j) { return means_in[at_rt(o.soa_means, c, j, o.k, o.d)]; });
			}
		} else if (lane == 0) {
			finish_padding_row(o, c);
		}
	}
	if (blockIdx.x == 0 && threadIdx.x == 0) finish_control(o.ctl, o.slot);
}

// ------------------------------------------------------------------------------------------
// exchange between ranks + finalize, in one kernel
// ------------------------------------------------------------------------------------------
//
// Every rank owns one receive buffer that its peers can write (mapped into their address space):
//   two slots x EXCHANGE_MAX_RANKS senders x (k*dim sums, k sizes), every word an 8-byte packet
//   (value in the low half, iteration count in the high half).
// A rank adds up its accumulator copies and stores each total, tagged with the iteration count,
// straight into the receive buffers of ALL ranks (its own included) with single 64-bit stores:
// value and tag arrive together, so no separate flag and no fence is needed, and the data cross
// NVLink once, as posted writes.  It then polls its OWN buffer, word by word, until the packets
// of every sender carry this iteration's count, adds the values in rank order - so every rank
// computes bit-identical means - divides, and writes the means and the next assignment's operands
// as finalize_prepare_kernel does.  Every block sends all its words before it waits for any, and
// the grid never exceeds the number of SMs, so no rank can wait for a word that its sender has not
// been able to send.  Two slots (iteration count & 1) are enough: a rank can send iteration t+2
// only after it has received every peer's t+1, which a peer sends after it has consumed t.
// Waits are bounded; one that runs out sets STATUS_WAIT_TIMEOUT and the kernel carries on.
__device__ __forceinline__ void st_packet(uint64_t* p, uint64_t v)
{
	asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ uint64_t ld_packet(const uint64_t* p)
{
	uint64_t v;
	asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
	return v;
}

struct ExchangePeers {
	uint64_t* base[EXCHANGE_MAX_RANKS];   // receive buffer of every rank (own one included), as seen from this GPU
};

// Packets of word `w` from all `world` senders, once each carries `epoch` (or the time limit has passed).
__device__ __forceinline__ void poll_packets(const uint64_t* slot, size_t words, size_t w, uint32_t world, uint32_t epoch,
	uint64_t wait_limit_ns, uint32_t* timed_out, uint32_t (&value)[EXCHANGE_MAX_RANKS])
{
	uint64_t v[EXCHANGE_MAX_RANKS];
	#pragma unroll
	for (uint32_t r = 0; r < EXCHANGE_MAX_RANKS; ++r) v[r] = r < world ? ld_packet(slot + (size_t)r * words + w) : 0ull;
	uint64_t t0 = 0;
	uint32_t spins = 0;
	while (true) {
		bool missing = false;
		#pragma unroll
		for (uint32_t r = 0; r < EXCHANGE_MAX_RANKS; ++r)
			if (r < world && (uint32_t)(v[r] >> 32) != epoch) { missing = true; v[r] = ld_packet(slot + (size_t)r * words + w); }
		if (!missing) break;
		if ((++spins & 31u) == 0) {
			uint64_t now;
			asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
			if (t0 == 0) t0 = now;
			else if (now - t0 > wait_limit_ns || *reinterpret_cast<volatile uint32_t*>(timed_out)) { *timed_out = 1; break; }
		}
	}
	#pragma unroll
	for (uint32_t r = 0; r < EXCHANGE_MAX_RANKS; ++r) value[r] = (uint32_t)v[r];
}

__global__ void __launch_bounds__(256) exchange_finalize_kernel(float* __restrict__ acc, uint32_t* __restrict__ counts,
	uint32_t replicas, size_t rep_stride, ExchangePeers peers, uint32_t world, uint32_t rank, uint32_t epoch,
	uint64_t wait_limit_ns, RowSinks o)
{
	__shared__ uint32_t s_timeout;
	const uint32_t lane = threadIdx.x & 31u, wpb = blockDim.x >> 5;
	const uint32_t gwarp = blockIdx.x * wpb + (threadIdx.x >> 5), gwarps = gridDim.x * wpb;
	const uint32_t rows_total = rows_to_finish(o);
	const size_t kd = (size_t)o.k * o.d;
	const size_t words = exchange_slot_words(o.k, o.d);
	const size_t slot_off = (size_t)(epoch & 1u) * EXCHANGE_MAX_RANKS * words;
	const uint64_t tag = (uint64_t)epoch << 32;
	// once a wait has run out (status word still set: the host has not looked yet), later iterations
	// of the same run do not wait again
	if (threadIdx.x == 0) s_timeout = (o.ctl->status & (uint32_t)STATUS_WAIT_TIMEOUT) ? 1u : 0u;
	__syncthreads();
	if (s_timeout) wait_limit_ns = 0;

	// 1. send this rank's totals of the block's rows to every rank
	for (uint32_t c = gwarp; c < o.k; c += gwarps) {
		for (uint32_t j = lane; j < o.d; j += 32) {
			const size_t w = (size_t)c * o.d + j;
			const uint64_t pkt = tag | __float_as_uint(sum_and_clear(acc + w, replicas, rep_stride));
			for (uint32_t r = 0; r < world; ++r) st_packet(peers.base[r] + slot_off + (size_t)rank * words + w, pkt);
		}
		// sizes: the lanes share the accumulator copies, then lane r sends to rank r
		uint32_t cnt = 0;
		for (uint32_t r = lane; r < replicas; r += 32) { cnt += counts[c + r * rep_stride]; counts[c + r * rep_stride] = 0; }
		#pragma unroll
		for (int off = 16; off > 0; off >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
		if (lane < world) st_packet(peers.base[lane] + slot_off + (size_t)rank * words + kd + c, tag | cnt);
	}

	// 2. receive all ranks' totals (from this rank's own buffer), add in rank order, divide, next operands
	const uint64_t* slot = peers.base[rank] + slot_off;
	for (uint32_t c = gwarp; c < rows_total; c += gwarps) {
		if (c < o.k) {
			uint32_t part[EXCHANGE_MAX_RANKS];
			poll_packets(slot, words, kd + c, world, epoch, wait_limit_ns, &s_timeout, part);
			uint32_t cnt = 0;
			#pragma unroll
			for (uint32_t r = 0; r < EXCHANGE_MAX_RANKS; ++r) if (r < world) cnt += part[r];
			const float divisor = (float)cnt;
			finish_row(o, c, lane, true, cnt, [&](uint32_t j) {
				uint32_t bits[EXCHANGE_MAX_RANKS];
				poll_packets(slot, words, (size_t)c * o.d + j, world, epoch, wait_limit_ns, &s_timeout, bits);
				float sum = 0.0f;
				#pragma unroll
				for (uint32_t r = 0; r < EXCHANGE_MAX_RANKS; ++r) if (r < world) sum += __uint_as_float(bits[r]);
				return cnt ? __fdiv_rn(sum, divisor) : 0.0f;
			});
		} else if (lane == 0) {
			finish_padding_row(o, c);
		}
	}
	__syncthreads();
	if (threadIdx.x == 0 && s_timeout) atomicOr(&o.ctl->status, (uint32_t)STATUS_WAIT_TIMEOUT);
	if (blockIdx.x == 0 && threadIdx.x == 0) finish_control(o.ctl, o.slot);
}

static RowSinks make_sinks(float* means_out, uint32_t* sizes_out, const Shape& s, const SimtMeans* sm, const TcMeans* tc, Control* ctl, int slot)
{
	RowSinks o;
	o.means_out = means_out; o.sizes_out = sizes_out;
	o.k = s.k; o.d = s.dim; o.soa_means = s.soa_means;
	o.cprep = sm ? sm->rows : nullptr; o.rs = simt_row_stride(s.dim); o.srows = simt_rows(s.k);
	o.b_hi = tc ? tc->b_hi : nullptr; o.b_lo = tc ? tc->b_lo : nullptr;
	o.cnorm = tc ? tc->cnorm : nullptr; o.b_aug = tc ? tc->b_aug : nullptr;
	o.center = tc ? tc->center : (sm ? sm->center : nullptr);
	o.k_pad = tc ? tc->k_pad : 0; o.d_pad = tc ? tc->d_pad : 0;
	o.ctl = ctl; o.slot = slot;
	o.divide = 1;
	return o;
}

static uint32_t sink_rows(const Shape& s, const SimtMeans* sm, const TcMeans* tc)
{
	uint32_t rows_total = s.k;
	if (sm) rows_total = std::max(rows_total, simt_rows(s.k));
	if (tc) rows_total = std::max(rows_total, tc->k_pad);
	return rows_total;
}

size_t exchange_buffer_bytes(uint32_t k, uint32_t dim)
{
	return 2 * (size_t)EXCHANGE_MAX_RANKS * exchange_slot_words(k, dim) * sizeof(uint64_t);
}

cudaError_t launch_exchange_finalize(float* acc, uint32_t* counts, uint32_t replicas, void* const* peer_bases, uint32_t world,
	uint32_t rank, uint32_t epoch, uint64_t wait_limit_ns, float* means_out, uint32_t* sizes_out, const Shape& s,
	const SimtMeans* sm, const TcMeans* tc, Control* ctl, int slot, cudaStream_t stream)
{
	if (world < 1 || world > EXCHANGE_MAX_RANKS || rank >= world) return cudaErrorInvalidValue;
	ExchangePeers peers;
	for (uint32_t r = 0; r < EXCHANGE_MAX_RANKS; ++r) peers.base[r] = r < world ? static_cast<uint64_t*>(peer_bases[r]) : nullptr;
	const uint32_t rows_total = sink_rows(s, sm, tc);
	// never more blocks than SMs: all of them are resident together (see the kernel)
	const uint32_t wpb = 8;
	const uint32_t grid = std::min<uint32_t>(std::max<uint32_t>((rows_total + wpb - 1) / wpb, 1), (uint32_t)current_sm_count());
	exchange_finalize_kernel<<<grid, wpb * 32, 0, stream>>>(acc, counts, replicas, acc_replica_stride(s.k, s.dim), peers, world, rank, epoch,
		wait_limit_ns, make_sinks(means_out, sizes_out, s, sm, tc, ctl, slot));
	return cudaGetLastError();
}

static void launch_fp(bool finalize, float* acc, uint32_t* counts, uint32_t replicas, const float* means_in, float* means_out,
	uint32_t* sizes_out, const Shape& s, const SimtMeans* sm, const TcMeans* tc, Control* ctl, int slot, cudaStream_t stream, bool divide = true)
{
	const size_t rep_stride = acc_replica_stride(s.k, s.dim);
	const uint32_t rows_total = sink_rows(s, sm, tc);
	const uint32_t wpb = 8;
	uint32_t grid = (rows_total + wpb - 1) / wpb;
	grid = std::min<uint32_t>(std::max<uint32_t>(grid, 1), (uint32_t)current_sm_count() * 8);
	RowSinks o = make_sinks(means_out, sizes_out, s, sm, tc, ctl, slot);
	o.divide = divide ? 1 : 0;
	if (finalize)
		finalize_prepare_kernel<true><<<grid, wpb * 32, 0, stream>>>(acc, counts, replicas, rep_stride, means_in, o);
	else
		finalize_prepare_kernel<false><<<grid, wpb * 32, 0, stream>>>(acc, counts, replicas, rep_stride, means_in, o);
}

void launch_prepare_means(const float* means, const Shape& s, const SimtMeans* sm, const TcMeans* tc,
	Control* ctl, int slot, cudaStream_t stream)
{
	launch_fp(false, nullptr, nullptr, 1, means, nullptr, nullptr, s, sm, tc, ctl, slot, stream);
}

void launch_finalize(float* acc, uint32_t* counts, uint32_t replicas, float* means_out, uint32_t* sizes_out, const Shape& s,
	const SimtMeans* sm, const TcMeans* tc, Control* ctl, int slot, cudaStream_t stream)
{
	launch_fp(true, acc, counts, replicas, nullptr, means_out, sizes_out, s, sm, tc, ctl, slot, stream);
}

void launch_finalize_sums(float* acc, uint32_t* counts, uint32_t replicas, float* sums_out, const Shape& s, Control* ctl, cudaStream_t stream)
{
	launch_fp(true, acc, counts, replicas, nullptr, sums_out, nullptr, s, nullptr, nullptr, ctl, 1, stream, false);
}

// ------------------------------------------------------------------------------------------
// write-only probes of the atomic-add throughput
// ------------------------------------------------------------------------------------------
//
// The counterparts of atomicFakeKernel / atomicShmFakeKernel of the reference's bucketing study
// (experimental/bucketing-cuda/bucketing-cuda/kernels/kernels.cu:455-469, 496-531): one thread per
// input value that reads nothing and adds the constant 0.1 to bucket (i / dim) % k, dimension
// i % dim - the cost of the reductions alone.  The shared variant keeps the first `cached` buckets
// in shared memory and flushes them at the end of the block.
template<bool SOA>
__global__ void __launch_bounds__(256) probe_atomics_kernel(float* __restrict__ result, uint64_t total, uint32_t k, uint32_t d, uint32_t cached)
{
	extern __shared__ float cache[];
	for (uint32_t e = threadIdx.x; e < cached * d; e += blockDim.x) cache[e] = 0.0f;
	if (cached) __syncthreads();
	for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
		const uint32_t j = (uint32_t)(i % d);
		const uint32_t target = (uint32_t)((i / d) % k);
		if (target < cached) atomicAdd(&cache[target * d + j], 0.1f);
		else atomicAdd(&result[at<SOA>(target, j, k, d)], 0.1f);
	}
	if (cached) {
		__syncthreads();
		for (uint32_t e = threadIdx.x; e < cached * d; e += blockDim.x) atomicAdd(&result[at<SOA>(e / d, e % d, k, d)], cache[e]);
	}
}

cudaError_t launch_probe_atomics(float* result, uint64_t n, uint32_t k, uint32_t dim, int soa, bool shared_cache, uint32_t items_per_thread,
	cudaStream_t stream)
{
	const uint64_t total = n * dim;
	const uint64_t threads = (total + items_per_thread - 1) / items_per_thread;
	const uint64_t blocks = std::min<uint64_t>(std::max<uint64_t>((threads + 255) / 256, 1), 0x7fffffffull);
	uint32_t cached = 0;
	size_t smem = 0;
	if (shared_cache) {
		cached = (uint32_t)std::min<size_t>(k, (96 * 1024) / ((size_t)dim * sizeof(float)));
		smem = (size_t)cached * dim * sizeof(float);
	}
	if (soa) {
		if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(probe_atomics_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
		probe_atomics_kernel<true><<<(uint32_t)blocks, 256, smem, stream>>>(result, total, k, dim, cached);
	} else {
		if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(probe_atomics_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
		probe_atomics_kernel<false><<<(uint32_t)blocks, 256, smem, stream>>>(result, total, k, dim, cached);
	}
	return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------
// recognising the point set of a stateless call
// ------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256) points_fingerprint_kernel(const uint32_t* __restrict__ bits, uint64_t words, PointsKey* __restrict__ key)
{
	const uint32_t lane = threadIdx.x & 31u;
	const uint64_t lines = (words + 31) / 32;
	const uint64_t samples = (lines + 15) / 16 + 1;             // every 16th line, and the last one
	const uint64_t gwarp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, gwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
	unsigned long long acc = 0;
	for (uint64_t sidx = gwarp; sidx < samples; sidx += gwarps) {
		const uint64_t line = sidx + 1 == samples ? lines - 1 : sidx * 16;
		const uint64_t i = line * 32 + lane;
		if (i < words && (sidx + 1 == samples || line < lines)) {
			unsigned long long x = ((unsigned long long)bits[i] << 32) ^ (i * 0x9E3779B97F4A7C15ull);
			x ^= x >> 29; x *= 0xBF58476D1CE4E5B9ull; x ^= x >> 32;
			acc += x;
		}
	}
	#pragma unroll
	for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
	if (lane == 0 && acc) atomicAdd(&key->fp_new, acc);
}

__global__ void points_key_decide_kernel(PointsKey* key, unsigned long long ptr, unsigned long long n, uint32_t dim, uint32_t layout,
	uint32_t variant, Control* ctl)
{
	const bool same = key->fp_old == key->fp_new && key->ptr == ptr && key->n == n && key->dim == dim && key->layout == layout &&
		key->variant == variant;
	key->valid = same ? 1u : 0u;
	key->fp_old = key->fp_new;
	key->ptr = ptr; key->n = n; key->dim = dim; key->layout = layout; key->variant = variant;
	if (!same) ctl->xmax2 = 0.0f;
}

cudaError_t launch_points_fingerprint(const float* pts, uint64_t words, PointsKey* key, int sm_count, cudaStream_t stream)
{
	const uint64_t samples = ((words + 31) / 32 + 15) / 16 + 1;
	const uint32_t grid = (uint32_t)std::min<uint64_t>((samples + 7) / 8, (uint64_t)sm_count * 8);
	points_fingerprint_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(pts), words, key);
	return cudaGetLastError();
}

cudaError_t launch_points_key_decide(PointsKey* key, const float* pts, const Shape& s, int variant, Control* ctl, cudaStream_t stream)
{
	points_key_decide_kernel<<<1, 1, 0, stream>>>(key, (unsigned long long)reinterpret_cast<uintptr_t>(pts), s.n, s.dim, (uint32_t)s.soa,
		(uint32_t)variant, ctl);
	return cudaGetLastError();
}

// Adds replicas 1.. into replica 0 and clears them (needed before the sums leave the GPU).
__global__ void __launch_bounds__(256) merge_replicas_kernel(float* __restrict__ acc, uint32_t* __restrict__ counts,
	uint32_t replicas, size_t rep_stride, size_t kd, uint32_t k)
{
	for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < kd + k; e += (size_t)gridDim.x * blockDim.x) {
		if (e < kd) {
			float sum = acc[e];
			for (uint32_t r = 1; r < replicas; ++r) { sum += acc[r * rep_stride + e]; acc[r * rep_stride + e] = 0.0f; }
			acc[e] = sum;
		} else {
			const size_t c = e - kd;
			uint32_t sum = counts[c];
			for (uint32_t r = 1; r < replicas; ++r) { sum += counts[r * rep_stride + c]; counts[r * rep_stride + c] = 0; }
			counts[c] = sum;
		}
	}
}

void launch_merge_replicas(float* acc, uint32_t* counts, uint32_t replicas, const Shape& s, cudaStream_t stream)
{
	if (replicas <= 1) return;
	const size_t kd = (size_t)s.k * s.dim;
	const uint32_t grid = (uint32_t)std::min<size_t>((kd + s.k + 255) / 256, (size_t)current_sm_count() * 8);
	merge_replicas_kernel<<<grid, 256, 0, stream>>>(acc, counts, replicas, acc_replica_stride(s.k, s.dim), kd, s.k);
}

// ------------------------------------------------------------------------------------------
// update
// ------------------------------------------------------------------------------------------

template<bool SOA, bool SHARED>
__global__ void __launch_bounds__(UPD_THREADS) update_kernel(const float* __restrict__ pts,
	const uint32_t* __restrict__ asg, float* __restrict__ acc, uint32_t* __restrict__ counts,
	uint64_t n, uint32_t k, uint32_t d, uint32_t dstride, uint32_t replicas, Control* __restrict__ ctl)
{
	extern __shared__ __align__(16) float sacc[];
	const uint32_t tid = threadIdx.x;
	const size_t rep_floats = (size_t)k * dstride;
	uint32_t* scnt = reinterpret_cast<uint32_t*>(sacc + rep_floats * replicas);

	float* my;
	uint32_t* mycnt;
	uint32_t stride;
	if (SHARED) {
		for (size_t e = tid; e < rep_floats * replicas + (size_t)k * replicas; e += UPD_THREADS) sacc[e] = 0.0f;
		__syncthreads();
		const uint32_t r = (tid >> 5) % replicas;
		my = sacc + rep_floats * r;
		mycnt = scnt + (size_t)k * r;
		stride = dstride;
	} else {
		my = acc;
		mycnt = counts;
		stride = d;
	}

	// contiguous slice of points per block, a multiple of 32 points
	uint64_t per = (n + gridDim.x - 1) / gridDim.x;
	per = (per + 31) / 32 * 32;
	const uint64_t p0 = (uint64_t)blockIdx.x * per;
	uint64_t p1 = p0 + per;
	if (p1 > n) p1 = n;
	bool bad = false;

	if (p0 < p1) {
		if (SOA) {
			for (uint64_t i = p0 + tid; i < p1; i += UPD_THREADS) {
				const uint32_t a = asg[i];
				if (a >= k) { bad = true; continue; }
				atomicAdd(&mycnt[a], 1u);
				float* row = my + (size_t)a * stride;
				uint32_t j = 0;
				for (; j + 4 <= d; j += 4) {
					const float v0 = pts[(size_t)(j + 0) * n + i];
					const float v1 = pts[(size_t)(j + 1) * n + i];
					const float v2 = pts[(size_t)(j + 2) * n + i];
					const float v3 = pts[(size_t)(j + 3) * n + i];
					atomicAdd(&row[j + 0], v0);
					atomicAdd(&row[j + 1], v1);
					atomicAdd(&row[j + 2], v2);
					atomicAdd(&row[j + 3], v3);
				}
				for (; j < d; ++j) atomicAdd(&row[j], pts[(size_t)j * n + i]);
			}
		} else {
			// flat walk over the (p1-p0)*d values of the slice; (point, dim) advance without division
			const uint64_t count = (p1 - p0) * d;
			const float* src = pts + (size_t)p0 * d;
			const uint32_t* a_src = asg + p0;
			uint64_t il = tid / d;
			uint32_t j = tid % d;
			const uint32_t step_i = UPD_THREADS / d, step_j = UPD_THREADS % d;
			for (uint64_t le = tid; le < count; le += UPD_THREADS) {
				const uint32_t a = a_src[il];
				const float v = src[le];
				if (a < k) {
					atomicAdd(&my[(size_t)a * stride + j], v);
					if (j == 0) atomicAdd(&mycnt[a], 1u);
				} else {
					bad = true;
				}
				il += step_i;
				j += step_j;
				if (j >= d) { j -= d; ++il; }
			}
		}
	}
	if (bad) atomicOr(&ctl->status, (uint32_t)STATUS_BAD_INDEX);

	if (SHARED) {
		__syncthreads();
		const uint32_t kd = k * d;
		uint32_t c = tid / d, j = tid % d;
		const uint32_t step_c = UPD_THREADS / d, step_j = UPD_THREADS % d;
		for (uint32_t e = tid; e < kd; e += UPD_THREADS) {
			float s = 0.0f;
			for (uint32_t r = 0; r < replicas; ++r) s += sacc[rep_floats * r + (size_t)c * dstride + j];
			if (s != 0.0f) atomicAdd(&acc[e], s);
			c += step_c;
			j += step_j;
			if (j >= d) { j -= d; ++c; }
		}
		for (uint32_t cc = tid; cc < k; cc += UPD_THREADS) {
			uint32_t t = 0;
			for (uint32_t r = 0; r < replicas; ++r) t += scnt[(size_t)k * r + cc];
			if (t) atomicAdd(&counts[cc], t);
		}
	}
}


// Row-wise variant: one warp adds one point's 32-dimension slice to its cluster's row with a
// single coalesced reduction (32 lanes = 32 consecutive floats = one 128-byte line, which the L2
// atomic unit takes in one operation).  For SoA points a 32x32 tile is transposed through
// shared memory first so that the loads stay coalesced too.  Best when k*dim is large enough
// that the rows rarely collide; the per-cluster sizes go to global integer atomics.
constexpr int ROWS_THREADS = 256;


// VEC: dim is a multiple of 4 and the buffers are 16-byte aligned, so that 8 lanes cover a
// 32-dimension slice with one 128-bit vector reduction each and a warp handles 4 points per
// instruction.
template<bool SOA, bool VEC>
__global__ void __launch_bounds__(ROWS_THREADS) update_rows_kernel(const float* __restrict__ pts,
	const uint32_t* __restrict__ asg, float* __restrict__ acc, uint32_t* __restrict__ counts,
	uint64_t n, uint32_t k, uint32_t d, uint32_t replicas, size_t rep_stride, Control* __restrict__ ctl)
{
	// blocks spread over `replicas` copies of the accumulators so that fewer reductions meet on a line
	acc += (blockIdx.x % replicas) * rep_stride;
	counts += (blockIdx.x % replicas) * rep_stride;
	// every warp works on its own group of 32 points, with a private transpose tile
	__shared__ float tiles[ROWS_THREADS / 32][32][33];
	const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
	constexpr uint32_t WARPS = ROWS_THREADS / 32;
	float (*tile)[33] = tiles[warp];
	const uint64_t groups = (n + 31) / 32;
	bool bad = false;
	for (uint64_t grp = (uint64_t)blockIdx.x * WARPS + warp; grp < groups; grp += (uint64_t)gridDim.x * WARPS) {
		const uint64_t p0 = grp * 32;
		const uint64_t pmine = p0 + lane;
		uint32_t amine = pmine < n ? asg[pmine] : 0xffffffffu;      // lane i holds the cluster of point p0+i
		if (pmine < n && amine >= k) { bad = true; amine = 0xffffffffu; }
		if (amine != 0xffffffffu) atomicAdd(&counts[amine], 1u);
		for (uint32_t c0 = 0; c0 < d; c0 += 32) {
			if (SOA) {
				// 32 independent coalesced loads per lane (dimension-major), then transpose
				float v[32];
				#pragma unroll
				for (uint32_t dl = 0; dl < 32; ++dl)
					v[dl] = (c0 + dl < d && pmine < n) ? pts[(size_t)(c0 + dl) * n + pmine] : 0.0f;
				__syncwarp();
				#pragma unroll
				for (uint32_t dl = 0; dl < 32; ++dl) tile[dl][lane] = v[dl];
				__syncwarp();
				if (VEC) {
					const uint32_t sub = lane >> 3, q4 = (lane & 7u) * 4;     // point within a group of 4, first of 4 dims
					#pragma unroll
					for (uint32_t it = 0; it < 8; ++it) {
						const uint32_t pl = it * 4 + sub;
						const uint32_t a = __shfl_sync(0xffffffffu, amine, pl);
						if (a != 0xffffffffu && c0 + q4 < d)
							red_add_v4(&acc[(size_t)a * d + c0 + q4], tile[q4 + 0][pl], tile[q4 + 1][pl], tile[q4 + 2][pl], tile[q4 + 3][pl]);
					}
				} else {
					#pragma unroll 8
					for (uint32_t pl = 0; pl < 32; ++pl) {
						const uint32_t a = __shfl_sync(0xffffffffu, amine, pl);
						if (a != 0xffffffffu && c0 + lane < d) atomicAdd(&acc[(size_t)a * d + c0 + lane], tile[lane][pl]);
					}
				}
			} else if (VEC) {
				const uint32_t sub = lane >> 3, q4 = (lane & 7u) * 4;
				#pragma unroll
				for (uint32_t it = 0; it < 8; ++it) {
					const uint32_t pl = it * 4 + sub;
					const uint32_t a = __shfl_sync(0xffffffffu, amine, pl);
					if (a != 0xffffffffu && c0 + q4 < d) {
						const float4 v = *reinterpret_cast<const float4*>(&pts[(size_t)(p0 + pl) * d + c0 + q4]);
						red_add_v4(&acc[(size_t)a * d + c0 + q4], v.x, v.y, v.z, v.w);
					}
				}
			} else {
				#pragma unroll 8
				for (uint32_t pl = 0; pl < 32; ++pl) {
					const uint32_t a = __shfl_sync(0xffffffffu, amine, pl);
					if (a != 0xffffffffu && c0 + lane < d)
						atomicAdd(&acc[(size_t)a * d + c0 + lane], pts[(size_t)(p0 + pl) * d + c0 + lane]);
				}
			}
		}
	}
	if (bad) atomicOr(&ctl->status, (uint32_t)STATUS_BAD_INDEX);
}

// ------------------------------------------------------------------------------------------
// update for few clusters: block-local counting sort, then one reduction per (cluster, chunk)
// ------------------------------------------------------------------------------------------
//
// With few clusters every global or shared-memory reduction of the row-wise kernels lands on
// one of a few hundred hot rows, and the memory system serialises them.  Here a block takes a
// chunk of SORT_CHUNK consecutive points and sorts their positions by cluster in shared memory
// (histogram, prefix sum, scatter).  Groups of `dg` lanes (one lane per dimension) then walk
// equal shares of the sorted order, adding rows into a register while the cluster stays the
// same and sending one row of reductions when it changes.  The number of reductions drops by
// about the number of points per cluster and chunk (8 for 256 clusters), and the sums reach the
// accumulators pre-added in a fixed small tree, which also keeps the rounding error down.

constexpr uint32_t SORT_THREADS = 256;
constexpr uint32_t SORT_CHUNK = 2048;
constexpr uint32_t SORT_PER_THREAD = SORT_CHUNK / SORT_THREADS;
constexpr uint32_t SORT_MAX_K = 1024;
constexpr uint32_t SORT_SCAN = (SORT_MAX_K + 1 + SORT_THREADS - 1) / SORT_THREADS;   // buckets per thread in the scan

bool update_sorted_supported(const Shape& s) { return s.k <= SORT_MAX_K; }

template<bool SOA, int VW>
__global__ void __launch_bounds__(SORT_THREADS) update_sorted_kernel(const float* __restrict__ pts,
	const uint32_t* __restrict__ asg, float* __restrict__ acc, uint32_t* __restrict__ counts,
	uint64_t n, uint32_t k, uint32_t d, uint32_t dg, uint32_t replicas, size_t rep_stride, Control* __restrict__ ctl)
{
	acc += (blockIdx.x % replicas) * rep_stride;
	counts += (blockIdx.x % replicas) * rep_stride;
	__shared__ uint32_t start[SORT_MAX_K + 2];      // after the scan: first sorted position of each cluster (k = trash bucket)
	__shared__ __align__(8) uint16_t order[SORT_CHUNK];     // sorted position -> point within the chunk
	__shared__ __align__(8) uint16_t cl_sorted[SORT_CHUNK]; // sorted position -> cluster
	__shared__ uint32_t warp_sums[SORT_THREADS / 32];
	const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
	const uint32_t nsub = 32 / dg;                  // lane groups per warp
	const uint32_t dl = lane % dg, sub = lane / dg;
	const uint32_t walker = warp * nsub + sub, walkers = (SORT_THREADS / 32) * nsub;
	const uint64_t chunks = (n + SORT_CHUNK - 1) / SORT_CHUNK;
	bool bad = false;
	for (uint64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
		const uint64_t base = chunk * SORT_CHUNK;
		const uint32_t cnt = (uint32_t)(n - base < SORT_CHUNK ? n - base : SORT_CHUNK);
		__syncthreads();                            // the previous chunk's walkers are done
		for (uint32_t c = tid; c <= k; c += SORT_THREADS) start[c] = 0;
		__syncthreads();
		uint32_t mine[SORT_PER_THREAD], rank[SORT_PER_THREAD];
		#pragma unroll
		for (uint32_t r = 0; r < SORT_PER_THREAD; ++r) {
			const uint32_t i = r * SORT_THREADS + tid;
			uint32_t c = k;                         // trash bucket: beyond the chunk or a bad index
			if (i < cnt) {
				c = asg[base + i];
				if (c >= k) { bad = true; c = k; }
			}
			mine[r] = c;
			rank[r] = atomicAdd(&start[c], 1u);     // the histogram pass also hands out the place within the bucket
		}
		__syncthreads();
		// exclusive prefix sum over k + 1 buckets: a few buckets per thread, warp scan, warp totals
		{
			uint32_t v[SORT_SCAN], local = 0;
			#pragma unroll
			for (uint32_t r = 0; r < SORT_SCAN; ++r) { const uint32_t c = tid * SORT_SCAN + r; v[r] = c <= k ? start[c] : 0; local += v[r]; }
			uint32_t incl = local;
			#pragma unroll
			for (uint32_t off = 1; off < 32; off <<= 1) { const uint32_t o = __shfl_up_sync(0xffffffffu, incl, off); if (lane >= off) incl += o; }
			if (lane == 31) warp_sums[warp] = incl;
			__syncthreads();
			uint32_t before = 0;
			for (uint32_t w = 0; w < warp; ++w) before += warp_sums[w];
			uint32_t run = before + incl - local;
			#pragma unroll
			for (uint32_t r = 0; r < SORT_SCAN; ++r) {
				const uint32_t c = tid * SORT_SCAN + r;
				if (c <= k) start[c] = run;
				run += v[r];
			}
		}
		__syncthreads();
		// sizes straight from the histogram; scatter of the positions
		for (uint32_t c = tid; c < k; c += SORT_THREADS) {
			const uint32_t sz = start[c + 1] - start[c];
			if (sz) atomicAdd(&counts[c], sz);
		}
		#pragma unroll
		for (uint32_t r = 0; r < SORT_PER_THREAD; ++r) {
			const uint32_t pos = start[mine[r]] + rank[r];
			order[pos] = (uint16_t)(r * SORT_THREADS + tid);
			cl_sorted[pos] = (uint16_t)mine[r];
		}
		__syncthreads();
		// every lane group walks an equal, 4-aligned share of the sorted order (the trash bucket is last)
		const uint32_t total = start[k];
		const uint32_t share = ((total + walkers - 1) / walkers + 3) & ~3u;
		const uint32_t w0 = min(walker * share, total), w1 = min(w0 + share, total);
		if (VW == 4) {
			// row-major points, dim a multiple of 4: a lane holds four dimensions
			const float4* rows = reinterpret_cast<const float4*>(pts + (size_t)base * d);
			const uint32_t d4 = d >> 2;
			for (uint32_t c0 = 0; c0 < d4; c0 += dg) {
				const uint32_t j4 = c0 + dl;
				const bool jok = j4 < d4;
				float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
				uint32_t cur = w0 < w1 ? cl_sorted[w0] : 0u;
				for (uint32_t sp = w0; sp < w1; sp += 4) {
					const uint2 o2 = *reinterpret_cast<const uint2*>(&order[sp]);
					const uint2 c2 = *reinterpret_cast<const uint2*>(&cl_sorted[sp]);
					const uint32_t oi[4] = {o2.x & 0xffffu, o2.x >> 16, o2.y & 0xffffu, o2.y >> 16};
					const uint32_t ci[4] = {c2.x & 0xffffu, c2.x >> 16, c2.y & 0xffffu, c2.y >> 16};
					float4 x[4];
					#pragma unroll
					for (uint32_t u = 0; u < 4; ++u) {
						x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
						if (sp + u < w1 && jok) x[u] = rows[oi[u] * d4 + j4];
					}
					#pragma unroll
					for (uint32_t u = 0; u < 4; ++u) {
						if (sp + u < w1) {
							if (ci[u] != cur) {
								if (jok) red_add_v4(&acc[(size_t)cur * d + j4 * 4], sum.x, sum.y, sum.z, sum.w);
								sum = make_float4(0.f, 0.f, 0.f, 0.f);
								cur = ci[u];
							}
							sum.x += x[u].x; sum.y += x[u].y; sum.z += x[u].z; sum.w += x[u].w;
						}
					}
				}
				if (w0 < w1 && jok) red_add_v4(&acc[(size_t)cur * d + j4 * 4], sum.x, sum.y, sum.z, sum.w);
			}
		} else if (VW == 2) {
			// row-major points, even dim: a lane holds two dimensions
			const float2* rows = reinterpret_cast<const float2*>(pts + (size_t)base * d);
			const uint32_t d2 = d >> 1;
			for (uint32_t c0 = 0; c0 < d2; c0 += dg) {
				const uint32_t j2 = c0 + dl;
				const bool jok = j2 < d2;
				float2 sum = make_float2(0.f, 0.f);
				uint32_t cur = w0 < w1 ? cl_sorted[w0] : 0u;
				for (uint32_t sp = w0; sp < w1; sp += 4) {
					const uint2 o2 = *reinterpret_cast<const uint2*>(&order[sp]);
					const uint2 c2 = *reinterpret_cast<const uint2*>(&cl_sorted[sp]);
					const uint32_t oi[4] = {o2.x & 0xffffu, o2.x >> 16, o2.y & 0xffffu, o2.y >> 16};
					const uint32_t ci[4] = {c2.x & 0xffffu, c2.x >> 16, c2.y & 0xffffu, c2.y >> 16};
					float2 x[4];
					#pragma unroll
					for (uint32_t u = 0; u < 4; ++u) {
						x[u] = make_float2(0.f, 0.f);
						if (sp + u < w1 && jok) x[u] = rows[oi[u] * d2 + j2];
					}
					#pragma unroll
					for (uint32_t u = 0; u < 4; ++u) {
						if (sp + u < w1) {
							if (ci[u] != cur) {
								if (jok) red_add_v2(&acc[(size_t)cur * d + j2 * 2], sum.x, sum.y);
								sum = make_float2(0.f, 0.f);
								cur = ci[u];
							}
							sum.x += x[u].x; sum.y += x[u].y;
						}
					}
				}
				if (w0 < w1 && jok) red_add_v2(&acc[(size_t)cur * d + j2 * 2], sum.x, sum.y);
			}
		} else {
			for (uint32_t c0 = 0; c0 < d; c0 += dg) {
				const uint32_t j = c0 + dl;
				const bool jok = j < d;
				// 32-bit offsets from the chunk's first point
				const float* col = SOA ? pts + (size_t)j * n + base : pts + (size_t)base * d + j;
				const uint32_t pstride = SOA ? 1u : d;
				float sum = 0.0f;
				uint32_t cur = w0 < w1 ? cl_sorted[w0] : 0u;
				for (uint32_t sp = w0; sp < w1; sp += 4) {
					// four sorted positions at a time: indices and clusters as one 8-byte load each
					const uint2 o2 = *reinterpret_cast<const uint2*>(&order[sp]);
					const uint2 c2 = *reinterpret_cast<const uint2*>(&cl_sorted[sp]);
					const uint32_t oi[4] = {o2.x & 0xffffu, o2.x >> 16, o2.y & 0xffffu, o2.y >> 16};
					const uint32_t ci[4] = {c2.x & 0xffffu, c2.x >> 16, c2.y & 0xffffu, c2.y >> 16};
					float x[4];
					#pragma unroll
					for (uint32_t u = 0; u < 4; ++u) {
						x[u] = 0.0f;
						if (sp + u < w1 && jok) x[u] = col[oi[u] * pstride];
					}
					#pragma unroll
					for (uint32_t u = 0; u < 4; ++u) {
						if (sp + u < w1) {
							if (ci[u] != cur) {
								if (jok) atomicAdd(&acc[(size_t)cur * d + j], sum);
								sum = 0.0f;
								cur = ci[u];
							}
							sum += x[u];
						}
					}
				}
				if (w0 < w1 && jok) atomicAdd(&acc[(size_t)cur * d + j], sum);
			}
		}
	}
	if (bad) atomicOr(&ctl->status, (uint32_t)STATUS_BAD_INDEX);
}

static size_t update_replica_bytes(const Shape& s)
{
	const uint32_t dstride = s.dim | 1u;
	return (size_t)s.k * (dstride + 1) * sizeof(float);
}

bool update_shared_fits(const Shape& s, int /*device*/)
{
	return update_replica_bytes(s) <= SMEM_LIMIT - 1024 && (uint64_t)s.k * s.dim < (1ull << 31);
}

void launch_update(const float* pts, const uint32_t* asg, float* acc, uint32_t* counts, uint32_t replicas, const Shape& s,
	int variant, Control* ctl, int sm_count, cudaStream_t stream)
{
	if (variant == BKM_UPDATE_SORTED) {
		// row-major points whose rows are whole 16- or 8-byte vectors: a lane holds four or two dimensions
		const uintptr_t align = reinterpret_cast<uintptr_t>(pts) | reinterpret_cast<uintptr_t>(acc);
		const int vw = s.soa ? 1 : (s.dim % 4 == 0 && (align & 15u) == 0 ? 4 : (s.dim % 2 == 0 && (align & 7u) == 0 ? 2 : 1));
		const uint32_t per_point = s.dim / (uint32_t)vw;
		uint32_t dg = vw == 1 ? 2 : 1;              // lanes per point: the power of two that covers a row, at most 32
		while (dg < 32 && dg < per_point) dg <<= 1;
		const uint64_t chunks = (s.n + SORT_CHUNK - 1) / SORT_CHUNK;
		const uint32_t grid = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(chunks, 1), (uint64_t)sm_count * 8);
		const size_t rep_stride = acc_replica_stride(s.k, s.dim);
		if (s.soa) update_sorted_kernel<true, 1><<<grid, SORT_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, dg, replicas, rep_stride, ctl);
		else if (vw == 4) update_sorted_kernel<false, 4><<<grid, SORT_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, dg, replicas, rep_stride, ctl);
		else if (vw == 2) update_sorted_kernel<false, 2><<<grid, SORT_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, dg, replicas, rep_stride, ctl);
		else update_sorted_kernel<false, 1><<<grid, SORT_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, dg, replicas, rep_stride, ctl);
		return;
	}
	if (variant == BKM_UPDATE_ROWS) {
		const uint64_t groups = (s.n + 31) / 32;
		const uint64_t blocks = (groups + ROWS_THREADS / 32 - 1) / (ROWS_THREADS / 32);
		const uint32_t grid = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(blocks, 1), (uint64_t)sm_count * 6);
		const size_t rep_stride = acc_replica_stride(s.k, s.dim);
		const bool vec = s.dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(pts) | reinterpret_cast<uintptr_t>(acc)) & 15u) == 0;
		if (s.soa && vec) update_rows_kernel<true, true><<<grid, ROWS_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, replicas, rep_stride, ctl);
		else if (s.soa) update_rows_kernel<true, false><<<grid, ROWS_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, replicas, rep_stride, ctl);
		else if (vec) update_rows_kernel<false, true><<<grid, ROWS_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, replicas, rep_stride, ctl);
		else update_rows_kernel<false, false><<<grid, ROWS_THREADS, 0, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, replicas, rep_stride, ctl);
		return;
	}
	const uint32_t dstride = s.dim | 1u;
	const bool shared = variant == BKM_UPDATE_SHARED;
	uint32_t smem_replicas = 1;
	size_t smem = 0;
	if (shared) {
		const size_t per = update_replica_bytes(s);
		// aim at two resident blocks per SM when one replica is small enough, and at most 4 replicas
		const size_t budget = per <= 100 * 1024 ? 100 * 1024 : SMEM_LIMIT - 1024;
		smem_replicas = (uint32_t)std::min<size_t>(4, std::max<size_t>(1, budget / per));
		smem = per * smem_replicas;
	}
	int per_sm = 1;
#define BKM_LAUNCH_UPD(SOA, SH) do { \
		auto kern = update_kernel<SOA, SH>; \
		if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
		cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, UPD_THREADS, smem); \
		if (per_sm < 1) per_sm = 1; \
		if (per_sm > 4) per_sm = 4; \
		uint64_t want = (s.n + 1023) / 1024; \
		uint32_t grid = (uint32_t)std::min<uint64_t>(std::max<uint64_t>(want, 1), (uint64_t)sm_count * per_sm); \
		kern<<<grid, UPD_THREADS, smem, stream>>>(pts, asg, acc, counts, s.n, s.k, s.dim, dstride, smem_replicas, ctl); \
	} while (0)
	if (s.soa) { if (shared) BKM_LAUNCH_UPD(true, true); else BKM_LAUNCH_UPD(true, false); }
	else       { if (shared) BKM_LAUNCH_UPD(false, true); else BKM_LAUNCH_UPD(false, false); }
#undef BKM_LAUNCH_UPD
}

} // namespace bkm
