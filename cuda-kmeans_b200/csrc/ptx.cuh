// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk/tensor TMA copies, tcgen05 (TMEM
// allocation, MMA issue, commit, loads).  Every wait is bounded: after WAIT_LIMIT polls it
// gives up and reports failure so that the kernel can set a status bit and leave.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace bkm { namespace ptx {

// A wait gives up after this many nanoseconds (read from %globaltimer) - far beyond any
// legitimate wait in these kernels, short enough that a broken pipeline ends by itself.
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;
// How long one try_wait may keep the thread suspended before it returns to be polled again.
// A long slice keeps waiting threads from burning issue slots that the working warps need.
constexpr uint32_t WAIT_SLICE_NS = 20000u;

__device__ __forceinline__ uint64_t globaltimer_ns()
{
	uint64_t t;
	asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
	return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
	return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes mbarrier initialisation visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_mbar_init()
{
	asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
	asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
	uint32_t ok;
	asm volatile(
		"{\n"
		".reg .pred p;\n"
		"mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
		"selp.u32 %0, 1, 0, p;\n"
		"}\n"
		: "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(WAIT_SLICE_NS) : "memory");
	return ok != 0;
}

// Bounded wait.  Returns false if the phase did not complete within `limit_ns`.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = WAIT_LIMIT_NS)
{
	if (mbar_try_wait(bar, parity)) return true;
	const uint64_t t0 = globaltimer_ns();
	while (true) {
		if (mbar_try_wait(bar, parity)) return true;
		if (globaltimer_ns() - t0 > limit_ns) return false;
	}
}

// Up to `polls` rounds of (try_wait, sleep SLEEP_NS) as one six-instruction loop; true as soon as the phase is complete.
template<uint32_t SLEEP_NS>
__device__ __forceinline__ bool mbar_poll_round(uint64_t* bar, uint32_t parity, uint32_t polls)
{
	uint32_t ok;
	asm volatile(
		"{\n"
		".reg .pred done, more;\n"
		".reg .u32 left;\n"
		"mov.u32 left, %3;\n"
		"POLL_AGAIN:\n"
		"mbarrier.try_wait.parity.shared::cta.b64 done, [%1], %2, %4;\n"
		"@done bra POLL_END;\n"
		"nanosleep.u32 %5;\n"
		"sub.u32 left, left, 1;\n"
		"setp.ne.u32 more, left, 0;\n"
		"@more bra POLL_AGAIN;\n"
		"POLL_END:\n"
		"selp.u32 %0, 1, 0, done;\n"
		"}\n"
		: "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(polls), "r"(WAIT_SLICE_NS), "n"(SLEEP_NS) : "memory");
	return ok != 0;
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
		:: "r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// 2-D tiled TMA load: box at (x = innermost coordinate, y) of the tensor map -> shared.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int32_t x, int32_t y, uint64_t* bar)
{
	asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
		:: "r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void prefetch_tmap(const void* tmap)
{
	asm volatile("prefetch.tensormap [%0];" :: "l"(tmap) : "memory");
}

// ---- tcgen05 ----

// Allocates `cols` TMEM columns (power of two, 32..512); the base address lands in *slot (shared).
// Executed by one full warp.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols)
{
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(slot)), "r"(cols) : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before()
{
	asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after()
{
	asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one()
{
	uint32_t pred;
	asm volatile(
		"{\n"
		".reg .pred p;\n"
		"elect.sync _|p, 0xffffffff;\n"
		"selp.u32 %0, 1, 0, p;\n"
		"}\n"
		: "=r"(pred));
	return pred != 0;
}

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::tf32, issued by one thread.
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
		"{\n"
		".reg .pred p;\n"
		"setp.ne.b32 p, %4, 0;\n"
		"tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
		"}\n"
		:: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// The same with the two 64-bit shared-memory descriptors given as 32-bit halves: within one
// operand tile only the low half (the address field) changes from instruction to instruction, so
// the issuing thread spends one 32-bit add per operand and MMA instead of 64-bit arithmetic.
__device__ __forceinline__ void mma_tf32_halves(uint32_t d_tmem, uint32_t a_lo32, uint32_t a_hi32, uint32_t b_lo32, uint32_t b_hi32, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
		"{\n"
		".reg .pred p;\n"
		".reg .b64 da, db;\n"
		"mov.b64 da, {%1, %2};\n"
		"mov.b64 db, {%3, %4};\n"
		"setp.ne.b32 p, %6, 0;\n"
		"tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n"
		"}\n"
		:: "r"(d_tmem), "r"(a_lo32), "r"(a_hi32), "r"(b_lo32), "r"(b_hi32), "r"(idesc), "r"(accumulate) : "memory");
}

// Arrives on `bar` once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar)
{
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit: thread t of the warp gets row (lane base + t),
// v[c] = column (col base + c).  taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
	asm volatile(
		"tcgen05.ld.sync.aligned.32x32b.x32.b32 "
		"{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
		"%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
		: "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
		  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
		  "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
		  "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
		: "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
	asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- CTA pairs (thread-block cluster of two, tcgen05 cta_group::2) ----

__device__ __forceinline__ uint32_t cluster_ctarank()
{
	uint32_t r;
	asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
	return r;
}

// Barrier over all threads of the cluster; orders shared-memory writes before it with reads after it.
__device__ __forceinline__ void cluster_sync()
{
	asm volatile("barrier.cluster.arrive.release.aligned;\n"
		"barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank)
{
	uint32_t r;
	asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
	return r;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
	asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v)
{
	asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(cluster_addr), "r"(v) : "memory");
}

// 2-D tiled TMA load into this CTA's shared memory whose completion bytes are counted on a
// barrier of the pair's first CTA: clearing bit 24 of a shared address turns it into that CTA's.
__device__ __forceinline__ uint32_t leader_cta_addr(uint32_t smem_addr) { return smem_addr & 0xFEFFFFFFu; }

__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, int32_t x, int32_t y, uint32_t leader_bar_addr)
{
	asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
		:: "r"(smem_u32(smem_dst)), "l"(tmap), "r"(leader_bar_addr), "r"(x), "r"(y) : "memory");
}

// TMEM allocation for a CTA pair: the same warp of both CTAs executes it.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t cols)
{
	asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(slot)), "r"(cols) : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair()
{
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols)
{
	asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}

// One MMA over both CTAs of the pair (M = 256: 128 accumulator rows in each CTA's tensor memory;
// each CTA's shared memory holds its 128 rows of A and its half of the N rows of B at the
// descriptor's address).  Issued by one thread of the pair's first CTA.
__device__ __forceinline__ void mma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
	asm volatile(
		"{\n"
		".reg .pred p;\n"
		"setp.ne.b32 p, %4, 0;\n"
		"tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
		"}\n"
		:: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// The same with the two 64-bit shared-memory descriptors given as 32-bit halves.  Within one
// operand tile only the low half (the address field) changes from instruction to instruction and
// the high half is a constant of the layout, which leaves the issuing thread one 32-bit add per
// operand and MMA instead of 64-bit descriptor arithmetic.  ACC = accumulate onto the destination.
template<bool ACC>
__device__ __forceinline__ void mma_tf32_pair_halves(uint32_t d_tmem, uint32_t a_lo32, uint32_t a_hi32, uint32_t b_lo32, uint32_t b_hi32, uint32_t idesc)
{
	asm volatile(
		"{\n"
		".reg .pred p;\n"
		".reg .b64 da, db;\n"
		"mov.b64 da, {%1, %2};\n"
		"mov.b64 db, {%3, %4};\n"
		"setp.ne.b32 p, %6, 0;\n"
		"tcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %5, p;\n"
		"}\n"
		:: "r"(d_tmem), "r"(a_lo32), "r"(a_hi32), "r"(b_lo32), "r"(b_hi32), "r"(idesc), "n"(ACC ? 1 : 0) : "memory");
}

// Arrives on the barrier at shared::cluster address `bar_addr` (of either CTA of the pair) once
// all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_addr)
{
	asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar_addr) : "memory");
}

}} // namespace bkm::ptx
