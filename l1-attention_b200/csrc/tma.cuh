// TMA (cp.async.bulk.tensor) and mbarrier helpers for sm_100a, plus host-side tensor-map encoding.
//
// Rules kept here:
//  * loads only, never multicast, always from this GPU's own memory;
//  * the innermost coordinate of every copy is a multiple of 16 bytes (callers pass width
//    offsets that are multiples of the 64-byte stage row, and 0 for the head/row axes that are
//    innermost in their tensors);
//  * every wait is bounded: after FAST_POLLS failed polls the waiter goes on by the global nanosecond
//    timer for at most WAIT_LIMIT_NS, then records an error code in the device error word and gives
//    up, so a lost copy cannot hang the GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace l1b {

// Address (on the current device) of the sticky error word: 0 = no error; a kernel whose bounded
// wait ran out stores a non-zero code there.  Read and cleared by l1attn_device_status().
int *device_error_word();

constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull; // two seconds: orders of magnitude beyond any copy these kernels wait for

__device__ __forceinline__ uint64_t global_timer_ns()
{
	uint64_t t;
	asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
	return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init()
{
	asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
	asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
	asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar_addr, uint32_t parity)
{
	uint32_t ok;
	asm volatile("{\n\t.reg .pred p;\n\t"
		     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
		     "selp.u32 %0, 1, 0, p;\n\t}"
		     : "=r"(ok)
		     : "r"(bar_addr), "r"(parity)
		     : "memory");
	return ok != 0;
}

// Waits by the clock alone: true when the phase with the given parity has completed, false (and *err set) once
// limit_ns have passed without that.  *polls, when given, receives the number of failed polls.
static __device__ __noinline__ bool mbar_wait_timed(uint64_t *bar, uint32_t parity, int *err, uint64_t limit_ns, unsigned *polls = nullptr)
{
	const uint32_t a = smem_u32(bar);
	const uint64_t t0 = global_timer_ns();
	unsigned n = 0;
	bool ok = false;
	while (!(ok = mbar_try(a, parity)) && global_timer_ns() - t0 <= limit_ns)
		n++;
	if (polls)
		*polls = n;
	if (!ok)
		*err = 1;
	return ok;
}

// The wait of the hot loops.  Its first phase is a bare poll loop and nothing else: waiting warps sit on the critical
// path of a pipeline stage, and anything more in that loop (a clock read every n-th poll, a sleep, a suspend hint)
// measured up to 1.8x slower kernels.  FAST_POLLS failed polls take about a second (each try_wait
// suspends the thread for a hardware time slice, measured at 4 us by tests/test_dense_gpu.py); only then -- a copy is
// late by orders of magnitude -- the wait goes on in a separate, clocked loop for at most WAIT_LIMIT_NS more
// before it gives up.
constexpr uint32_t FAST_POLLS = 1u << 18;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err)
{
	const uint32_t a = smem_u32(bar);
	for (uint32_t i = 0; i < FAST_POLLS; i++)
		if (mbar_try(a, parity))
			return true;
	return mbar_wait_timed(bar, parity, err, WAIT_LIMIT_NS);
}

// The wait of a producer that runs stages ahead of its consumers: nobody waits for it to wake up, so it sleeps
// between polls instead of taking issue slots from the warps that share its scheduler (0.7 % on the dense
// forward; on the consumers' waits the same sleep, or a suspend-time hint on try_wait, changed nothing: their
// polls fill issue slots that would otherwise stay empty).
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t *bar, uint32_t parity, int *err)
{
	const uint32_t a = smem_u32(bar);
	for (uint32_t i = 0; i < FAST_POLLS; i++) {
		if (mbar_try(a, parity))
			return true;
		asm volatile("nanosleep.u32 256;");
	}
	return mbar_wait_timed(bar, parity, err, WAIT_LIMIT_NS);
}

// 4-D tiled load global -> shared, completion signalled on `bar` (no multicast)
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1, int c2, int c3)
{
	asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
		     :
		     : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
		     : "memory");
}

// 4-D tiled store shared -> global (bulk async-group completion).  Parts of the box outside the
// tensor are clipped by the hardware; coordinates must be non-negative and c0 a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, const void *src, int c0, int c1, int c2, int c3)
{
	asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
		     :
		     : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
		     : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until every committed bulk store has finished READING its shared-memory source
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// makes generic-proxy shared-memory writes visible to the async proxy (before a bulk store reads them)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// barrier among the first `n` threads' warps only (id 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_barrier(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// ---- host side -----------------------------------------------------------------------------

// Encodes a 4-D tiled tensor map.  dims/box are innermost-first; strides_bytes has 3 entries (dims 1..3).
// Returns false when the driver entry point is missing or the encode call is refused (the
// caller then uses the kernel that needs no tensor map).
bool encode_tmap_4d(CUtensorMap *out, CUtensorMapDataType dt, const void *base, const uint64_t dims[4],
		    const uint64_t strides_bytes[3], const uint32_t box[4], CUtensorMapSwizzle swz);

} // namespace l1b
