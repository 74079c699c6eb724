// Host side of the TMA helpers: tensor-map encoding through the driver entry point (no link
// against libcuda), and the sticky device error word.
#include <mutex>
#include "common.cuh"
#include "tma.cuh"

namespace l1b {

namespace {
__device__ int l1b_kernel_error = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
				  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
				  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_once;

void resolve()
{
	void *fn = nullptr;
	cudaDriverEntryPointQueryResult qres;
	if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
	    qres == cudaDriverEntryPointSuccess)
		g_encode = reinterpret_cast<EncodeTiledFn>(fn);
	else
		(void)cudaGetLastError();
}
} // namespace

bool encode_tmap_4d(CUtensorMap *out, CUtensorMapDataType dt, const void *base, const uint64_t dims[4],
		    const uint64_t strides_bytes[3], const uint32_t box[4], CUtensorMapSwizzle swz)
{
	std::call_once(g_once, resolve);
	if (!g_encode)
		return false;
	cuuint64_t d[4], s[3];
	cuuint32_t b[4], es[4] = {1, 1, 1, 1};
	for (int i = 0; i < 4; i++) {
		d[i] = dims[i];
		b[i] = box[i];
	}
	for (int i = 0; i < 3; i++)
		s[i] = strides_bytes[i];
	const CUresult r = g_encode(out, dt, 4, const_cast<void *>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
				    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
	return r == CUDA_SUCCESS;
}

int *device_error_word()
{
	int *p = nullptr;
	if (cudaGetSymbolAddress(reinterpret_cast<void **>(&p), l1b_kernel_error) != cudaSuccess) {
		(void)cudaGetLastError();
		return nullptr;
	}
	return p;
}

} // namespace l1b

// Reads (and clears) the sticky error word set by a kernel whose bounded wait ran out.
extern "C" int l1attn_device_status(void)
{
	int v = 0;
	int *p = l1b::device_error_word();
	if (!p)
		return L1ATTN_ERR_CUDA;
	L1B_CUDA(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
	if (v) {
		L1B_CUDA(cudaMemset(p, 0, sizeof(int)));
		return L1ATTN_ERR_TIMEOUT;
	}
	return L1ATTN_OK;
}

// Copies the error word to *host_word on `stream` without waiting and without clearing it.  With host_word in
// pinned memory a caller can look at the word before its next launch and call l1attn_device_status() only when
// it is set.
extern "C" int l1attn_device_status_async(int *host_word, void *stream)
{
	int *p = l1b::device_error_word();
	if (!p || !host_word)
		return L1ATTN_ERR_ARG;
	L1B_CUDA(cudaMemcpyAsync(host_word, p, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
	return L1ATTN_OK;
}

namespace l1b {
namespace {
// One warp waits on a barrier that nothing ever completes, with a short limit: the wait runs out, the error word
// is set and the kernel returns.  Nothing faults and nothing hangs; it exists so that the give-up path of
// mbar_wait and the error word's set / read / clear cycle can be exercised.
__global__ void wait_timeout_probe_kernel(unsigned long long limit_ns, int *err, int *returned)
{ // returned[0]: 1 = the wait gave up, 2 = it succeeded (cannot happen); returned[1]: failed polls of thread 0
	__shared__ __align__(8) uint64_t bar;
	if (threadIdx.x == 0) {
		mbar_init(&bar, 1);
		mbar_fence_init();
	}
	__syncthreads();
	unsigned polls = 0;
	const bool ok = mbar_wait_timed(&bar, 0, err, limit_ns, &polls);
	if (threadIdx.x == 0) {
		returned[0] = ok ? 2 : 1;
		returned[1] = int(polls);
	}
}
} // namespace
} // namespace l1b

extern "C" int l1attn_test_wait_timeout(int limit_us, int *returned_dev, void *stream)
{
	if (limit_us < 1 || limit_us > 100000 || !returned_dev)
		return L1ATTN_ERR_ARG;
	int *err = l1b::device_error_word();
	if (!err)
		return L1ATTN_ERR_CUDA;
	l1b::wait_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(1000ull * limit_us, err, returned_dev);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}
