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
