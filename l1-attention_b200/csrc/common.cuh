// Shared helpers of libl1attn_b200: error plumbing, 16-byte vector types, sign transfer.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "l1attn_b200.h"

namespace l1b {

// Records the CUDA error for l1attn_last_cuda_error() and maps it to L1ATTN_ERR_CUDA.
int cuda_fail(cudaError_t e);

#define L1B_CUDA(call)                                  \
	do {                                            \
		cudaError_t e__ = (call);               \
		if (e__ != cudaSuccess)                 \
			return ::l1b::cuda_fail(e__);   \
	} while (0)

// After a kernel launch: pick up configuration errors without synchronising.
#define L1B_LAUNCH_CHECK() L1B_CUDA(cudaGetLastError())

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// 16-byte vector of T: float4 or double2.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
	using type = float4;
	static constexpr int N = 4;
};
template <> struct Vec16<double> {
	using type = double2;
	static constexpr int N = 2;
};

template <typename T, int N> struct alignas(sizeof(T) * N) Pack {
	T v[N];
};

// sign(d) * g with sign(0) = 0 (cuda/l1attn_cuda_kernel.cu:9-14 of the reference defines the
// same three-valued sign).  fp32: flip g's sign bit with d's, then drop exact ties.
__device__ __forceinline__ float sign_apply(float d, float g)
{
	float sg = __uint_as_float(__float_as_uint(g) ^ (__float_as_uint(d) & 0x80000000u));
	return d != 0.f ? sg : 0.f;
}
__device__ __forceinline__ double sign_apply(double d, double g)
{
	double sg = d > 0.0 ? g : -g;
	return d != 0.0 ? sg : 0.0;
}

__device__ __forceinline__ float absdiff(float a, float b) { return fabsf(a - b); }
__device__ __forceinline__ double absdiff(double a, double b) { return fabs(a - b); }

__device__ __forceinline__ float exp_t(float x) { return expf(x); }
__device__ __forceinline__ double exp_t(double x) { return exp(x); }

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem)
{
	unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Launchers implemented per file; all return an L1ATTN_* status and never synchronise.
int dense_fwd_launch(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads, int width,
		     int dtype, cudaStream_t st);
// fast paths: return 1 when they do not apply to the given shape / alignment / device
int dense_fwd_tma_launch(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads, int width,
			 int dtype, cudaStream_t st);
// tie_hdr: device tie header {count, overflow} or nullptr.  With a header whose overflow word is 0 every tile takes the
// compare form (the listed ties are repaired afterwards by dense_tiefix_launch); otherwise the flags decide.
// only_on_overflow: the kernel returns at once unless the header's overflow word is set (the single-visit kernel ran before it)
int dense_bwd_tma_launch(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, int bs, int n_tok,
			 int n_heads, int width, int dtype, const unsigned char *exact_flags, const int *tie_hdr,
			 int only_on_overflow, cudaStream_t st);
int dense_bwd_sv_launch(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, const int *tie_hdr,
			void *part, void *dq_part, int ns, int bs, int n_tok, int n_heads, int width, int dtype, cudaStream_t st);
// dk_sign: +1 after the two-pass kernel (a tie counted as -scale g in d_k), -1 after the single-visit kernel (+scale g)
int dense_tiefix_launch(const void *d_attn, void *d_q, void *d_k, const unsigned char *scratch, int bs, int n_tok,
			int n_heads, int width, int dk_sign, cudaStream_t st);
int dense_ties_launch(const float *q, const float *k, unsigned char *scratch, int bs, int n_tok, int n_heads, int width,
		      cudaStream_t st);
// scratch: dense_bwd_scratch_bytes() bytes of device memory, or nullptr (then every tile runs the exact loop)
int dense_bwd_launch(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, void *scratch, int bs,
		     int n_tok, int n_heads, int width, int dtype, cudaStream_t st);
size_t dense_bwd_scratch_bytes(int bs, int n_tok, int n_heads, int width, int dtype);
int dense_softmax_v_launch(const void *q, const void *k, const void *v, void *vo, void *lse, int bs, int n_tok, int n_heads,
			   int width, int v_width, int mode, int dtype, cudaStream_t st);
int dense_softmax_v_bwd_dx_launch(const void *q, const void *k, const void *v, const void *dvo, const void *lse,
				  const void *delta, void *dx, void *dv, int bs, int n_tok, int n_heads, int width, int v_width,
				  int dtype, cudaStream_t st);

// Layout of the sparse edge index (all int32, each array padded to 16 bytes):
//   slot_src [n_tok*dst_mxlen]  src token of slot (dst, r), or -1
//   csc_off  [n_tok+1]          start of every src token's list of incoming slots
//   csc_slot [cl]               slot ids (dst*dst_mxlen + r), grouped by src, in coo row order
//   cnt      [n_tok]            build-time counters
//   rank     [cl]               build-time per-row rank within its src group (-1: row skipped)
struct SparseIndex {
	int32_t *slot_src, *csc_off, *csc_slot, *cnt, *rank;
	size_t bytes;
};
SparseIndex sparse_index_view(void *base, int cl, int n_tok, int dst_mxlen);

} // namespace l1b
