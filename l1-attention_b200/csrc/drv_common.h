// Shared pieces of the three pybind drivers: input checks with the reference's messages
// (cuda/l1attn_cuda_drv.cpp:38-40), status -> exception, dtype code, current stream.
#pragma once
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <vector>
#include "l1attn_b200.h"

#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_INPUT(x) \
	CHECK_CUDA(x);  \
	CHECK_CONTIGUOUS(x)

// allow16: the sparse forward also takes float16 / bfloat16 storage (the reference dispatches Half
// there, cuda/l1attn_sparse_cuda_kernel.cu:405); every other operator is float32 / float64 only
inline int l1b_dtype(const torch::Tensor &t, const char *what, bool allow16 = false)
{
	if (t.scalar_type() == torch::kFloat32)
		return L1ATTN_F32;
	if (t.scalar_type() == torch::kFloat64)
		return L1ATTN_F64;
	if (allow16 && t.scalar_type() == torch::kFloat16)
		return L1ATTN_F16;
	if (allow16 && t.scalar_type() == torch::kBFloat16)
		return L1ATTN_BF16;
	TORCH_CHECK(false, what, ": expected float32 or float64 tensors", allow16 ? " (or float16 / bfloat16)" : "", ", got ",
		    t.scalar_type());
	return -1;
}

inline void l1b_same(const torch::Tensor &a, const torch::Tensor &b, const char *an, const char *bn, bool shape = true)
{
	TORCH_CHECK(a.scalar_type() == b.scalar_type(), an, " and ", bn, " must have the same dtype");
	TORCH_CHECK(a.device() == b.device(), an, " and ", bn, " must be on the same device");
	if (shape)
		TORCH_CHECK(a.sizes() == b.sizes(), an, " and ", bn, " must have the same shape");
}

inline void l1b_status(int rc, const char *fn)
{
	if (rc == L1ATTN_OK)
		return;
	if (rc == L1ATTN_ERR_CUDA || rc == L1ATTN_ERR_NOMEM)
		TORCH_CHECK(false, fn, ": ", l1attn_strerror(rc), " [",
			    cudaGetErrorString(static_cast<cudaError_t>(l1attn_last_cuda_error())), "]");
	TORCH_CHECK(false, fn, ": ", l1attn_strerror(rc));
}

inline void *l1b_stream() { return static_cast<void *>(at::cuda::getCurrentCUDAStream().stream()); }

// A kernel of the library that gives up a bounded wait sets a sticky word on the device and returns; its outputs
// are then garbage.  The drivers never synchronise, so they learn of it one call late: after every launch the
// word is copied, on the same stream, to a pinned host word (l1b_poll_status); the next driver call looks at that
// word first (l1b_check_pending) and raises if it is set.  A caller that needs the answer at once can call
// l1attn_device_status() through the C ABI, which synchronises.
inline int *l1b_status_word()
{
	static int *word = [] {
		int *p = nullptr;
		if (cudaHostAlloc(reinterpret_cast<void **>(&p), 64, cudaHostAllocDefault) != cudaSuccess) {
			(void)cudaGetLastError();
			return static_cast<int *>(nullptr);
		}
		*p = 0;
		return p;
	}();
	return word;
}

inline void l1b_check_pending(const char *fn)
{
	int *w = l1b_status_word();
	if (w && *reinterpret_cast<volatile int *>(w) != 0) {
		*w = 0;
		(void)l1attn_device_status(); // synchronises and clears the device word
		TORCH_CHECK(false, fn, ": an earlier kernel of this library gave up a bounded wait on an asynchronous copy; "
				       "the results of the calls made since the previous successful call are invalid");
	}
}

inline void l1b_poll_status()
{
	int *w = l1b_status_word();
	if (w)
		(void)l1attn_device_status_async(w, l1b_stream());
}
