// pybind module l1attn_cuda_drv: forward(q, k) -> [attn], backward(d_attn, q, k) -> [d_q, d_k].
// Same names, argument order and return lists as the reference driver
// (cuda/l1attn_cuda_drv.cpp:42-109); all arithmetic happens in libl1attn_b200.so behind the C ABI.
// Differences, all supersets: works on the tensor's own device and the current stream (the
// reference launches on the legacy default stream), needs no [b,h,t,w] copies, and checks that
// q and k agree in shape/dtype (the reference reads every size from q).
#include "drv_common.h"

std::vector<torch::Tensor> l1attn_forward(torch::Tensor q, torch::Tensor k)
{
	l1b_check_pending("l1attn forward");
	CHECK_INPUT(q);
	CHECK_INPUT(k);
	TORCH_CHECK(q.dim() == 4, "q must be [batch, n_tokens, heads, width]");
	l1b_same(q, k, "q", "k");
	const int dt = l1b_dtype(q, "l1attn forward");
	const c10::cuda::CUDAGuard guard(q.device());
	const int bs = q.size(0), n = q.size(1), h = q.size(2), w = q.size(3);
	auto attn = torch::empty({bs, n, n, h}, q.options().requires_grad(false));
	l1b_status(l1attn_dense_fwd(q.data_ptr(), k.data_ptr(), attn.data_ptr(), bs, n, h, w, dt, l1b_stream()),
		   "l1attn_dense_fwd");
	l1b_poll_status();
	return {attn};
}

std::vector<torch::Tensor> l1attn_backward(torch::Tensor d_attn, torch::Tensor q, torch::Tensor k)
{
	l1b_check_pending("l1attn backward");
	CHECK_INPUT(d_attn);
	CHECK_INPUT(q);
	CHECK_INPUT(k);
	TORCH_CHECK(q.dim() == 4, "q must be [batch, n_tokens, heads, width]");
	l1b_same(q, k, "q", "k");
	l1b_same(q, d_attn, "q", "d_attn", false);
	const int dt = l1b_dtype(q, "l1attn backward");
	const int bs = q.size(0), n = q.size(1), h = q.size(2), w = q.size(3);
	TORCH_CHECK(d_attn.dim() == 4 && d_attn.size(0) == bs && d_attn.size(1) == n && d_attn.size(2) == n &&
			    d_attn.size(3) == h,
		    "d_attn must be [batch, n_tokens, n_tokens, heads]");
	const c10::cuda::CUDAGuard guard(q.device());
	auto d_q = torch::empty_like(q), d_k = torch::empty_like(k);
	auto scratch = torch::empty({(long)l1attn_dense_bwd_scratch_bytes(bs, n, h, w, dt)},
				    torch::TensorOptions().dtype(torch::kUInt8).device(q.device()));
	l1b_status(l1attn_dense_bwd(d_attn.data_ptr(), q.data_ptr(), k.data_ptr(), d_q.data_ptr(), d_k.data_ptr(),
				    scratch.data_ptr(), bs, n, h, w, dt, l1b_stream()),
		   "l1attn_dense_bwd");
	l1b_poll_status();
	return {d_q, d_k};
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
	m.def("forward", &l1attn_forward, "L1Attn forward (CUDA, sm_100a)");
	m.def("backward", &l1attn_backward, "L1Attn backward (CUDA, sm_100a)");
}
