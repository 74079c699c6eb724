// pybind module l1attn_sparse_cuda_drv:
//   forward(v, q, k, coo, dst_mxlen, use_softmax) -> [vo, attn]
//   backward(dvo, v, q, k, coo, attn, dst_mxlen, use_softmax) -> [d_v, d_q, d_k]
// as the reference driver (cuda/l1attn_sparse_cuda_drv.cpp:32-74), plus expand_coo(co).
#include "drv_sparse_common.h"

std::vector<torch::Tensor> l1attnSparse_forward(torch::Tensor v, torch::Tensor q, torch::Tensor k, torch::Tensor coo,
						int dst_mxlen, bool use_softmax)
{
	CHECK_INPUT(v);
	CHECK_INPUT(q);
	CHECK_INPUT(k);
	CHECK_INPUT(coo);
	return l1b_sparse_forward(v, torch::Tensor(), q, k, coo, dst_mxlen, use_softmax, false);
}

std::vector<torch::Tensor> l1attnSparse_backward(torch::Tensor dvo, torch::Tensor v, torch::Tensor q, torch::Tensor k,
						 torch::Tensor coo, torch::Tensor attn, int dst_mxlen, bool use_softmax)
{
	CHECK_INPUT(dvo);
	CHECK_INPUT(v);
	CHECK_INPUT(q);
	CHECK_INPUT(k);
	CHECK_INPUT(coo);
	CHECK_INPUT(attn);
	return l1b_sparse_backward(dvo, v, torch::Tensor(), q, k, coo, attn, dst_mxlen, use_softmax, false);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
	m.def("forward", &l1attnSparse_forward, "L1AttnSparse forward (CUDA, sm_100a)");
	m.def("backward", &l1attnSparse_backward, "L1AttnSparse backward (CUDA, sm_100a)");
	m.def("expand_coo", &l1b_expand_coo, "expandCoo on the GPU");
	m.def("clear_index_cache", &l1b_clear_index_cache, "drop the cached edge indexes of this module");
}
