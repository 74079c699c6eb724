// pybind module l1attn_sparse_bidi_cuda_drv:
//   forward(vf, vb, q, k, coo, dst_mxlen, use_softmax) -> [vo, attn]
//   backward(dvo, vf, vb, q, k, coo, attn, dst_mxlen, use_softmax) -> [d_vf, d_vb, d_q, d_k]
// as the reference driver (cuda/l1attn_sparse_bidi_cuda_drv.cpp:34-80), plus expand_coo(co).
#include "drv_sparse_common.h"

std::vector<torch::Tensor> l1attnSparseBidi_forward(torch::Tensor vf, torch::Tensor vb, torch::Tensor q,
						    torch::Tensor k, torch::Tensor coo, int dst_mxlen, bool use_softmax)
{
	CHECK_INPUT(vf);
	CHECK_INPUT(vb);
	CHECK_INPUT(q);
	CHECK_INPUT(k);
	CHECK_INPUT(coo);
	return l1b_sparse_forward(vf, vb, q, k, coo, dst_mxlen, use_softmax, true);
}

std::vector<torch::Tensor> l1attnSparseBidi_backward(torch::Tensor dvo, torch::Tensor vf, torch::Tensor vb,
						     torch::Tensor q, torch::Tensor k, torch::Tensor coo,
						     torch::Tensor attn, int dst_mxlen, bool use_softmax)
{
	CHECK_INPUT(dvo);
	CHECK_INPUT(vf);
	CHECK_INPUT(vb);
	CHECK_INPUT(q);
	CHECK_INPUT(k);
	CHECK_INPUT(coo);
	CHECK_INPUT(attn);
	return l1b_sparse_backward(dvo, vf, vb, q, k, coo, attn, dst_mxlen, use_softmax, true);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
	m.def("forward", &l1attnSparseBidi_forward, "L1AttnSparseBidi forward (CUDA, sm_100a)");
	m.def("backward", &l1attnSparseBidi_backward, "L1AttnSparseBidi backward (CUDA, sm_100a)");
	m.def("expand_coo", &l1b_expand_coo, "expandCoo on the GPU");
	m.def("clear_index_cache", &l1b_clear_index_cache, "drop the cached edge indexes of this module");
}
