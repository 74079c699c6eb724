// Shared body of the l1attn_sparse_cuda_drv and l1attn_sparse_bidi_cuda_drv pybind modules.
//
// The reference's sparse kernels take only (coo, dst_mxlen) per call.  The kernels behind the C ABI
// want an edge index derived from coo (slot table + per-source lists); it is built on first use
// and cached per coo tensor, keyed on (storage pointer, version counter, sizes), so a graph that
// is reused across layers and steps is indexed once.  The cache keeps the coo tensor alive, so a
// freed-and-reused pointer cannot alias a stale entry.  A write that bypasses the version counter
// (coo.data[...] = ..., a raw-pointer kernel) is NOT seen: do not edit coo in place that way, or call
// clear_index_cache() (bound in both sparse modules) afterwards.  The cache holds at most 16 graphs.
#pragma once
#include <climits>
#include <cstdint>
#include <list>
#include <mutex>
#include "drv_common.h"

struct L1bIndexEntry {
	torch::Tensor coo, index;
	uint32_t version;
	int n_tok, dst_mxlen;
};

struct L1bIndexCache {
	std::mutex mu;
	std::list<L1bIndexEntry> entries; // most recent first
};
inline L1bIndexCache &l1b_index_cache()
{
	static L1bIndexCache c;
	return c;
}

// Drops every cached edge index (and the coo tensors they keep alive).
inline void l1b_clear_index_cache()
{
	L1bIndexCache &c = l1b_index_cache();
	std::lock_guard<std::mutex> lock(c.mu);
	c.entries.clear();
}

inline torch::Tensor l1b_index_for(const torch::Tensor &coo, int n_tok, int dst_mxlen)
{
	L1bIndexCache &holder = l1b_index_cache();
	std::list<L1bIndexEntry> &cache = holder.entries;
	const size_t max_entries = 16;
	std::lock_guard<std::mutex> lock(holder.mu);
	const uint32_t ver = coo._version();
	for (auto it = cache.begin(); it != cache.end(); ++it) {
		if (it->coo.data_ptr() == coo.data_ptr() && it->version == ver && it->coo.sizes() == coo.sizes() &&
		    it->n_tok == n_tok && it->dst_mxlen == dst_mxlen && it->coo.device() == coo.device()) {
			cache.splice(cache.begin(), cache, it);
			return cache.front().index;
		}
	}
	const int cl = coo.size(0);
	const size_t bytes = l1attn_sparse_index_bytes(cl, n_tok, dst_mxlen);
	auto opts = torch::TensorOptions().dtype(torch::kInt32).device(coo.device());
	auto index = torch::empty({(long)((bytes + 3) / 4)}, opts);
	auto status = torch::zeros({1}, opts);
	l1b_status(l1attn_sparse_build_index(coo.data_ptr<int>(), cl, n_tok, dst_mxlen, index.data_ptr(),
					     status.data_ptr<int>(), l1b_stream()),
		   "l1attn_sparse_build_index");
	// Out-of-range rows are undefined behaviour in the reference; here they are reported.
	const int st = status.item<int>();
	l1b_status(st, "coo");
	cache.push_front({coo, index, ver, n_tok, dst_mxlen});
	if (cache.size() > max_entries)
		cache.pop_back();
	return index;
}

inline void l1b_check_coo(const torch::Tensor &coo, const torch::Tensor &q)
{
	TORCH_CHECK(coo.scalar_type() == torch::kInt32, "coo must be int32 (the output of expandCoo)");
	TORCH_CHECK(coo.dim() == 2 && coo.size(1) == 4, "coo must be [n_edges, 4] (the output of expandCoo)");
	TORCH_CHECK(coo.device() == q.device(), "coo and q must be on the same device");
}

// vb is an undefined tensor for the one-directional operator
inline std::vector<torch::Tensor> l1b_sparse_forward(torch::Tensor v, torch::Tensor vb, torch::Tensor q,
						     torch::Tensor k, torch::Tensor coo, int dst_mxlen,
						     bool use_softmax, bool bidi)
{
	TORCH_CHECK(q.dim() == 4 && v.dim() == 4, "v, q, k must be [batch, n_tokens, heads, width]");
	l1b_same(q, k, "q", "k");
	l1b_same(q, v, "q", "v", false);
	TORCH_CHECK(v.size(0) == q.size(0) && v.size(1) == q.size(1) && v.size(2) == q.size(2),
		    "v must match q in batch, tokens and heads");
	if (bidi)
		l1b_same(v, vb, "vf", "vb");
	l1b_check_coo(coo, q);
	TORCH_CHECK(dst_mxlen >= 0, "dst_mxlen must be >= 0");
	const int dt = l1b_dtype(q, "l1attnSparse forward", true);
	const c10::cuda::CUDAGuard guard(q.device());
	const int bs = q.size(0), n = q.size(1), h = q.size(2), w = q.size(3), wv = v.size(3), cl = coo.size(0);
	auto index = l1b_index_for(coo, n, dst_mxlen);
	auto opts = q.options().requires_grad(false);
	auto attn = torch::empty({bs, n, dst_mxlen, h}, opts);
	auto vo = torch::empty({bs, n, h, wv}, opts);
	l1b_status(l1attn_sparse_fwd(v.data_ptr(), bidi ? vb.data_ptr() : nullptr, q.data_ptr(), k.data_ptr(),
				     index.data_ptr(), vo.data_ptr(), attn.data_ptr(), bs, n, h, w, wv, cl, dst_mxlen,
				     use_softmax, bidi, dt, l1b_stream()),
		   "l1attn_sparse_fwd");
	return {vo, attn};
}

inline std::vector<torch::Tensor> l1b_sparse_backward(torch::Tensor dvo, torch::Tensor v, torch::Tensor vb,
						      torch::Tensor q, torch::Tensor k, torch::Tensor coo,
						      torch::Tensor attn, int dst_mxlen, bool use_softmax, bool bidi)
{
	TORCH_CHECK(q.dim() == 4 && v.dim() == 4, "v, q, k must be [batch, n_tokens, heads, width]");
	l1b_same(q, k, "q", "k");
	l1b_same(v, dvo, "v", "dvo");
	l1b_same(q, v, "q", "v", false);
	l1b_same(q, attn, "q", "attn", false);
	if (bidi)
		l1b_same(v, vb, "vf", "vb");
	l1b_check_coo(coo, q);
	const int dt = l1b_dtype(q, "l1attnSparse backward");
	const int bs = q.size(0), n = q.size(1), h = q.size(2), w = q.size(3), wv = v.size(3), cl = coo.size(0);
	TORCH_CHECK(attn.dim() == 4 && attn.size(0) == bs && attn.size(1) == n && attn.size(2) == dst_mxlen &&
			    attn.size(3) == h,
		    "attn must be [batch, n_tokens, dst_mxlen, heads] as returned by forward");
	const c10::cuda::CUDAGuard guard(q.device());
	auto index = l1b_index_for(coo, n, dst_mxlen);
	auto d_v = torch::empty_like(v), d_q = torch::empty_like(q), d_k = torch::empty_like(k);
	torch::Tensor d_vb;
	if (bidi)
		d_vb = torch::empty_like(v);
	auto scratch = torch::empty_like(attn);
	l1b_status(l1attn_sparse_bwd(dvo.data_ptr(), v.data_ptr(), bidi ? vb.data_ptr() : nullptr, q.data_ptr(),
				     k.data_ptr(), index.data_ptr(), attn.data_ptr(), d_v.data_ptr(),
				     bidi ? d_vb.data_ptr() : nullptr, d_q.data_ptr(), d_k.data_ptr(), scratch.data_ptr(),
				     bs, n, h, w, wv, cl, dst_mxlen, use_softmax, bidi, dt, l1b_stream()),
		   "l1attn_sparse_bwd");
	if (bidi)
		return {d_v, d_vb, d_q, d_k};
	return {d_v, d_q, d_k};
}

// expandCoo on the GPU: co [cl,2] integer tensor (any integer dtype, CPU or CUDA) ->
// (coo int32 [cl,4] on co's device, dst_mxlen, src_mxlen); cuda/l1attn_sparse_cuda.py:58-101.
inline std::tuple<torch::Tensor, int, int> l1b_expand_coo(torch::Tensor co)
{
	TORCH_CHECK(co.dim() == 2 && co.size(1) >= 2, "co must be [n_edges, 2] rows of (dst, src)");
	TORCH_CHECK(at::isIntegralType(co.scalar_type(), false), "co must hold integers");
	const auto home = co.device();
	TORCH_CHECK(torch::cuda::is_available(), "expandCoo runs on the GPU and no CUDA device is available");
	auto dev = home.is_cuda() ? home : torch::Device(torch::kCUDA, c10::cuda::current_device());
	const c10::cuda::CUDAGuard guard(dev);
	auto cog = co.slice(1, 0, 2).to(dev, torch::kInt64).contiguous();
	const int cl = cog.size(0);
	auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(dev);
	auto coo = torch::zeros({cl, 4}, i32);
	auto mx = torch::ones({2}, i32);
	long long lo = 0, nkeys = 0;
	torch::Tensor counters;
	void *cnt = nullptr;
	if (cl > 0) {
		auto mm = torch::empty({2}, torch::TensorOptions().dtype(torch::kInt64).device(dev));
		l1b_status(l1attn_i64_minmax(cog.data_ptr<int64_t>(), 2LL * cl, mm.data_ptr<int64_t>(), l1b_stream()),
			   "l1attn_i64_minmax");
		auto mmh = mm.cpu();
		lo = mmh[0].item<int64_t>();
		const long long hi = mmh[1].item<int64_t>();
		// the expanded list is int32 (as the reference's is); the rank counters take memory proportional to hi - lo
		TORCH_CHECK(lo >= INT32_MIN && hi <= INT32_MAX, "expandCoo: token ids must fit in int32, got [", lo, ", ", hi, "]");
		nkeys = hi - lo + 1;
		const size_t nb = l1attn_expand_coo_scratch_bytes(nkeys);
		if (nb) {
			counters = torch::empty({(long)(nb / 4)}, i32);
			cnt = counters.data_ptr();
		}
	}
	l1b_status(l1attn_expand_coo(cl ? cog.data_ptr<int64_t>() : nullptr, cl, cl ? coo.data_ptr<int>() : nullptr,
				     mx.data_ptr<int>(), lo, nkeys, cnt, l1b_stream()),
		   "l1attn_expand_coo");
	auto mxh = mx.cpu();
	return {coo.to(home), mxh[0].item<int>(), mxh[1].item<int>()};
}
