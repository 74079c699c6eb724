// C ABI glue: argument checks of the dense entry points, error reporting, and the host-buffer
// entry points (copy in, run, copy out) with their per-device arena.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>
#include "common.cuh"

namespace l1b {

static thread_local int g_last_cuda = 0;

int cuda_fail(cudaError_t e)
{
	g_last_cuda = int(e);
	return e == cudaErrorMemoryAllocation ? L1ATTN_ERR_NOMEM : L1ATTN_ERR_CUDA;
}

namespace {

int check_dense(const void *const *ptrs, int nptr, int bs, int n_tok, int n_heads, int width, int dtype)
{
	if (bs < 0 || n_tok < 0 || n_heads < 0 || width < 1)
		return L1ATTN_ERR_ARG;
	if (dtype != L1ATTN_F32 && dtype != L1ATTN_F64)
		return L1ATTN_ERR_ARG;
	const bool empty = bs == 0 || n_tok == 0 || n_heads == 0;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	for (int i = 0; i < nptr; i++) {
		if (!ptrs[i] && !empty)
			return L1ATTN_ERR_ARG;
		if (ptrs[i] && !aligned(ptrs[i], es))
			return L1ATTN_ERR_ALIGN;
	}
	return L1ATTN_OK;
}

// Grow-only device arena of the *_host entry points, one per device.
struct Arena {
	void *base = nullptr;
	size_t cap = 0, used = 0;
};
std::mutex g_mu;
std::vector<Arena> g_arena;

Arena *arena_for_current(int *rc)
{
	int dev = 0;
	cudaError_t e = cudaGetDevice(&dev);
	if (e != cudaSuccess) {
		*rc = cuda_fail(e);
		return nullptr;
	}
	if (size_t(dev) >= g_arena.size())
		g_arena.resize(dev + 1);
	return &g_arena[dev];
}

int arena_reserve(Arena *a, size_t bytes)
{
	a->used = 0;
	if (bytes <= a->cap)
		return L1ATTN_OK;
	if (a->base) {
		L1B_CUDA(cudaDeviceSynchronize());
		L1B_CUDA(cudaFree(a->base));
		a->base = nullptr;
		a->cap = 0;
	}
	L1B_CUDA(cudaMalloc(&a->base, bytes));
	a->cap = bytes;
	return L1ATTN_OK;
}

size_t pad256(size_t n) { return (n + 255) / 256 * 256; }

void *arena_take(Arena *a, size_t bytes)
{
	void *p = static_cast<unsigned char *>(a->base) + a->used;
	a->used += pad256(bytes ? bytes : 1);
	return p;
}

} // namespace
} // namespace l1b

using namespace l1b;

extern "C" int l1attn_version(void) { return 100; }

extern "C" const char *l1attn_strerror(int code)
{
	switch (code) {
	case L1ATTN_OK: return "ok";
	case L1ATTN_ERR_ARG: return "invalid argument (NULL pointer, negative size or unknown dtype)";
	case L1ATTN_ERR_SHAPE: return "shape exceeds what the kernels can index";
	case L1ATTN_ERR_CUDA: return "CUDA runtime or launch failure (see l1attn_last_cuda_error)";
	case L1ATTN_ERR_INDEX: return "coo row outside [0,n_tok) x [0,n_tok) x [0,dst_mxlen)";
	case L1ATTN_ERR_NOMEM: return "out of device memory";
	case L1ATTN_ERR_ALIGN: return "tensor pointer not aligned to its element size";
	case L1ATTN_ERR_SCRATCH: return "the problem needs more scratch memory than the library's built-in static buffer holds";
	case L1ATTN_ERR_TIMEOUT: return "a kernel gave up a bounded wait on an asynchronous copy";
	default: return "unknown l1attn error code";
	}
}

extern "C" int l1attn_last_cuda_error(void) { return g_last_cuda; }

extern "C" int l1attn_dense_fwd(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads, int width,
				 int dtype, void *stream)
{
	const void *ptrs[] = {q, k, attn};
	int rc = check_dense(ptrs, 3, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	return dense_fwd_launch(q, k, attn, bs, n_tok, n_heads, width, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int l1attn_dense_softmax_v_fwd(const void *q, const void *k, const void *v, void *vo, void *lse, int bs, int n_tok,
					   int n_heads, int width, int v_width, int mode, int dtype, void *stream)
{
	const void *ptrs[] = {q, k, v, vo};
	int rc = check_dense(ptrs, 4, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	if (v_width < 1 || mode < L1ATTN_SV_SOFTMAX || mode > L1ATTN_SV_EXP)
		return L1ATTN_ERR_ARG;
	if (lse && !aligned(lse, dtype == L1ATTN_F64 ? 8 : 4))
		return L1ATTN_ERR_ALIGN;
	return dense_softmax_v_launch(q, k, v, vo, lse, bs, n_tok, n_heads, width, v_width, mode, dtype,
				      static_cast<cudaStream_t>(stream));
}

extern "C" int l1attn_dense_softmax_v_bwd_dx(const void *q, const void *k, const void *v, const void *dvo, const void *lse,
					      const void *delta, void *dx, void *dv, int bs, int n_tok, int n_heads, int width,
					      int v_width, int dtype, void *stream)
{
	const void *ptrs[] = {q, k, v, dvo, lse, delta, dx, dv};
	int rc = check_dense(ptrs, 8, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	if (v_width < 1)
		return L1ATTN_ERR_ARG;
	return dense_softmax_v_bwd_dx_launch(q, k, v, dvo, lse, delta, dx, dv, bs, n_tok, n_heads, width, v_width, dtype,
					     static_cast<cudaStream_t>(stream));
}

extern "C" size_t l1attn_dense_bwd_scratch_bytes(int bs, int n_tok, int n_heads, int width, int dtype)
{
	return dense_bwd_scratch_bytes(bs, n_tok, n_heads, width, dtype);
}

extern "C" int l1attn_dense_bwd(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, void *scratch,
				 int bs, int n_tok, int n_heads, int width, int dtype, void *stream)
{
	const void *ptrs[] = {d_attn, q, k, d_q, d_k};
	int rc = check_dense(ptrs, 5, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	return dense_bwd_launch(d_attn, q, k, d_q, d_k, scratch, bs, n_tok, n_heads, width, dtype,
				static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- host-buffer entry points

#define H2D(dst, src, n) L1B_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, 0))
#define D2H(dst, src, n) L1B_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, 0))

extern "C" int l1attn_dense_fwd_host(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads,
				      int width, int dtype)
{
	const void *ptrs[] = {q, k, attn};
	int rc = check_dense(ptrs, 3, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(bs) * n_tok * n_heads * width * es, na = size_t(bs) * n_tok * n_tok * n_heads * es;
	if (na == 0)
		return L1ATTN_OK;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	if ((rc = arena_reserve(ar, 2 * pad256(nqk) + pad256(na))))
		return rc;
	void *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk), *da = arena_take(ar, na);
	H2D(dq, q, nqk);
	H2D(dk, k, nqk);
	if ((rc = dense_fwd_launch(dq, dk, da, bs, n_tok, n_heads, width, dtype, 0)))
		return rc;
	D2H(attn, da, na);
	L1B_CUDA(cudaStreamSynchronize(0));
	return L1ATTN_OK;
}

extern "C" int l1attn_dense_softmax_v_fwd_host(const void *q, const void *k, const void *v, void *vo, int bs, int n_tok,
						int n_heads, int width, int v_width, int mode, int dtype)
{
	const void *ptrs[] = {q, k, v, vo};
	int rc = check_dense(ptrs, 4, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	if (v_width < 1 || mode < L1ATTN_SV_SOFTMAX || mode > L1ATTN_SV_EXP)
		return L1ATTN_ERR_ARG;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(bs) * n_tok * n_heads * width * es, nv = size_t(bs) * n_tok * n_heads * v_width * es;
	if (nv == 0)
		return L1ATTN_OK;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	if ((rc = arena_reserve(ar, 2 * pad256(nqk) + 2 * pad256(nv))))
		return rc;
	void *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk), *dv = arena_take(ar, nv), *dvo = arena_take(ar, nv);
	H2D(dq, q, nqk);
	H2D(dk, k, nqk);
	H2D(dv, v, nv);
	if ((rc = dense_softmax_v_launch(dq, dk, dv, dvo, nullptr, bs, n_tok, n_heads, width, v_width, mode, dtype, 0)))
		return rc;
	D2H(vo, dvo, nv);
	L1B_CUDA(cudaStreamSynchronize(0));
	return L1ATTN_OK;
}

extern "C" int l1attn_dense_bwd_host(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, int bs,
				      int n_tok, int n_heads, int width, int dtype)
{
	const void *ptrs[] = {d_attn, q, k, d_q, d_k};
	int rc = check_dense(ptrs, 5, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(bs) * n_tok * n_heads * width * es, na = size_t(bs) * n_tok * n_tok * n_heads * es;
	if (na == 0)
		return L1ATTN_OK;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	const size_t nsc = dense_bwd_scratch_bytes(bs, n_tok, n_heads, width, dtype);
	if ((rc = arena_reserve(ar, 4 * pad256(nqk) + pad256(na) + pad256(nsc))))
		return rc;
	void *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk), *dg = arena_take(ar, na);
	void *ddq = arena_take(ar, nqk), *ddk = arena_take(ar, nqk), *dsc = arena_take(ar, nsc);
	H2D(dq, q, nqk);
	H2D(dk, k, nqk);
	H2D(dg, d_attn, na);
	if ((rc = dense_bwd_launch(dg, dq, dk, ddq, ddk, dsc, bs, n_tok, n_heads, width, dtype, 0)))
		return rc;
	D2H(d_q, ddq, nqk);
	D2H(d_k, ddk, nqk);
	L1B_CUDA(cudaStreamSynchronize(0));
	return L1ATTN_OK;
}

extern "C" int l1attn_sparse_fwd_host(const void *v, const void *vb, const void *q, const void *k,
				       const int32_t *coo, void *vo, void *attn, int bs, int n_tok, int n_heads,
				       int width, int v_width, int cl, int dst_mxlen, int use_softmax, int bidi, int dtype)
{
	if (bs < 0 || n_tok < 0 || n_heads < 0 || width < 1 || v_width < 1 || cl < 0 || dst_mxlen < 0 ||
	    (dtype != L1ATTN_F32 && dtype != L1ATTN_F64))
		return L1ATTN_ERR_ARG;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(bs) * n_tok * n_heads * width * es, nv = size_t(bs) * n_tok * n_heads * v_width * es;
	const size_t na = size_t(bs) * n_tok * dst_mxlen * n_heads * es, nc = size_t(cl) * 16;
	if (nv == 0)
		return L1ATTN_OK;
	if (!v || !q || !k || !vo || (na && !attn) || (cl && !coo) || (bidi && !vb))
		return L1ATTN_ERR_ARG;
	const size_t nix = l1attn_sparse_index_bytes(cl, n_tok, dst_mxlen);
	int rc;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	if ((rc = arena_reserve(ar, 2 * pad256(nqk) + 3 * pad256(nv) + pad256(na) + pad256(nc) + pad256(nix) + 256)))
		return rc;
	void *dv = arena_take(ar, nv), *dvb = arena_take(ar, nv), *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk);
	void *dvo = arena_take(ar, nv), *da = arena_take(ar, na), *dc = arena_take(ar, nc), *dix = arena_take(ar, nix);
	int32_t *dstat = static_cast<int32_t *>(arena_take(ar, 4));
	H2D(dv, v, nv);
	if (bidi)
		H2D(dvb, vb, nv);
	H2D(dq, q, nqk);
	H2D(dk, k, nqk);
	if (cl)
		H2D(dc, coo, nc);
	if ((rc = l1attn_sparse_build_index(static_cast<int32_t *>(dc), cl, n_tok, dst_mxlen, dix, dstat, 0)))
		return rc;
	if ((rc = l1attn_sparse_fwd(dv, dvb, dq, dk, dix, dvo, da, bs, n_tok, n_heads, width, v_width, cl, dst_mxlen,
				    use_softmax, bidi, dtype, 0)))
		return rc;
	int32_t stat = 0;
	D2H(vo, dvo, nv);
	if (na)
		D2H(attn, da, na);
	D2H(&stat, dstat, 4);
	L1B_CUDA(cudaStreamSynchronize(0));
	return stat;
}

extern "C" int l1attn_sparse_bwd_host(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
				       const int32_t *coo, const void *attn, void *d_v, void *d_vb, void *d_q,
				       void *d_k, int bs, int n_tok, int n_heads, int width, int v_width, int cl,
				       int dst_mxlen, int use_softmax, int bidi, int dtype)
{
	if (bs < 0 || n_tok < 0 || n_heads < 0 || width < 1 || v_width < 1 || cl < 0 || dst_mxlen < 0 ||
	    (dtype != L1ATTN_F32 && dtype != L1ATTN_F64))
		return L1ATTN_ERR_ARG;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(bs) * n_tok * n_heads * width * es, nv = size_t(bs) * n_tok * n_heads * v_width * es;
	const size_t na = size_t(bs) * n_tok * dst_mxlen * n_heads * es, nc = size_t(cl) * 16;
	if (nv == 0)
		return L1ATTN_OK;
	if (!dvo || !v || !q || !k || !d_v || !d_q || !d_k || (na && !attn) || (cl && !coo) || (bidi && (!vb || !d_vb)))
		return L1ATTN_ERR_ARG;
	const size_t nix = l1attn_sparse_index_bytes(cl, n_tok, dst_mxlen);
	int rc;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	if ((rc = arena_reserve(ar, 4 * pad256(nqk) + 5 * pad256(nv) + 2 * pad256(na) + pad256(nc) + pad256(nix) + 256)))
		return rc;
	void *ddvo = arena_take(ar, nv), *dv = arena_take(ar, nv), *dvb = arena_take(ar, nv);
	void *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk), *da = arena_take(ar, na);
	void *gdv = arena_take(ar, nv), *gdvb = arena_take(ar, nv), *gdq = arena_take(ar, nqk), *gdk = arena_take(ar, nqk);
	void *dx = arena_take(ar, na), *dc = arena_take(ar, nc), *dix = arena_take(ar, nix);
	int32_t *dstat = static_cast<int32_t *>(arena_take(ar, 4));
	H2D(ddvo, dvo, nv);
	H2D(dv, v, nv);
	if (bidi)
		H2D(dvb, vb, nv);
	H2D(dq, q, nqk);
	H2D(dk, k, nqk);
	if (na)
		H2D(da, attn, na);
	if (cl)
		H2D(dc, coo, nc);
	if ((rc = l1attn_sparse_build_index(static_cast<int32_t *>(dc), cl, n_tok, dst_mxlen, dix, dstat, 0)))
		return rc;
	if ((rc = l1attn_sparse_bwd(ddvo, dv, dvb, dq, dk, dix, da, gdv, gdvb, gdq, gdk, dx, bs, n_tok, n_heads, width,
				    v_width, cl, dst_mxlen, use_softmax, bidi, dtype, 0)))
		return rc;
	int32_t stat = 0;
	D2H(d_v, gdv, nv);
	if (bidi)
		D2H(d_vb, gdvb, nv);
	D2H(d_q, gdq, nqk);
	D2H(d_k, gdk, nqk);
	D2H(&stat, dstat, 4);
	L1B_CUDA(cudaStreamSynchronize(0));
	return stat;
}

extern "C" int l1attn_expand_coo_host(const int64_t *co, int cl, int32_t *coo, int *dst_mxlen, int *src_mxlen)
{
	if (cl < 0 || !dst_mxlen || !src_mxlen || (cl > 0 && (!co || !coo)))
		return L1ATTN_ERR_ARG;
	int rc;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	const size_t nco = size_t(cl) * 16, ncoo = size_t(cl) * 16;
	// first pass: key range (needs a round trip to size the counters)
	if ((rc = arena_reserve(ar, pad256(nco) + pad256(ncoo) + 512)))
		return rc;
	void *dco = arena_take(ar, nco), *dcoo = arena_take(ar, ncoo);
	int64_t *dmm = static_cast<int64_t *>(arena_take(ar, 16));
	int32_t *dmx = static_cast<int32_t *>(arena_take(ar, 8));
	long long lo = 0, n_keys = 0;
	if (cl) {
		H2D(dco, co, nco);
		if ((rc = l1attn_i64_minmax(static_cast<int64_t *>(dco), 2LL * cl, dmm, 0)))
			return rc;
		int64_t mm[2];
		D2H(mm, dmm, 16);
		L1B_CUDA(cudaStreamSynchronize(0));
		lo = mm[0];
		n_keys = mm[1] - mm[0] + 1;
	}
	void *cnt = nullptr;
	const size_t ncnt = l1attn_expand_coo_scratch_bytes(n_keys);
	if (ncnt)
		L1B_CUDA(cudaMalloc(&cnt, ncnt)); // rare: more than 51200 distinct token ids
	rc = l1attn_expand_coo(static_cast<int64_t *>(dco), cl, static_cast<int32_t *>(dcoo), dmx, lo, n_keys, cnt, 0);
	int32_t mx[2] = {1, 1};
	if (!rc) {
		cudaError_t e = cudaSuccess;
		if (cl)
			e = cudaMemcpyAsync(coo, dcoo, ncoo, cudaMemcpyDeviceToHost, 0);
		if (e == cudaSuccess)
			e = cudaMemcpyAsync(mx, dmx, 8, cudaMemcpyDeviceToHost, 0);
		if (e == cudaSuccess)
			e = cudaStreamSynchronize(0);
		if (e != cudaSuccess)
			rc = cuda_fail(e);
	}
	if (cnt)
		cudaFree(cnt);
	*dst_mxlen = mx[0];
	*src_mxlen = mx[1];
	return rc;
}

extern "C" int l1attn_host_release(void)
{
	int rc = L1ATTN_OK;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	if (ar->base) {
		L1B_CUDA(cudaDeviceSynchronize());
		L1B_CUDA(cudaFree(ar->base));
	}
	*ar = Arena();
	return L1ATTN_OK;
}
