// C ABI glue: argument checks of the dense entry points, error reporting, and the host-buffer
// entry points (copy in, run, copy out) with their per-device arena.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
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

// Per-device state of the *_host entry points: a grow-only device arena, one stream per PCIe direction, three
// compute streams and a small pinned block for values read back asynchronously.
// Every batch item of every call is a chain copy in -> kernels -> copy out across those streams (events in
// between): ALL copies in go through one stream and ALL copies out through another, each in the order of the
// calls, so both directions of the link stay busy at once -- also across calls: the inputs of an independent
// backward cross while the scores of the preceding forward leave (measured on this PCIe 5 x16 host: 54 GB/s in
// alone, 50 GB/s out alone, 90 GB/s with both; with the copies on the items' own streams the directions took
// turns and a [16,1024,16,64] forward + backward took 42 ms instead of 29 ms).
// Every call takes fresh slices of the arena (bump allocation), so calls enqueued one after the other without
// a synchronisation in between never share device buffers; l1attn_host_sync() waits for all of them and makes
// the whole arena available again.
constexpr int NPIPE = 3; // compute streams one call rotates its batch items over
constexpr int NSTAT = 64;
struct Arena {
	void *base = nullptr;
	size_t cap = 0, used = 0;
	cudaStream_t st[NPIPE] = {};          // kernels
	cudaStream_t s_in = nullptr, s_out = nullptr; // host -> device, device -> host
	std::vector<cudaEvent_t> evs;         // pool, handed out in order, all free again after a sync
	size_t nev = 0;
	int32_t *stat = nullptr; // pinned, NSTAT words
	int nstat = 0;
	bool ready = false;
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
	Arena *a = &g_arena[dev];
	if (!a->ready) {
		for (int i = 0; i < NPIPE && e == cudaSuccess; i++)
			e = cudaStreamCreateWithFlags(&a->st[i], cudaStreamNonBlocking);
		if (e == cudaSuccess)
			e = cudaStreamCreateWithFlags(&a->s_in, cudaStreamNonBlocking);
		if (e == cudaSuccess)
			e = cudaStreamCreateWithFlags(&a->s_out, cudaStreamNonBlocking);
		if (e == cudaSuccess)
			e = cudaHostAlloc(reinterpret_cast<void **>(&a->stat), NSTAT * sizeof(int32_t), cudaHostAllocDefault);
		if (e != cudaSuccess) {
			*rc = cuda_fail(e);
			return nullptr;
		}
		a->ready = true;
	}
	return a;
}

// `to` will not start what is enqueued on it from here on before everything enqueued on `from` so far has finished
int stream_after(Arena *a, cudaStream_t to, cudaStream_t from)
{
	if (a->nev == a->evs.size()) {
		cudaEvent_t ev;
		L1B_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
		a->evs.push_back(ev);
	}
	cudaEvent_t ev = a->evs[a->nev++];
	L1B_CUDA(cudaEventRecord(ev, from));
	L1B_CUDA(cudaStreamWaitEvent(to, ev, 0));
	return L1ATTN_OK;
}

// Waits for everything the *_host calls have enqueued on this device; returns the first deferred status
// (an out-of-range coo row found by an index build) and makes the arena's memory available again.
int arena_sync(Arena *a)
{
	L1B_CUDA(cudaStreamSynchronize(a->s_in));
	for (int i = 0; i < NPIPE; i++)
		L1B_CUDA(cudaStreamSynchronize(a->st[i]));
	L1B_CUDA(cudaStreamSynchronize(a->s_out));
	a->nev = 0;
	int rc = L1ATTN_OK;
	for (int i = 0; i < a->nstat; i++)
		if (a->stat[i] != 0 && rc == L1ATTN_OK)
			rc = a->stat[i];
	a->nstat = 0;
	a->used = 0;
	return rc;
}

size_t pad256(size_t n) { return (n + 255) / 256 * 256; }

// Makes `bytes` more bytes available.  When the arena has to grow, or has no room left for a deferred status
// word, everything in flight is waited for first (earlier asynchronous calls then simply finish early);
// *deferred receives their status.  It grows to what the calls enqueued since the last synchronisation need
// TOGETHER, so that the same sequence of calls fits next time without a wait in the middle (a forward and a
// backward enqueued back to back would otherwise take turns on the link instead of sharing it).
int arena_reserve(Arena *a, size_t bytes, int *deferred)
{
	*deferred = L1ATTN_OK;
	const size_t need = a->used + bytes;
	if (need <= a->cap && a->nstat < NSTAT)
		return L1ATTN_OK;
	*deferred = arena_sync(a);
	if (*deferred == L1ATTN_ERR_CUDA)
		return *deferred;
	if (need <= a->cap)
		return L1ATTN_OK;
	if (a->base) {
		L1B_CUDA(cudaFree(a->base));
		a->base = nullptr;
		a->cap = 0;
	}
	cudaError_t e = cudaMalloc(&a->base, need);
	if (e != cudaSuccess && need > bytes) { // not enough memory for the whole sequence: room for this call alone
		(void)cudaGetLastError();
		e = cudaMalloc(&a->base, bytes);
		if (e == cudaSuccess)
			a->cap = bytes;
	} else if (e == cudaSuccess) {
		a->cap = need;
	}
	if (e != cudaSuccess)
		return cuda_fail(e);
	return L1ATTN_OK;
}

void *arena_take(Arena *a, size_t bytes)
{
	void *p = static_cast<unsigned char *>(a->base) + a->used;
	a->used += pad256(bytes ? bytes : 1);
	return p;
}

inline const void *off(const void *p, size_t bytes) { return static_cast<const unsigned char *>(p) + bytes; }
inline void *off(void *p, size_t bytes) { return static_cast<unsigned char *>(p) + bytes; }

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
//
// One batch item at a time: its inputs go in on the copy-in stream, its kernels run on one of the three compute
// streams (in rotation) once they have arrived, its results leave on the copy-out stream once the kernels are done.
// While item b computes, item b+1's inputs cross PCIe in one direction and item b-1's results in the other.
// The *_async forms return once everything is enqueued; the plain forms add l1attn_host_sync().

#define H2D(dst, src, n, st) L1B_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, st))
#define D2H(dst, src, n, st) L1B_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, st))
#define L1B_TRY(call)                \
	do {                         \
		const int rc_ = (call); \
		if (rc_)             \
			return rc_;  \
	} while (0)

extern "C" int l1attn_host_sync(void)
{
	int rc = L1ATTN_OK;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	return arena_sync(ar);
}

// Batch items per chain of the dense host entry points: copies of ~128 MB use the link better than smaller ones, but
// a call should still be at least eight chains long so that the pipeline fills.
static int host_group(int bs, size_t bytes_per_item)
{
	if (const char *e = getenv("L1ATTN_HOST_GROUP")) // experiments: fixed group size
		return atoi(e) > 0 ? atoi(e) : 1;
	int g = 1;
	while (g < 8 && size_t(2 * g) * bytes_per_item <= (size_t(160) << 20) && bs / (2 * g) >= 8)
		g *= 2;
	return g;
}

// keeps the first error of an asynchronous call and of the deferred statuses it had to collect on the way
static int first_error(int a, int b) { return a != L1ATTN_OK ? a : b; }

extern "C" int l1attn_dense_fwd_host_async(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads,
					    int width, int dtype)
{
	const void *ptrs[] = {q, k, attn};
	int rc = check_dense(ptrs, 3, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(n_tok) * n_heads * width * es, na = size_t(n_tok) * n_tok * n_heads * es; // per batch item
	if (na == 0 || bs == 0)
		return L1ATTN_OK;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	int deferred;
	if ((rc = arena_reserve(ar, size_t(bs) * (2 * pad256(nqk) + pad256(na)), &deferred)))
		return rc;
	const int G = host_group(bs, na);
	for (int b = 0, it = 0; b < bs; b += G, it++) {
		const int g = bs - b < G ? bs - b : G; // batch items of this chain
		cudaStream_t st = ar->st[it % NPIPE];
		void *dq = arena_take(ar, g * nqk), *dk = arena_take(ar, g * nqk), *da = arena_take(ar, g * na);
		H2D(dq, off(q, b * nqk), g * nqk, ar->s_in);
		H2D(dk, off(k, b * nqk), g * nqk, ar->s_in);
		L1B_TRY(stream_after(ar, st, ar->s_in));
		if ((rc = dense_fwd_launch(dq, dk, da, g, n_tok, n_heads, width, dtype, st)))
			return rc;
		L1B_TRY(stream_after(ar, ar->s_out, st));
		D2H(off(attn, b * na), da, g * na, ar->s_out);
	}
	return deferred;
}

extern "C" int l1attn_dense_fwd_host(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads,
				      int width, int dtype)
{
	const int rc = l1attn_dense_fwd_host_async(q, k, attn, bs, n_tok, n_heads, width, dtype);
	return first_error(rc, l1attn_host_sync());
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
	const size_t nqk = size_t(n_tok) * n_heads * width * es, nv = size_t(n_tok) * n_heads * v_width * es;
	if (nv == 0 || bs == 0)
		return L1ATTN_OK;
	int deferred;
	{
		std::lock_guard<std::mutex> lock(g_mu);
		Arena *ar = arena_for_current(&rc);
		if (!ar)
			return rc;
		if ((rc = arena_reserve(ar, size_t(bs) * (2 * pad256(nqk) + 2 * pad256(nv)), &deferred)))
			return rc;
		for (int b = 0; b < bs; b++) {
			cudaStream_t st = ar->st[b % NPIPE];
			void *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk), *dv = arena_take(ar, nv), *dvo = arena_take(ar, nv);
			H2D(dq, off(q, b * nqk), nqk, ar->s_in);
			H2D(dk, off(k, b * nqk), nqk, ar->s_in);
			H2D(dv, off(v, b * nv), nv, ar->s_in);
			L1B_TRY(stream_after(ar, st, ar->s_in));
			if ((rc = dense_softmax_v_launch(dq, dk, dv, dvo, nullptr, 1, n_tok, n_heads, width, v_width, mode, dtype, st)))
				return rc;
			L1B_TRY(stream_after(ar, ar->s_out, st));
			D2H(off(vo, b * nv), dvo, nv, ar->s_out);
		}
	}
	return first_error(deferred, l1attn_host_sync());
}

extern "C" int l1attn_dense_bwd_host_async(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, int bs,
					    int n_tok, int n_heads, int width, int dtype)
{
	const void *ptrs[] = {d_attn, q, k, d_q, d_k};
	int rc = check_dense(ptrs, 5, bs, n_tok, n_heads, width, dtype);
	if (rc)
		return rc;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(n_tok) * n_heads * width * es, na = size_t(n_tok) * n_tok * n_heads * es;
	if (na == 0 || bs == 0)
		return L1ATTN_OK;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	const int G = host_group(bs, na);
	const size_t nsc = dense_bwd_scratch_bytes(G, n_tok, n_heads, width, dtype);
	int deferred;
	if ((rc = arena_reserve(ar, size_t(bs) * (4 * pad256(nqk) + pad256(na)) + size_t((bs + G - 1) / G) * pad256(nsc) + 4096, &deferred)))
		return rc;
	for (int b = 0, it = 0; b < bs; b += G, it++) {
		const int g = bs - b < G ? bs - b : G;
		cudaStream_t st = ar->st[it % NPIPE];
		void *dq = arena_take(ar, g * nqk), *dk = arena_take(ar, g * nqk), *dg = arena_take(ar, g * na);
		void *ddq = arena_take(ar, g * nqk), *ddk = arena_take(ar, g * nqk), *dsc = arena_take(ar, nsc);
		H2D(dq, off(q, b * nqk), g * nqk, ar->s_in);
		H2D(dk, off(k, b * nqk), g * nqk, ar->s_in);
		H2D(dg, off(d_attn, b * na), g * na, ar->s_in);
		L1B_TRY(stream_after(ar, st, ar->s_in));
		if ((rc = dense_bwd_launch(dg, dq, dk, ddq, ddk, dsc, g, n_tok, n_heads, width, dtype, st)))
			return rc;
		L1B_TRY(stream_after(ar, ar->s_out, st));
		D2H(off(d_q, b * nqk), ddq, g * nqk, ar->s_out);
		D2H(off(d_k, b * nqk), ddk, g * nqk, ar->s_out);
	}
	return deferred;
}

extern "C" int l1attn_dense_bwd_host(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, int bs,
				      int n_tok, int n_heads, int width, int dtype)
{
	const int rc = l1attn_dense_bwd_host_async(d_attn, q, k, d_q, d_k, bs, n_tok, n_heads, width, dtype);
	return first_error(rc, l1attn_host_sync());
}

// coo -> device, edge index built on the first compute stream; the other compute streams wait for it.  The status
// word of the index build (an out-of-range row) is read back into the pinned block and reported by the next
// l1attn_host_sync().
static int host_index(Arena *ar, const int32_t *coo, int cl, int n_tok, int dst_mxlen, void **dix)
{
	const size_t nc = size_t(cl) * 16, nix = l1attn_sparse_index_bytes(cl, n_tok, dst_mxlen);
	void *dc = arena_take(ar, nc);
	*dix = arena_take(ar, nix);
	int32_t *dstat = static_cast<int32_t *>(arena_take(ar, 4));
	if (cl)
		H2D(dc, coo, nc, ar->s_in);
	L1B_TRY(stream_after(ar, ar->st[0], ar->s_in));
	int rc = l1attn_sparse_build_index(static_cast<int32_t *>(dc), cl, n_tok, dst_mxlen, *dix, dstat, ar->st[0]);
	if (rc)
		return rc;
	int32_t *hstat = &ar->stat[ar->nstat++];
	*hstat = 0;
	L1B_TRY(stream_after(ar, ar->s_out, ar->st[0]));
	D2H(hstat, dstat, 4, ar->s_out);
	for (int i = 1; i < NPIPE; i++)
		L1B_TRY(stream_after(ar, ar->st[i], ar->st[0]));
	return L1ATTN_OK;
}

extern "C" int l1attn_sparse_fwd_host_async(const void *v, const void *vb, const void *q, const void *k,
					     const int32_t *coo, void *vo, void *attn, int bs, int n_tok, int n_heads,
					     int width, int v_width, int cl, int dst_mxlen, int use_softmax, int bidi, int dtype)
{
	if (bs < 0 || n_tok < 0 || n_heads < 0 || width < 1 || v_width < 1 || cl < 0 || dst_mxlen < 0 ||
	    (dtype != L1ATTN_F32 && dtype != L1ATTN_F64))
		return L1ATTN_ERR_ARG;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(n_tok) * n_heads * width * es, nv = size_t(n_tok) * n_heads * v_width * es;
	const size_t na = size_t(n_tok) * dst_mxlen * n_heads * es, nc = size_t(cl) * 16; // per batch item
	if (nv == 0 || bs == 0)
		return L1ATTN_OK;
	if (!v || !q || !k || !vo || (na && !attn) || (cl && !coo) || (bidi && !vb))
		return L1ATTN_ERR_ARG;
	const size_t nix = l1attn_sparse_index_bytes(cl, n_tok, dst_mxlen);
	int rc;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	int deferred;
	if ((rc = arena_reserve(ar, size_t(bs) * (2 * pad256(nqk) + 3 * pad256(nv) + pad256(na)) + pad256(nc) + pad256(nix) + 512,
				&deferred)))
		return rc;
	void *dix;
	if ((rc = host_index(ar, coo, cl, n_tok, dst_mxlen, &dix)))
		return rc;
	for (int b = 0; b < bs; b++) {
		cudaStream_t st = ar->st[b % NPIPE];
		void *dv = arena_take(ar, nv), *dvb = arena_take(ar, nv), *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk);
		void *dvo = arena_take(ar, nv), *da = arena_take(ar, na);
		H2D(dv, off(v, b * nv), nv, ar->s_in);
		if (bidi)
			H2D(dvb, off(vb, b * nv), nv, ar->s_in);
		H2D(dq, off(q, b * nqk), nqk, ar->s_in);
		H2D(dk, off(k, b * nqk), nqk, ar->s_in);
		L1B_TRY(stream_after(ar, st, ar->s_in));
		if ((rc = l1attn_sparse_fwd(dv, dvb, dq, dk, dix, dvo, da, 1, n_tok, n_heads, width, v_width, cl, dst_mxlen,
					    use_softmax, bidi, dtype, st)))
			return rc;
		L1B_TRY(stream_after(ar, ar->s_out, st));
		D2H(off(vo, b * nv), dvo, nv, ar->s_out);
		if (na)
			D2H(off(attn, b * na), da, na, ar->s_out);
	}
	return deferred;
}

extern "C" int l1attn_sparse_fwd_host(const void *v, const void *vb, const void *q, const void *k,
				       const int32_t *coo, void *vo, void *attn, int bs, int n_tok, int n_heads,
				       int width, int v_width, int cl, int dst_mxlen, int use_softmax, int bidi, int dtype)
{
	const int rc = l1attn_sparse_fwd_host_async(v, vb, q, k, coo, vo, attn, bs, n_tok, n_heads, width, v_width, cl,
						    dst_mxlen, use_softmax, bidi, dtype);
	return first_error(rc, l1attn_host_sync());
}

extern "C" int l1attn_sparse_bwd_host_async(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
					     const int32_t *coo, const void *attn, void *d_v, void *d_vb, void *d_q,
					     void *d_k, int bs, int n_tok, int n_heads, int width, int v_width, int cl,
					     int dst_mxlen, int use_softmax, int bidi, int dtype)
{
	if (bs < 0 || n_tok < 0 || n_heads < 0 || width < 1 || v_width < 1 || cl < 0 || dst_mxlen < 0 ||
	    (dtype != L1ATTN_F32 && dtype != L1ATTN_F64))
		return L1ATTN_ERR_ARG;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	const size_t nqk = size_t(n_tok) * n_heads * width * es, nv = size_t(n_tok) * n_heads * v_width * es;
	const size_t na = size_t(n_tok) * dst_mxlen * n_heads * es, nc = size_t(cl) * 16;
	if (nv == 0 || bs == 0)
		return L1ATTN_OK;
	if (!dvo || !v || !q || !k || !d_v || !d_q || !d_k || (na && !attn) || (cl && !coo) || (bidi && (!vb || !d_vb)))
		return L1ATTN_ERR_ARG;
	const size_t nix = l1attn_sparse_index_bytes(cl, n_tok, dst_mxlen);
	int rc;
	std::lock_guard<std::mutex> lock(g_mu);
	Arena *ar = arena_for_current(&rc);
	if (!ar)
		return rc;
	int deferred;
	if ((rc = arena_reserve(ar, size_t(bs) * (4 * pad256(nqk) + 5 * pad256(nv) + 2 * pad256(na ? na : 1)) + pad256(nc) + pad256(nix) + 512,
				&deferred)))
		return rc;
	void *dix;
	if ((rc = host_index(ar, coo, cl, n_tok, dst_mxlen, &dix)))
		return rc;
	for (int b = 0; b < bs; b++) {
		cudaStream_t st = ar->st[b % NPIPE];
		void *ddvo = arena_take(ar, nv), *dv = arena_take(ar, nv), *dvb = arena_take(ar, nv);
		void *dq = arena_take(ar, nqk), *dk = arena_take(ar, nqk), *da = arena_take(ar, na);
		void *gdv = arena_take(ar, nv), *gdvb = arena_take(ar, nv), *gdq = arena_take(ar, nqk), *gdk = arena_take(ar, nqk);
		void *dx = arena_take(ar, na);
		H2D(ddvo, off(dvo, b * nv), nv, ar->s_in);
		H2D(dv, off(v, b * nv), nv, ar->s_in);
		if (bidi)
			H2D(dvb, off(vb, b * nv), nv, ar->s_in);
		H2D(dq, off(q, b * nqk), nqk, ar->s_in);
		H2D(dk, off(k, b * nqk), nqk, ar->s_in);
		if (na)
			H2D(da, off(attn, b * na), na, ar->s_in);
		L1B_TRY(stream_after(ar, st, ar->s_in));
		if ((rc = l1attn_sparse_bwd(ddvo, dv, dvb, dq, dk, dix, da, gdv, gdvb, gdq, gdk, dx, 1, n_tok, n_heads, width,
					    v_width, cl, dst_mxlen, use_softmax, bidi, dtype, st)))
			return rc;
		L1B_TRY(stream_after(ar, ar->s_out, st));
		D2H(off(d_v, b * nv), gdv, nv, ar->s_out);
		if (bidi)
			D2H(off(d_vb, b * nv), gdvb, nv, ar->s_out);
		D2H(off(d_q, b * nqk), gdq, nqk, ar->s_out);
		D2H(off(d_k, b * nqk), gdk, nqk, ar->s_out);
	}
	return deferred;
}

extern "C" int l1attn_sparse_bwd_host(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
				       const int32_t *coo, const void *attn, void *d_v, void *d_vb, void *d_q,
				       void *d_k, int bs, int n_tok, int n_heads, int width, int v_width, int cl,
				       int dst_mxlen, int use_softmax, int bidi, int dtype)
{
	const int rc = l1attn_sparse_bwd_host_async(dvo, v, vb, q, k, coo, attn, d_v, d_vb, d_q, d_k, bs, n_tok, n_heads,
						    width, v_width, cl, dst_mxlen, use_softmax, bidi, dtype);
	return first_error(rc, l1attn_host_sync());
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
	int deferred;
	if ((rc = arena_reserve(ar, pad256(nco) + pad256(ncoo) + 512, &deferred)))
		return rc;
	if (deferred)
		return deferred;
	cudaStream_t st = ar->st[0];
	const size_t mark = ar->used; // this call is synchronous: its slices are handed back before it returns
	void *dco = arena_take(ar, nco), *dcoo = arena_take(ar, ncoo);
	int64_t *dmm = static_cast<int64_t *>(arena_take(ar, 16));
	int32_t *dmx = static_cast<int32_t *>(arena_take(ar, 8));
	ar->used = mark;
	// first pass: key range (needs a round trip to size the counters)
	long long lo = 0, n_keys = 0;
	if (cl) {
		H2D(dco, co, nco, st);
		if ((rc = l1attn_i64_minmax(static_cast<int64_t *>(dco), 2LL * cl, dmm, st)))
			return rc;
		int64_t mm[2];
		D2H(mm, dmm, 16, st);
		L1B_CUDA(cudaStreamSynchronize(st));
		if (mm[0] < INT32_MIN || mm[1] > INT32_MAX)
			return L1ATTN_ERR_SHAPE; // the expanded list is int32, as the reference's is
		lo = mm[0];
		n_keys = mm[1] - mm[0] + 1;
	}
	void *cnt = nullptr;
	const size_t ncnt = l1attn_expand_coo_scratch_bytes(n_keys);
	if (ncnt)
		L1B_CUDA(cudaMalloc(&cnt, ncnt)); // rare: more than 51200 distinct token ids
	rc = l1attn_expand_coo(static_cast<int64_t *>(dco), cl, static_cast<int32_t *>(dcoo), dmx, lo, n_keys, cnt, st);
	int32_t mx[2] = {1, 1};
	if (!rc) {
		cudaError_t e = cudaSuccess;
		if (cl)
			e = cudaMemcpyAsync(coo, dcoo, ncoo, cudaMemcpyDeviceToHost, st);
		if (e == cudaSuccess)
			e = cudaMemcpyAsync(mx, dmx, 8, cudaMemcpyDeviceToHost, st);
		if (e == cudaSuccess)
			e = cudaStreamSynchronize(st);
		if (e != cudaSuccess)
			rc = cuda_fail(e);
	} else {
		(void)cudaStreamSynchronize(st);
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
	rc = arena_sync(ar);
	if (ar->base) {
		L1B_CUDA(cudaDeviceSynchronize());
		L1B_CUDA(cudaFree(ar->base));
	}
	ar->base = nullptr;
	ar->cap = 0;
	return rc;
}
