// Integer graph preprocessing: expandCoo on the GPU and the edge index of the sparse kernels.
//
// Both need, for every row i of a key column, rank_i = #{j < i : key_j == key_i} -- the running
// per-key counter of the reference's Python loop (cuda/l1attn_sparse_cuda.py:70-91).  The order
// is part of the result (bit-exact contract), so it is computed by ONE warp that walks the rows
// in order, 32 at a time: lanes holding the same key find each other with match.any, take
// consecutive ranks after the key's running count and the highest such lane writes the count
// back.  Counts live in shared memory (up to SMEM_KEYS keys) or in a caller-provided global
// array.  The dst and src columns are independent and run as two CTAs.
#include "common.cuh"

namespace l1b {
namespace {

constexpr int SMEM_KEYS = 50 * 1024; // int32 counters that fit beside nothing else in 227 KB

// keys[i*stride], i < n; rows whose key is outside [key_lo, key_lo+n_keys) get rank -1 and are
// not counted.  rank_out[i*rstride] may alias keys (each row's key is read before its rank is
// written, and rows are prefetched strictly ahead).  blockIdx.x selects the column: pointers
// advance by `col_step` elements, counts by n_keys, max_out by 1.
template <typename K>
__global__ void __launch_bounds__(32) rank_by_key_kernel(const K *keys, int stride, int n, long long key_lo,
							  long long n_keys, int32_t *rank_out, int rstride,
							  int32_t *counts, int32_t *max_out, int col_step,
							  int use_smem)
{
	extern __shared__ int32_t scnt[];
	const int lane = threadIdx.x;
	keys += size_t(blockIdx.x) * col_step;
	rank_out += size_t(blockIdx.x) * col_step;
	int32_t *cnt = use_smem ? scnt : counts + size_t(blockIdx.x) * n_keys;
	if (use_smem)
		for (long long i = lane; i < n_keys; i += 32)
			scnt[i] = 0;
	__syncwarp();
	int mx = 0; // the reference starts its maxima at 0, so an empty list reports length 1
	long long nxt = 0;
	if (lane < n)
		nxt = (long long)keys[size_t(lane) * stride];
	for (int base = 0; base < n; base += 32) {
		const int i = base + lane;
		const long long key = nxt - key_lo;
		if (i + 32 < n)
			nxt = (long long)keys[size_t(i + 32) * stride];
		const bool valid = i < n && key >= 0 && key < n_keys;
		const unsigned act = __ballot_sync(0xffffffffu, valid);
		int rank = -1;
		if (valid) {
			const unsigned m = __match_any_sync(act, key);
			const int seen = cnt[key]; // every lane of the group reads the counter ...
			__syncwarp(act);           // ... before its highest lane overwrites it
			rank = seen + __popc(m & ((1u << lane) - 1u));
			if (lane == 31 - __clz(m))
				cnt[key] = rank + 1;
		}
		__syncwarp();
		if (i < n)
			rank_out[size_t(i) * rstride] = rank;
		mx = max(mx, rank);
	}
	for (int o = 16; o > 0; o >>= 1)
		mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
	if (max_out && lane == 0)
		max_out[blockIdx.x] = mx + 1;
	if (use_smem && counts) { // hand the final counts to the caller (index build needs them)
		__syncwarp();
		int32_t *gc = counts + size_t(blockIdx.x) * n_keys;
		for (long long i = lane; i < n_keys; i += 32)
			gc[i] = scnt[i];
	}
}

// coo[i][0..1] = (int32) co[i][0..1]
__global__ void expand_copy_kernel(const int64_t *co, int cl, int32_t *coo)
{
	const int i = blockIdx.x * blockDim.x + threadIdx.x;
	if (i < cl) {
		coo[4 * size_t(i) + 0] = int32_t(co[2 * size_t(i) + 0]);
		coo[4 * size_t(i) + 1] = int32_t(co[2 * size_t(i) + 1]);
	}
}

__global__ void __launch_bounds__(1024) minmax_kernel(const int64_t *x, long long n, int64_t *out)
{
	__shared__ long long slo[32], shi[32];
	long long lo = INT64_MAX, hi = INT64_MIN;
	for (long long i = threadIdx.x; i < n; i += blockDim.x) {
		const long long v = x[i];
		lo = min(lo, v);
		hi = max(hi, v);
	}
	for (int o = 16; o > 0; o >>= 1) {
		lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
		hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
	}
	if ((threadIdx.x & 31) == 0) {
		slo[threadIdx.x >> 5] = lo;
		shi[threadIdx.x >> 5] = hi;
	}
	__syncthreads();
	if (threadIdx.x < 32) {
		lo = threadIdx.x < (blockDim.x >> 5) ? slo[threadIdx.x] : INT64_MAX;
		hi = threadIdx.x < (blockDim.x >> 5) ? shi[threadIdx.x] : INT64_MIN;
		for (int o = 16; o > 0; o >>= 1) {
			lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
			hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
		}
		if (threadIdx.x == 0) {
			out[0] = lo;
			out[1] = hi;
		}
	}
}

// ---- sparse edge index ------------------------------------------------------------------

__global__ void idx_init_kernel(int32_t *slot_src, long long nslot, int32_t *cnt, int n_tok, int32_t *status)
{
	const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
	if (i < nslot)
		slot_src[i] = -1;
	if (i < n_tok)
		cnt[i] = 0;
	if (i == 0 && status)
		*status = 0;
}

// slot table + the key column for the src ranking (invalid rows: key -1)
__global__ void idx_scatter_kernel(const int32_t *coo, int cl, int n_tok, int dm, int32_t *slot_src,
				   int32_t *key, int32_t *status)
{
	const int c = blockIdx.x * blockDim.x + threadIdx.x;
	if (c >= cl)
		return;
	const int dst = coo[4 * size_t(c)], src = coo[4 * size_t(c) + 1], r = coo[4 * size_t(c) + 2];
	const bool ok = dst >= 0 && dst < n_tok && src >= 0 && src < n_tok && r >= 0 && r < dm;
	if (ok) {
		slot_src[size_t(dst) * dm + r] = src;
	} else if (status) {
		*status = L1ATTN_ERR_INDEX;
	}
	key[c] = ok ? src : -1;
}

// exclusive scan of cnt[0..n) into off[0..n], one CTA
__global__ void __launch_bounds__(1024) idx_scan_kernel(const int32_t *cnt, int32_t *off, int n)
{
	__shared__ int32_t wsum[32];
	__shared__ int32_t carry_s;
	if (threadIdx.x == 0)
		carry_s = 0;
	__syncthreads();
	const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	for (int base = 0; base < n; base += 1024) {
		const int i = base + threadIdx.x;
		const int v = i < n ? cnt[i] : 0;
		int x = v;
		for (int o = 1; o < 32; o <<= 1) {
			const int y = __shfl_up_sync(0xffffffffu, x, o);
			if (lane >= o)
				x += y;
		}
		if (lane == 31)
			wsum[warp] = x;
		__syncthreads();
		if (warp == 0) {
			int s = wsum[lane];
			for (int o = 1; o < 32; o <<= 1) {
				const int y = __shfl_up_sync(0xffffffffu, s, o);
				if (lane >= o)
					s += y;
			}
			wsum[lane] = s; // inclusive over warps
		}
		__syncthreads();
		const int carry = carry_s;
		const int incl = x + (warp ? wsum[warp - 1] : 0) + carry;
		if (i < n)
			off[i] = incl - v;
		__syncthreads();
		if (threadIdx.x == 1023)
			carry_s = incl;
		__syncthreads();
	}
	if (threadIdx.x == 0)
		off[n] = carry_s;
}

__global__ void idx_fill_kernel(const int32_t *coo, const int32_t *rank, const int32_t *off, int32_t *csc_slot,
				int cl, int dm)
{
	const int c = blockIdx.x * blockDim.x + threadIdx.x;
	if (c >= cl)
		return;
	const int rk = rank[c];
	if (rk < 0)
		return;
	const int dst = coo[4 * size_t(c)], src = coo[4 * size_t(c) + 1], r = coo[4 * size_t(c) + 2];
	csc_slot[off[src] + rk] = dst * dm + r;
}

size_t pad16(size_t n_int) { return ((n_int * 4 + 15) / 16) * 16; }

template <typename K>
int launch_rank(const K *keys, int stride, int n, long long key_lo, long long n_keys, int32_t *rank_out,
		int rstride, int32_t *counts, int32_t *max_out, int col_step, int ncol, cudaStream_t st)
{
	const int use_smem = n_keys <= SMEM_KEYS;
	if (!use_smem && !counts)
		return L1ATTN_ERR_ARG;
	auto kern = rank_by_key_kernel<K>;
	size_t smem = use_smem ? size_t(n_keys) * 4 : 0;
	if (smem > 48 * 1024)
		L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	if (!use_smem)
		L1B_CUDA(cudaMemsetAsync(counts, 0, size_t(ncol) * n_keys * 4, st));
	kern<<<ncol, 32, smem, st>>>(keys, stride, n, key_lo, n_keys, rank_out, rstride, counts, max_out, col_step,
				     use_smem);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace

SparseIndex sparse_index_view(void *base, int cl, int n_tok, int dst_mxlen)
{
	SparseIndex ix;
	unsigned char *p = static_cast<unsigned char *>(base);
	size_t o = 0;
	ix.slot_src = reinterpret_cast<int32_t *>(p + o);
	o += pad16(size_t(n_tok) * dst_mxlen);
	ix.csc_off = reinterpret_cast<int32_t *>(p + o);
	o += pad16(size_t(n_tok) + 1);
	ix.csc_slot = reinterpret_cast<int32_t *>(p + o);
	o += pad16(size_t(cl));
	ix.cnt = reinterpret_cast<int32_t *>(p + o);
	o += pad16(size_t(n_tok));
	ix.rank = reinterpret_cast<int32_t *>(p + o);
	o += pad16(size_t(cl));
	ix.bytes = o ? o : 16;
	return ix;
}

} // namespace l1b

using namespace l1b;

extern "C" size_t l1attn_sparse_index_bytes(int cl, int n_tok, int dst_mxlen)
{
	if (cl < 0 || n_tok < 0 || dst_mxlen < 0)
		return 0;
	return sparse_index_view(nullptr, cl, n_tok, dst_mxlen).bytes;
}

extern "C" int l1attn_sparse_build_index(const int32_t *coo, int cl, int n_tok, int dst_mxlen, void *index,
					  int32_t *status, void *stream)
{
	if (cl < 0 || n_tok < 0 || dst_mxlen < 0 || !index || (cl > 0 && !coo))
		return L1ATTN_ERR_ARG;
	if ((long long)n_tok * dst_mxlen > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	SparseIndex ix = sparse_index_view(index, cl, n_tok, dst_mxlen);
	const long long nslot = (long long)n_tok * dst_mxlen;
	const long long ninit = nslot > n_tok ? nslot : n_tok;
	idx_init_kernel<<<unsigned((ninit + 255) / 256 + 1), 256, 0, st>>>(ix.slot_src, nslot, ix.cnt, n_tok, status);
	L1B_LAUNCH_CHECK();
	if (cl > 0) {
		idx_scatter_kernel<<<(cl + 255) / 256, 256, 0, st>>>(coo, cl, n_tok, dst_mxlen, ix.slot_src, ix.rank, status);
		L1B_LAUNCH_CHECK();
		int rc = launch_rank<int32_t>(ix.rank, 1, cl, 0, n_tok, ix.rank, 1, ix.cnt, nullptr, 0, 1, st);
		if (rc)
			return rc;
	}
	idx_scan_kernel<<<1, 1024, 0, st>>>(ix.cnt, ix.csc_off, n_tok);
	L1B_LAUNCH_CHECK();
	if (cl > 0) {
		idx_fill_kernel<<<(cl + 255) / 256, 256, 0, st>>>(coo, ix.rank, ix.csc_off, ix.csc_slot, cl, dst_mxlen);
		L1B_LAUNCH_CHECK();
	}
	return L1ATTN_OK;
}

extern "C" size_t l1attn_expand_coo_scratch_bytes(long long n_keys)
{
	if (n_keys <= SMEM_KEYS)
		return 0;
	return size_t(n_keys) * 2 * 4;
}

extern "C" int l1attn_expand_coo(const int64_t *co, int cl, int32_t *coo, int32_t *mxlen, long long key_lo,
				  long long n_keys, void *counters, void *stream)
{
	if (cl < 0 || !mxlen || n_keys < 0 || (cl > 0 && (!co || !coo)))
		return L1ATTN_ERR_ARG;
	if (n_keys > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	if (cl > 0) {
		expand_copy_kernel<<<(cl + 255) / 256, 256, 0, st>>>(co, cl, coo);
		L1B_LAUNCH_CHECK();
	}
	// column 0 -> ranks into coo[:,2], column 1 -> coo[:,3]; with cl == 0 the kernel still writes mxlen = 1
	int32_t *cnt = n_keys > SMEM_KEYS ? static_cast<int32_t *>(counters) : nullptr;
	return launch_rank<int64_t>(co, 2, cl, key_lo, n_keys, coo ? coo + 2 : nullptr, 4, cnt, mxlen, 1, 2, st);
}

extern "C" int l1attn_i64_minmax(const int64_t *x, long long n, int64_t *out, void *stream)
{
	if (n < 0 || !out || (n > 0 && !x))
		return L1ATTN_ERR_ARG;
	minmax_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(x, n, out);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}
