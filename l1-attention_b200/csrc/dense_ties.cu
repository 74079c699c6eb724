// Tie detector for the fast dense backward.
//
// The two-instruction form of the backward (dense_bwd_tma.cu) is valid for a stretch of work only
// if none of its `a` values equals a `b` value of the same (batch, head, width index): sign(0) must
// be 0, and the compare form cannot see a tie.  This kernel finds every token row that takes part
// in such a tie and marks the tiles that contain one (layout: dense_bwd_tiles.h); the backward
// runs its exact loop where a marked x tile meets a marked y tile and the short loop elsewhere.
//
// Exact, not probabilistic: one CTA per (batch, head, group of NC width columns) builds, per
// column, an open-addressing hash SET of the key values and one of the query values in shared
// memory (canonical bit patterns: -0 becomes +0; NaNs are left out because they equal nothing) and
// probes each with the other side's values, comparing full bit patterns.  Tables hold
// 2^k >= 2*n_tok slots, so probing always ends at an empty slot.  Values are fetched in batches
// into registers first so that the global-memory latency is paid once per batch, not once per value.
#include "common.cuh"
#include "dense_bwd_tiles.h"

namespace l1b {
namespace {

constexpr unsigned EMPTY = 0xffffffffu; // a NaN pattern: never inserted
constexpr int NT = 256;
constexpr int TB = 4; // tokens per thread per batch

__device__ __forceinline__ unsigned canon(float x) { return __float_as_uint(x + 0.0f); }
__device__ __forceinline__ unsigned slot_of(unsigned bits, int log2p) { return (bits * 2654435761u) >> (32 - log2p); }

__device__ __forceinline__ void insert(unsigned *tab, unsigned mask, int log2p, float x)
{
	if (x != x)
		return;
	const unsigned bits = canon(x);
	unsigned s = slot_of(bits, log2p);
	for (unsigned n = 0; n <= mask; n++) { // bounded; the table is never more than half full
		const unsigned old = atomicCAS(&tab[s], EMPTY, bits);
		if (old == EMPTY || old == bits)
			return;
		s = (s + 1) & mask;
	}
}
__device__ __forceinline__ bool contains(const unsigned *tab, unsigned mask, int log2p, float x)
{
	if (x != x)
		return false;
	const unsigned bits = canon(x);
	unsigned s = slot_of(bits, log2p);
	for (unsigned n = 0; n <= mask; n++) {
		const unsigned v = tab[s];
		if (v == bits)
			return true;
		if (v == EMPTY)
			return false;
		s = (s + 1) & mask;
	}
	return false;
}

// loads TB tokens x NC columns of one tensor for this thread (zero / NaN-free padding is not
// needed: out-of-range tokens are marked by valid[])
template <int NC>
__device__ __forceinline__ void load_batch(const float *base, size_t row, int t0, int n_tok, int ncol, float (&v)[TB][NC])
{
#pragma unroll
	for (int i = 0; i < TB; i++) {
		const int t = t0 + i * NT;
		if (NC == 4 && ncol == 4) {
			float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
			if (t < n_tok)
				x = *reinterpret_cast<const float4 *>(base + size_t(t) * row);
			v[i][0] = x.x;
			v[i][1 % NC] = x.y;
			v[i][2 % NC] = x.z;
			v[i][3 % NC] = x.w;
		} else {
#pragma unroll
			for (int j = 0; j < NC; j++)
				v[i][j] = (t < n_tok && j < ncol) ? base[size_t(t) * row + j] : 0.f;
		}
	}
}

// grid: bs * n_heads * ceil(width / NC) CTAs.  smem: NC * 2 tables of (1 << log2p) words.
template <int NC>
__global__ void __launch_bounds__(NT) dense_ties_kernel(const float *__restrict__ q, const float *__restrict__ k,
							 unsigned char *flags, int n_tok, int n_heads, int width, int log2p,
							 BwdFlagLayout fl)
{
	extern __shared__ unsigned tabs[]; // [NC][2][P]: [..][0] = set of k values, [..][1] = set of q values
	const unsigned P = 1u << log2p, mask = P - 1;
	const int ncg = (width + NC - 1) / NC;
	unsigned r = blockIdx.x;
	const int w0 = int(r % ncg) * NC;
	r /= ncg;
	const int h = int(r % n_heads);
	const int b = int(r / n_heads);
	const int ncol = min(NC, width - w0);
	for (unsigned i = threadIdx.x; i < unsigned(NC) * 2 * P; i += NT)
		tabs[i] = EMPTY;
	__syncthreads();
	const size_t row = size_t(n_heads) * width;
	const float *qb = q + size_t(b) * n_tok * row + size_t(h) * width + w0;
	const float *kb = k + size_t(b) * n_tok * row + size_t(h) * width + w0;
	float qv[TB][NC], kv[TB][NC];
	for (int t0 = threadIdx.x; t0 < n_tok; t0 += NT * TB) {
		load_batch<NC>(qb, row, t0, n_tok, ncol, qv);
		load_batch<NC>(kb, row, t0, n_tok, ncol, kv);
#pragma unroll
		for (int i = 0; i < TB; i++)
			if (t0 + i * NT < n_tok)
#pragma unroll
				for (int j = 0; j < NC; j++)
					if (j < ncol) {
						insert(tabs + (size_t(j) * 2 + 0) * P, mask, log2p, kv[i][j]);
						insert(tabs + (size_t(j) * 2 + 1) * P, mask, log2p, qv[i][j]);
					}
	}
	__syncthreads();
	const unsigned nhg = (n_heads + BWD_HG - 1) / BWD_HG, nws = (width + BWD_WS - 1) / BWD_WS;
	unsigned char *xq = flags + fl.xoff(0), *xk = flags + fl.xoff(1), *yk = flags + fl.yoff(0), *yq = flags + fl.yoff(1);
	for (int t0 = threadIdx.x; t0 < n_tok; t0 += NT * TB) {
		if (n_tok > NT * TB) { // a single batch is still in registers
			load_batch<NC>(qb, row, t0, n_tok, ncol, qv);
			load_batch<NC>(kb, row, t0, n_tok, ncol, kv);
		}
#pragma unroll
		for (int i = 0; i < TB; i++) {
			const int t = t0 + i * NT;
			if (t >= n_tok)
				continue;
#pragma unroll
			for (int j = 0; j < NC; j++) {
				if (j >= ncol)
					continue;
				const size_t g = (size_t(b) * nhg + unsigned(h) / BWD_HG) * nws + unsigned(w0 + j) / BWD_WS;
				if (contains(tabs + (size_t(j) * 2 + 0) * P, mask, log2p, qv[i][j])) { // q row t equals some k
					xq[g * fl.nxt + t / BWD_TX] = 1;
					yq[g * fl.ny + t / BWD_TY] = 1;
				}
				if (contains(tabs + (size_t(j) * 2 + 1) * P, mask, log2p, kv[i][j])) { // k row t equals some q
					xk[g * fl.nxt + t / BWD_TX] = 1;
					yk[g * fl.ny + t / BWD_TY] = 1;
				}
			}
		}
	}
}

template <int NC>
int launch_nc(const float *q, const float *k, unsigned char *flags, int bs, int n_tok, int n_heads, int width, int log2p,
	      const BwdFlagLayout &fl, cudaStream_t st)
{
	const long long grid = (long long)bs * n_heads * ((width + NC - 1) / NC);
	if (grid > 0x7fffffffLL)
		return 1;
	const size_t smem = size_t(NC) * 2 * (size_t(1) << log2p) * 4;
	L1B_CUDA(cudaFuncSetAttribute(dense_ties_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	dense_ties_kernel<NC><<<unsigned(grid), NT, smem, st>>>(q, k, flags, n_tok, n_heads, width, log2p, fl);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace

// Fills the flag arrays (device, bwd_flag_layout(...).bytes() bytes).  Returns L1ATTN_OK, a negative
// error, or 1 when n_tok is too large for the shared-memory tables (the caller then runs every
// tile with the exact loop).
int dense_ties_launch(const float *q, const float *k, unsigned char *flags, int bs, int n_tok, int n_heads, int width,
		      cudaStream_t st)
{
	int log2p = 1;
	while ((1 << log2p) < 2 * n_tok)
		log2p++;
	const size_t per_col = size_t(2) * (size_t(1) << log2p) * 4;
	const size_t budget = 200 * 1024;
	if (per_col > budget || width % 4 != 0)
		return 1;
	const BwdFlagLayout fl = bwd_flag_layout(bs, n_tok, n_heads, width);
	L1B_CUDA(cudaMemsetAsync(flags, 0, fl.bytes(), st));
	if (4 * per_col <= budget / 3) // three CTAs of four columns per SM
		return launch_nc<4>(q, k, flags, bs, n_tok, n_heads, width, log2p, fl, st);
	if (2 * per_col <= budget)
		return launch_nc<2>(q, k, flags, bs, n_tok, n_heads, width, log2p, fl, st);
	return launch_nc<1>(q, k, flags, bs, n_tok, n_heads, width, log2p, fl, st);
}

} // namespace l1b
