// Tie detector for the fast dense backward.
//
// The two-instruction form of the backward (dense_bwd_tma.cu) is valid for a stretch of work only
// if none of its `a` values equals a `b` value of the same (batch, head, width index): sign(0) must
// be 0, and the compare form cannot see a tie.  This kernel finds every token row that takes part
// in such a tie and marks the row groups that contain one (layout: dense_bwd_tiles.h); a warp of the
// backward runs its exact loop where its marked x rows meet a marked y tile and the short loop elsewhere.
//
// Exact, in two steps.  One CTA handles NC width columns of one (batch, head):
//   1. filter: every k value sets three bits of one hashed word of its column's bitmap in shared
//      memory; a q value whose three bits are all set is a candidate.  With 64 bits per token (up to
//      4096 tokens) the false-candidate rate is ~1/1000 per value: about four candidates per CTA;
//   2. proof: every candidate value is compared, bit pattern against bit pattern, with all k values
//      of its column (held in registers by the threads that loaded them).  Matching k rows and
//      the candidate's q row are the rows that tie.
// Values are canonical bit patterns (-0 becomes +0); NaNs are skipped because they equal nothing.
// If a CTA finds more candidates than its list holds (heavy ties: padded tokens, q == k) it falls
// back to marking conservatively: the candidate q rows it could not list and every k row of the
// group.  Marking too much only costs speed, never correctness.
#include "common.cuh"
#include "dense_bwd_tiles.h"

namespace l1b {
namespace {

constexpr int NT_MAX = 1024; // threads per CTA: 256..1024, chosen so that one batch of TB tokens per thread covers n_tok when possible
constexpr int TB = 4;    // tokens per thread per batch
constexpr int CAP = 512; // candidate list entries per CTA

__device__ __forceinline__ unsigned canon(float x) { return __float_as_uint(x + 0.0f); }
// The three filter bits of a value lie in ONE 32-bit word of its column's bitmap: the word comes from the top bits of
// one hash, the bit positions from a second one.  One shared-memory atomic per k value and one load per q value (bits
// in two words cost twice that, and the shared-memory atomics and the proof loop over the candidates are what
// bounds this kernel; two bits in one word gave three times the false candidates and a 35 % slower kernel).
__device__ __forceinline__ unsigned hash_word(unsigned b, int sh) { return (b * 0x9E3779B1u) >> sh; } // sh = 32 - log2(words)
__device__ __forceinline__ unsigned hash_bits(unsigned b)
{
	const unsigned x = (b ^ (b >> 15)) * 0xC2B2AE3Du;
	return (1u << (x >> 27)) | (1u << ((x >> 22) & 31u)) | (1u << ((x >> 17) & 31u));
}

template <int NC>
__device__ __forceinline__ void load_batch(const float *base, size_t row, int t0, int n_tok, int ncol, float (&v)[TB][NC])
{
	const int NT = blockDim.x;
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

// grid: bs * n_heads * ceil(width / NC) CTAs.  smem: NC bitmaps of (1 << log2bits) bits.
template <int NC>
__global__ void __launch_bounds__(NT_MAX) dense_ties_kernel(const float *__restrict__ q, const float *__restrict__ k,
							 unsigned char *flags, int n_tok, int n_heads, int width,
							 int log2bits, BwdFlagLayout fl, int *tie_hdr, uint4 *tie_list)
{
	extern __shared__ unsigned bitmap[]; // [NC][words]
	__shared__ unsigned cand_bits[CAP];  // candidate value
	__shared__ unsigned cand_where[CAP]; // (column << 24) | q token
	__shared__ unsigned char cand_hit[CAP];
	__shared__ int n_cand, overflow;
	const int NT = blockDim.x;
	const unsigned words = 1u << (log2bits - 5);
	const int sh = 32 - (log2bits - 5);
	const int ncg = (width + NC - 1) / NC;
	unsigned r = blockIdx.x;
	const int w0 = int(r % ncg) * NC;
	r /= ncg;
	const int h = int(r % n_heads);
	const int b = int(r / n_heads);
	const int ncol = min(NC, width - w0);
	{
		uint4 *bm4 = reinterpret_cast<uint4 *>(bitmap);
		for (unsigned i = threadIdx.x; i < NC * words / 4; i += NT)
			bm4[i] = make_uint4(0u, 0u, 0u, 0u);
		for (int i = threadIdx.x; i < CAP; i += NT)
			cand_hit[i] = 0;
		if (threadIdx.x == 0) {
			n_cand = 0;
			overflow = 0;
		}
	}
	__syncthreads();
	const size_t row = size_t(n_heads) * width;
	const float *qb = q + size_t(b) * n_tok * row + size_t(h) * width + w0;
	const float *kb = k + size_t(b) * n_tok * row + size_t(h) * width + w0;
	unsigned char *xq = flags + fl.xoff(0), *xk = flags + fl.xoff(1), *yk = flags + fl.yoff(0), *yq = flags + fl.yoff(1);
	const bool one_batch = n_tok <= NT * TB;
	float v[TB][NC];

	// 1a. k values -> bitmaps
	for (int t0 = threadIdx.x; t0 < n_tok; t0 += NT * TB) {
		load_batch<NC>(kb, row, t0, n_tok, ncol, v);
#pragma unroll
		for (int i = 0; i < TB; i++)
#pragma unroll
			for (int j = 0; j < NC; j++) {
				const float x = v[i][j];
				if (t0 + i * NT < n_tok && j < ncol && x == x) {
					const unsigned bits = canon(x);
					atomicOr(&bitmap[j * words + hash_word(bits, sh)], hash_bits(bits));
				}
			}
	}
	__syncthreads();
	// 1b. q values that pass the filter -> candidate list
	{
		float qv[TB][NC];
		for (int t0 = threadIdx.x; t0 < n_tok; t0 += NT * TB) {
			load_batch<NC>(qb, row, t0, n_tok, ncol, qv);
#pragma unroll
			for (int i = 0; i < TB; i++)
#pragma unroll
				for (int j = 0; j < NC; j++) {
					const float x = qv[i][j];
					const int t = t0 + i * NT;
					if (t < n_tok && j < ncol && x == x) {
						const unsigned bits = canon(x), want = hash_bits(bits);
						if ((bitmap[j * words + hash_word(bits, sh)] & want) == want) {
							{
								const int idx = atomicAdd(&n_cand, 1);
								if (idx < CAP) {
									cand_bits[idx] = bits;
									cand_where[idx] = (unsigned(j) << 24) | unsigned(t);
								} else { // list full: mark this q row without proof
									const size_t g = fl.group(b, h, w0 + j);
									xq[g * fl.nxf + t / BWD_XF] = 1;
									yq[g * fl.ny + t / BWD_TY] = 1;
									overflow = 1;
									tie_hdr[1] = 1; // not every tie of this call gets listed
								}
							}
						}
					}
				}
		}
	}
	__syncthreads();
	const int nc = min(n_cand, CAP);
	if (nc == 0 && !overflow)
		return;
	// 2. proof: candidates against every k value of their column (k batch still in v when one_batch)
	for (int t0 = threadIdx.x; t0 < n_tok; t0 += NT * TB) {
		if (!one_batch)
			load_batch<NC>(kb, row, t0, n_tok, ncol, v);
		for (int ci = 0; ci < nc; ci++) {
			const unsigned bits = cand_bits[ci];
			const int col = int(cand_where[ci] >> 24);
#pragma unroll
			for (int i = 0; i < TB; i++) {
				const int t = t0 + i * NT;
#pragma unroll
				for (int j = 0; j < NC; j++)
					if (j == col && t < n_tok && v[i][j] == v[i][j] && canon(v[i][j]) == bits) {
						const size_t g = fl.group(b, h, w0 + j);
						xk[g * fl.nxf + t / BWD_XF] = 1; // k row t equals a q value
						yk[g * fl.ny + t / BWD_TY] = 1;
						cand_hit[ci] = 1;
						// the proven tie itself, for the fix kernel: (batch, head, column), query row, source row
						const int idx = atomicAdd(&tie_hdr[0], 1);
						if (idx < BWD_TIE_CAP)
							tie_list[idx] = make_uint4((unsigned(b) * n_heads + h) * width + w0 + j,
										   cand_where[ci] & 0xffffffu, unsigned(t), 0u);
						else
							tie_hdr[1] = 1;
					}
			}
		}
		if (overflow) { // unlisted candidates may match any k row: mark them all
#pragma unroll
			for (int i = 0; i < TB; i++) {
				const int t = t0 + i * NT;
				if (t < n_tok)
					for (int j = 0; j < ncol; j++) {
						const size_t g = fl.group(b, h, w0 + j);
						xk[g * fl.nxf + t / BWD_XF] = 1;
						yk[g * fl.ny + t / BWD_TY] = 1;
					}
			}
		}
	}
	__syncthreads();
	for (int ci = threadIdx.x; ci < nc; ci += NT)
		if (cand_hit[ci]) { // proven: this q row equals some k value
			const unsigned wv = cand_where[ci];
			const int t = int(wv & 0xffffffu), j = int(wv >> 24);
			const size_t g = fl.group(b, h, w0 + j);
			xq[g * fl.nxf + t / BWD_XF] = 1;
			yq[g * fl.ny + t / BWD_TY] = 1;
		}
}

template <int NC>
int launch_nc(const float *q, const float *k, unsigned char *flags, int bs, int n_tok, int n_heads, int width, int log2bits,
	      const BwdFlagLayout &fl, int *tie_hdr, uint4 *tie_list, cudaStream_t st)
{
	const long long grid = (long long)bs * n_heads * ((width + NC - 1) / NC);
	if (grid > 0x7fffffffLL)
		return 1;
	const size_t smem = size_t(NC) * (size_t(1) << log2bits) / 8;
	L1B_CUDA(cudaFuncSetAttribute(dense_ties_kernel<NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	int nt = 256;
	while (nt < NT_MAX && nt * TB < n_tok)
		nt *= 2;
	dense_ties_kernel<NC><<<unsigned(grid), nt, smem, st>>>(q, k, flags, n_tok, n_heads, width, log2bits, fl, tie_hdr, tie_list);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

// Repairs the listed ties after the compare-form backward.  That form counts a term as +g where a > b and as -g
// otherwise, so a tie q == k (which must contribute nothing) has put -scale * g into d_q[b][t][h][w]: it gets
// scale * g[b][s][t][h] back.  d_k[b][s][h][w] received -scale * g from the two-pass kernel (which compares k > q
// for it) and +scale * g from the single-visit kernel (one compare q > k for both): dk_sign = +1 / -1.
// One CTA.  The list arrives in no particular order (the detector appends with an atomic counter), so it is
// ranked first -- by (column, query row, source row) for d_q, by (column, source row, query row) for d_k -- and
// every run of entries that hit the same output element is summed by one thread in rank order: the result
// does not depend on the order of arrival.
__global__ void __launch_bounds__(1024)
dense_tiefix_kernel(const int *__restrict__ tie_hdr, const uint4 *__restrict__ ties, const float *__restrict__ g,
		    float *__restrict__ d_q, float *__restrict__ d_k, int n_tok, int n_heads, int width, float scale, float dk_scale)
{
	extern __shared__ __align__(16) unsigned char fix_smem[];
	if (tie_hdr[1] != 0)
		return; // list incomplete: the backward ran its exact loops instead
	const int n = min(tie_hdr[0], BWD_TIE_CAP);
	if (n == 0)
		return;
	uint4 *e = reinterpret_cast<uint4 *>(fix_smem);                             // {column, query row, source row, -}
	int *perm_q = reinterpret_cast<int *>(fix_smem + size_t(BWD_TIE_CAP) * 16); // rank -> entry, d_q order
	int *perm_k = perm_q + BWD_TIE_CAP;
	for (int i = threadIdx.x; i < n; i += blockDim.x)
		e[i] = ties[i];
	__syncthreads();
	for (int i = threadIdx.x; i < n; i += blockDim.x) {
		const uint4 a = e[i];
		int rq = 0, rk = 0;
		for (int j = 0; j < n; j++) {
			const uint4 c = e[j];
			const bool col_lt = c.x < a.x, col_eq = c.x == a.x;
			rq += (col_lt || (col_eq && (c.y < a.y || (c.y == a.y && c.z < a.z)))) ? 1 : 0;
			rk += (col_lt || (col_eq && (c.z < a.z || (c.z == a.z && c.y < a.y)))) ? 1 : 0;
		}
		perm_q[rq] = i; // entries are distinct (column, query row, source row) triples: the ranks are a permutation
		perm_k[rk] = i;
	}
	__syncthreads();
	const size_t row = size_t(n_heads) * width;
	const unsigned hwn = unsigned(n_heads) * unsigned(width);
	auto gval = [&](const uint4 &a) -> float {
		const unsigned b = a.x / hwn, hh = (a.x % hwn) / unsigned(width);
		return g[((size_t(b) * n_tok + a.z) * n_tok + a.y) * n_heads + hh];
	};
	for (int p = threadIdx.x; p < n; p += blockDim.x) {
		const uint4 a = e[perm_q[p]];
		if (p == 0 || e[perm_q[p - 1]].x != a.x || e[perm_q[p - 1]].y != a.y) {
			float sum = 0.f;
			for (int pp = p; pp < n; pp++) {
				const uint4 c = e[perm_q[pp]];
				if (c.x != a.x || c.y != a.y)
					break;
				sum += gval(c);
			}
			d_q[(size_t(a.x / hwn) * n_tok + a.y) * row + a.x % hwn] += scale * sum;
		}
	}
	for (int p = threadIdx.x; p < n; p += blockDim.x) {
		const uint4 a = e[perm_k[p]];
		if (p == 0 || e[perm_k[p - 1]].x != a.x || e[perm_k[p - 1]].z != a.z) {
			float sum = 0.f;
			for (int pp = p; pp < n; pp++) {
				const uint4 c = e[perm_k[pp]];
				if (c.x != a.x || c.z != a.z)
					break;
				sum += gval(c);
			}
			d_k[(size_t(a.x / hwn) * n_tok + a.z) * row + a.x % hwn] += dk_scale * sum;
		}
	}
}

} // namespace

// Fills the flag arrays, the tie header and the tie list in `scratch` (device, laid out by bwd_scratch_layout();
// the d_q partials behind them are not touched).  Returns L1ATTN_OK, a negative
// error, or 1 when the detector does not apply (token index beyond 24 bits, width not a multiple of 4,
// q or k not 16-byte aligned);
// the caller then runs every tile with the exact loop.
int dense_ties_launch(const float *q, const float *k, unsigned char *scratch, int bs, int n_tok, int n_heads, int width,
		      cudaStream_t st)
{
	if (width % 4 != 0 || n_tok >= (1 << 24))
		return 1;
	if (!aligned(q, 16) || !aligned(k, 16))
		return 1; // the kernel reads four columns as one 16-byte vector; the C ABI only promises element alignment
	// 64 bits per token (32 KiB per CTA at 1024 tokens: seven CTAs per SM hide the load latency; 128 bits per
	// token held three and took twice the time for 1/4 of the false candidates) up to 4096 tokens, fewer
	// beyond: more false candidates to prove, and past ~16k tokens the list overflows into the
	// conservative marking.  Four columns per CTA keep the global loads 16 bytes wide.
	int log2bits = 15;
	while (log2bits < 18 && (1 << log2bits) < 64 * n_tok)
		log2bits++;
	if ((unsigned long long)bs * n_heads * width > 0xffffffffull)
		return 1; // a tie entry holds the (batch, head, column) index in 32 bits
	const BwdFlagLayout fl = bwd_flag_layout(bs, n_tok, n_heads, width);
	const BwdScratchLayout sl = bwd_scratch_layout(bs, n_tok, n_heads, width);
	L1B_CUDA(cudaMemsetAsync(scratch, 0, sl.hdr + 256, st)); // flags and header
	return launch_nc<4>(q, k, scratch + sl.flags, bs, n_tok, n_heads, width, log2bits, fl,
			    reinterpret_cast<int *>(scratch + sl.hdr), reinterpret_cast<uint4 *>(scratch + sl.ties), st);
}

// Enqueue after the compare-form backward: adds the listed ties' terms back (no-op when the list overflowed).
int dense_tiefix_launch(const void *d_attn, void *d_q, void *d_k, const unsigned char *scratch, int bs, int n_tok,
			int n_heads, int width, int dk_sign, cudaStream_t st)
{
	const BwdScratchLayout sl = bwd_scratch_layout(bs, n_tok, n_heads, width);
	const size_t smem = size_t(BWD_TIE_CAP) * (16 + 8);
	L1B_CUDA(cudaFuncSetAttribute(dense_tiefix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	dense_tiefix_kernel<<<1, 1024, smem, st>>>(reinterpret_cast<const int *>(scratch + sl.hdr),
						   reinterpret_cast<const uint4 *>(scratch + sl.ties), (const float *)d_attn,
						   (float *)d_q, (float *)d_k, n_tok, n_heads, width,
						   float(-1.0 / sqrt(double(width))), float(-dk_sign / sqrt(double(width))));
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace l1b
