// Dense L1 scores, forward -- the B200 fast path.
//
//   attn[b][s][t][h] = scale * sum_w |q[b][t][h][w] - k[b][s][h][w]|
//
// Persistent kernel: one CTA of 16 warps per SM walks a list of (batch, head-group of 8, query
// tile of 64, key tile of 64) work items.
//   * operands arrive by TMA tensor copies (cp.async.bulk.tensor, no multicast): per stage the
//     64-byte-wide width chunk of the q tile and of the k tile, as [token][head][16 B chunk] boxes
//     with the 64-byte hardware swizzle, into a ring of NSTAGE shared-memory stages, each guarded
//     by a full/empty mbarrier pair.  One lane issues them NSTAGE-1 chunks ahead of the math and
//     runs on across work items, so the next item's tiles land while the current one is reduced;
//   * every warp computes: lanes = 8 heads x 4 query rows, each thread keeps an 8 x 8 (query, key)
//     register tile of its head, reads operands with conflict-free 16-byte shared loads (the
//     swizzle spreads the 8 head-lanes over 8 bank groups) and spends 2 FP32 instructions per
//     term (subtract; add with |.| as a source modifier);
//   * the 8 head-lanes write 32 contiguous bytes per (s, t), so every store of a warp fills
//     whole sectors of the heads-innermost output, and no [b,h,t,w] copy of q/k is ever made.
// Out-of-range rows/heads/width are zero-filled by TMA (|0-0| adds nothing) and masked at the store.
// Every mbarrier wait is bounded (tma.cuh); on a timeout the CTA stops and the error word is set.
#include "common.cuh"
#include "tma.cuh"

namespace l1b {
namespace {

constexpr int HG = 8;       // heads per work item
constexpr int LT = 4;       // lanes along the query axis
constexpr int CH = 4;       // 16-byte chunks per (token, head) row per stage
constexpr int NCW = 16;     // consumer warps
constexpr int NSTAGE = 3;
constexpr int TT = 64, TS = 64;
constexpr int TM = 8, TN = 8;
constexpr int STAGE_BYTES = (TT + TS) * HG * CH * 16; // 65536
constexpr int NTHREADS = NCW * 32;

struct Work {
	int ntt, nst, nhg;
	long long total;
};

struct Item {
	int t0, s0, h0, b;
};
__device__ __forceinline__ Item decode_item(const Work &wk, long long r)
{
	Item x;
	x.t0 = int(r % wk.ntt) * TT;
	r /= wk.ntt;
	x.s0 = int(r % wk.nst) * TS;
	r /= wk.nst;
	x.h0 = int(r % wk.nhg) * HG;
	x.b = int(r / wk.nhg);
	return x;
}

template <typename T>
__global__ void __launch_bounds__(NTHREADS, 1)
dense_fwd_tma_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
		     T *__restrict__ attn, int n_tok, int n_heads, int width, T scale, Work wk, int *err)
{
	constexpr int VEC = 16 / sizeof(T);
	constexpr int WC = CH * VEC;
	using V = Pack<T, VEC>;
	extern __shared__ __align__(1024) unsigned char smem_raw[];
	unsigned char *stages = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
	__shared__ __align__(8) uint64_t full_bar[NSTAGE], empty_bar[NSTAGE];

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	if (tid == 0) {
		for (int s = 0; s < NSTAGE; s++) {
			mbar_init(&full_bar[s], 1);
			mbar_init(&empty_bar[s], NCW);
		}
		mbar_fence_init();
	}
	__syncthreads();

	const int nchunk = (width + WC - 1) / WC;
	const bool issuer = tid == 0;

	// issuing side: a cursor (p_item, p_ci, p_it) that runs NSTAGE-1 chunks ahead of the math
	long long p_item = blockIdx.x;
	int p_ci = 0;
	uint32_t p_it = 0;
	bool dead = false;
	auto issue_one = [&]() {
		if (p_item >= wk.total)
			return;
		const int st = p_it % NSTAGE;
		if (!mbar_wait(&empty_bar[st], ((p_it / NSTAGE) & 1) ^ 1, err)) {
			dead = true;
			return;
		}
		const Item x = decode_item(wk, p_item);
		unsigned char *dst = stages + size_t(st) * STAGE_BYTES;
		mbar_expect_tx(&full_bar[st], STAGE_BYTES);
		tma_load_4d(dst, &qmap, &full_bar[st], p_ci * WC, x.h0, x.t0, x.b);
		tma_load_4d(dst + TT * HG * CH * 16, &kmap, &full_bar[st], p_ci * WC, x.h0, x.s0, x.b);
		p_it++;
		if (++p_ci == nchunk) {
			p_ci = 0;
			p_item += gridDim.x;
		}
	};
	if (issuer)
		for (int i = 0; i < NSTAGE - 1; i++)
			issue_one();

	const int lane_h = lane & 7, lane_t = lane >> 3;
	const int wt = warp & 1, ws = warp >> 1; // 2 query halves x 8 key groups
	const int sw = (lane_h >> 1) & 3;        // TMA 64-byte swizzle: chunk ^= address bits 7..8 = (head >> 1) & 3
	uint32_t it = 0;
	for (long long item = blockIdx.x; item < wk.total; item += gridDim.x) {
		const Item x = decode_item(wk, item);
		T acc[TM][TN];
#pragma unroll
		for (int i = 0; i < TM; i++)
#pragma unroll
			for (int j = 0; j < TN; j++)
				acc[i][j] = T(0);

		for (int ci = 0; ci < nchunk; ci++, it++) {
			if (issuer) {
				issue_one(); // refills the stage that every warp released after chunk it-1
				if (dead)
					return;
			}
			__syncwarp();
			const int st = it % NSTAGE;
			if (!mbar_wait(&full_bar[st], (it / NSTAGE) & 1, err))
				return;
			const V *Q = reinterpret_cast<const V *>(stages + size_t(st) * STAGE_BYTES);
			const V *K = Q + TT * HG * CH;
			const V *qp = Q + ((wt * 32 + lane_t) * HG + lane_h) * CH;
			const V *kp = K + ((ws * TN) * HG + lane_h) * CH;
#pragma unroll
			for (int c = 0; c < CH; c++) {
				const int pc = c ^ sw;
				V kv[TN];
#pragma unroll
				for (int j = 0; j < TN; j++)
					kv[j] = kp[j * HG * CH + pc];
#pragma unroll
				for (int i = 0; i < TM; i++) {
					const V qv = qp[i * LT * HG * CH + pc];
#pragma unroll
					for (int j = 0; j < TN; j++)
#pragma unroll
						for (int e = 0; e < VEC; e++)
							acc[i][j] += absdiff(qv.v[e], kv[j].v[e]);
				}
			}
			__syncwarp();
			if (lane == 0)
				mbar_arrive(&empty_bar[st]);
		}

		const int h = x.h0 + lane_h;
		if (h < n_heads) {
			T *ab = attn + size_t(x.b) * n_tok * n_tok * n_heads + h;
#pragma unroll
			for (int j = 0; j < TN; j++) {
				const int s = x.s0 + ws * TN + j;
				if (s >= n_tok)
					continue;
				T *row = ab + size_t(s) * n_tok * n_heads;
#pragma unroll
				for (int i = 0; i < TM; i++) {
					const int t = x.t0 + wt * 32 + lane_t + LT * i;
					if (t < n_tok)
						row[size_t(t) * n_heads] = acc[i][j] * scale;
				}
			}
		}
	}
}

template <typename T> CUtensorMapDataType tmap_dtype();
template <> CUtensorMapDataType tmap_dtype<float>() { return CU_TENSOR_MAP_DATA_TYPE_FLOAT32; }

template <typename T>
int launch(const T *q, const T *k, T *attn, int bs, int n_tok, int n_heads, int width, cudaStream_t st)
{
	constexpr int VEC = 16 / sizeof(T);
	// tensor [bs][n_tok][n_heads][width], innermost first; one stage row is CH*VEC elements = 64 bytes
	const uint64_t dims[4] = {uint64_t(width), uint64_t(n_heads), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t strides[3] = {uint64_t(width) * sizeof(T), uint64_t(n_heads) * width * sizeof(T),
				     uint64_t(n_tok) * n_heads * width * sizeof(T)};
	const uint32_t qbox[4] = {CH * VEC, HG, TT, 1}, kbox[4] = {CH * VEC, HG, TS, 1};
	CUtensorMap qmap, kmap;
	if (!encode_tmap_4d(&qmap, tmap_dtype<T>(), q, dims, strides, qbox, CU_TENSOR_MAP_SWIZZLE_64B) ||
	    !encode_tmap_4d(&kmap, tmap_dtype<T>(), k, dims, strides, kbox, CU_TENSOR_MAP_SWIZZLE_64B))
		return 1; // caller falls back to the kernel without tensor maps
	int *err = device_error_word();
	if (!err)
		return 1;
	Work wk;
	wk.ntt = (n_tok + TT - 1) / TT;
	wk.nst = (n_tok + TS - 1) / TS;
	wk.nhg = (n_heads + HG - 1) / HG;
	wk.total = (long long)bs * wk.nhg * wk.ntt * wk.nst;
	int dev = 0, sms = 0;
	L1B_CUDA(cudaGetDevice(&dev));
	L1B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
	const long long grid = wk.total < sms ? wk.total : sms;
	const size_t smem = size_t(NSTAGE) * STAGE_BYTES + 1024;
	auto kern = dense_fwd_tma_kernel<T>;
	L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	const T scale = T(-1.0 / sqrt(double(width)));
	kern<<<unsigned(grid), NTHREADS, smem, st>>>(qmap, kmap, attn, n_tok, n_heads, width, scale, wk, err);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace

// Returns L1ATTN_OK, a negative error, or 1 when this path does not apply (width rows not 16-byte
// multiples, unaligned base, no tensor-map support) and the caller should use the generic kernel.
int dense_fwd_tma_launch(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads, int width,
			 int dtype, cudaStream_t st)
{
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	if ((size_t(width) * es) % 16 != 0 || !aligned(q, 16) || !aligned(k, 16))
		return 1;
	if (dtype != L1ATTN_F32)
		return 1; // an 8 x 8 tile of doubles does not fit the register file; fp64 uses the generic kernel
	return launch<float>((const float *)q, (const float *)k, (float *)attn, bs, n_tok, n_heads, width, st);
}

} // namespace l1b
