// Dense L1 scores, forward:  attn[b][s][t][h] = scale * sum_w |q[b][t][h][w] - k[b][s][h][w]|.
//
// One CTA owns a (query tile, key tile) for a group of 8 heads of one batch item and walks the
// width in chunks of 64 bytes per (token, head) row, double-buffered in shared memory with
// cp.async.  The 8 heads are spread over 8 adjacent lanes, so that
//   * every output store of a warp writes whole 32-byte sectors (the output has heads innermost);
//   * no transpose of q/k is needed (the reference makes [b,h,t,w] copies first);
// and each thread keeps a TM x TN register tile of (query, key) pairs of its head, so one
// 16-byte shared-memory read feeds TN (resp. TM) x 4 abs-difference terms.
// Shared memory is XOR-swizzled on the 16-byte chunk index so the 8 head-lanes hit 8 different
// bank groups.
#include <cstdlib>
#include "common.cuh"

namespace l1b {
namespace {

constexpr int HG = 8; // heads per CTA = lanes along heads
constexpr int LT = 4; // lanes along the query axis
constexpr int CH = 4; // 16-byte chunks per (token, head) row per stage

template <typename T, int TM, int TN, int NWARP>
__global__ void __launch_bounds__(NWARP * 32, sizeof(T) == 4 ? 2 : 1)
dense_fwd_kernel(const T *__restrict__ q, const T *__restrict__ k, T *__restrict__ attn,
		 int n_tok, int n_heads, int width, T scale, int vec_ok, int ntt, int nst, int nhg)
{
	constexpr int VEC = 16 / sizeof(T);
	constexpr int WC = CH * VEC;   // width elements per stage
	constexpr int TT = LT * TM;    // query tile
	constexpr int TS = NWARP * TN; // key tile
	constexpr int NT = NWARP * 32;
	constexpr int QV = TT * HG * CH, KV = TS * HG * CH; // 16-byte vectors per stage
	using V = Pack<T, VEC>;
	extern __shared__ __align__(16) unsigned char smem_raw[];
	V *smem = reinterpret_cast<V *>(smem_raw); // [2][QV + KV]

	const int tid = threadIdx.x;
	const int lane = tid & 31, warp = tid >> 5;
	const int lane_h = lane & 7, lane_t = lane >> 3;
	long long bid = blockIdx.x;
	const int t0 = int(bid % ntt) * TT;
	bid /= ntt;
	const int s0 = int(bid % nst) * TS;
	bid /= nst;
	const int h0 = int(bid % nhg) * HG;
	const int b = int(bid / nhg);

	const size_t row = size_t(n_heads) * width; // elements per token
	const T *qb = q + size_t(b) * n_tok * row;
	const T *kb = k + size_t(b) * n_tok * row;

	auto load_stage = [&](int stage, int w0) {
		V *base = smem + stage * (QV + KV);
		for (int v = tid; v < QV + KV; v += NT) {
			const bool is_k = v >= QV;
			const int vv = is_k ? v - QV : v;
			const int c = vv % CH, h = (vv / CH) % HG, tok = vv / (CH * HG);
			const int gt = (is_k ? s0 : t0) + tok, gh = h0 + h, gw = w0 + c * VEC;
			V *dst = base + (is_k ? QV : 0) + (tok * HG + h) * CH + (c ^ ((h >> 1) & 3));
			const T *src = (is_k ? kb : qb) + size_t(gt) * row + size_t(gh) * width + gw;
			const bool tok_ok = gt < n_tok && gh < n_heads;
			if (tok_ok && vec_ok && gw + VEC <= width) {
				cp_async16(dst, src);
			} else {
				V z;
#pragma unroll
				for (int e = 0; e < VEC; e++)
					z.v[e] = (tok_ok && gw + e < width) ? src[e] : T(0);
				*dst = z;
			}
		}
	};

	T acc[TM][TN];
#pragma unroll
	for (int i = 0; i < TM; i++)
#pragma unroll
		for (int j = 0; j < TN; j++)
			acc[i][j] = T(0);

	const int sw = (lane_h >> 1) & 3;
	const int nchunk = (width + WC - 1) / WC;
	load_stage(0, 0);
	cp_async_commit();
	for (int ci = 0; ci < nchunk; ci++) {
		if (ci + 1 < nchunk) {
			load_stage((ci + 1) & 1, (ci + 1) * WC);
			cp_async_commit();
			cp_async_wait<1>();
		} else {
			cp_async_wait<0>();
		}
		__syncthreads();
		const V *Q = smem + (ci & 1) * (QV + KV);
		const V *K = Q + QV;
#pragma unroll
		for (int c = 0; c < CH; c++) {
			const int pc = c ^ sw;
			V kv[TN];
#pragma unroll
			for (int j = 0; j < TN; j++)
				kv[j] = K[((warp * TN + j) * HG + lane_h) * CH + pc];
#pragma unroll
			for (int i = 0; i < TM; i++) {
				const V qv = Q[((lane_t + LT * i) * HG + lane_h) * CH + pc];
#pragma unroll
				for (int j = 0; j < TN; j++)
#pragma unroll
					for (int e = 0; e < VEC; e++)
						acc[i][j] += absdiff(qv.v[e], kv[j].v[e]);
			}
		}
		__syncthreads();
	}

	const int h = h0 + lane_h;
	if (h < n_heads) {
		T *ab = attn + size_t(b) * n_tok * n_tok * n_heads;
#pragma unroll
		for (int j = 0; j < TN; j++) {
			const int s = s0 + warp * TN + j;
			if (s >= n_tok)
				continue;
#pragma unroll
			for (int i = 0; i < TM; i++) {
				const int t = t0 + lane_t + LT * i;
				if (t < n_tok)
					ab[(size_t(s) * n_tok + t) * n_heads + h] = acc[i][j] * scale;
			}
		}
	}
}

template <typename T, int TM, int TN, int NWARP>
int launch(const T *q, const T *k, T *attn, int bs, int n_tok, int n_heads, int width, cudaStream_t st)
{
	constexpr int VEC = 16 / sizeof(T);
	constexpr int TT = LT * TM, TS = NWARP * TN;
	const int ntt = (n_tok + TT - 1) / TT, nst = (n_tok + TS - 1) / TS, nhg = (n_heads + HG - 1) / HG;
	const long long nblk = (long long)bs * nhg * ntt * nst;
	if (nblk > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	const size_t smem = 2 * size_t(TT + TS) * HG * CH * 16;
	auto kern = dense_fwd_kernel<T, TM, TN, NWARP>;
	L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	const int vec_ok = (width % VEC == 0) && aligned(q, 16) && aligned(k, 16);
	const T scale = T(-1.0 / sqrt(double(width)));
	kern<<<unsigned(nblk), NWARP * 32, smem, st>>>(q, k, attn, n_tok, n_heads, width, scale, vec_ok, ntt, nst, nhg);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace

int dense_fwd_launch(const void *q, const void *k, void *attn, int bs, int n_tok, int n_heads, int width,
		     int dtype, cudaStream_t st)
{
	if (bs == 0 || n_tok == 0 || n_heads == 0)
		return L1ATTN_OK;
	static const bool no_tma = getenv("L1ATTN_NO_TMA") != nullptr; // debugging aid: force the generic kernel
	if (!no_tma) {
		const int rc = dense_fwd_tma_launch(q, k, attn, bs, n_tok, n_heads, width, dtype, st);
		if (rc <= 0)
			return rc;
	}
	if (dtype == L1ATTN_F32)
		return launch<float, 8, 8, 8>((const float *)q, (const float *)k, (float *)attn, bs, n_tok, n_heads, width, st);
	return launch<double, 4, 4, 8>((const double *)q, (const double *)k, (double *)attn, bs, n_tok, n_heads, width, st);
}

} // namespace l1b
