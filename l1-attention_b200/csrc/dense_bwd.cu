// Dense L1 scores, backward:
//   d_q[b][t][h][w] =  scale * sum_s sign(q[b][t][h][w] - k[b][s][h][w]) * g[b][s][t][h]
//   d_k[b][s][h][w] = -scale * sum_t sign(q[b][t][h][w] - k[b][s][h][w]) * g[b][s][t][h]
// with sign(0) = 0.  Both are instances of
//   out[x][h][w] = scale * sum_y sign(a[x][h][w] - b[y][h][w]) * G(x, y, h)
// (d_q: a=q, b=k, G(t,s)=g[s][t];  d_k: a=k, b=q, G(s,t)=g[s][t]), so one kernel serves both
// and one launch runs the two passes side by side (blockIdx decides).  Each CTA owns an x tile,
// 8 heads and a slice of the width, keeps its `a` values and accumulators in registers and
// streams y in tiles through shared memory.  Every output element is produced by exactly one
// thread in a fixed order: no atomics, bit-reproducible.
#include <cstdlib>
#include "common.cuh"
#include "dense_bwd_tiles.h"

namespace l1b {
namespace {

constexpr int HG = 8;  // heads per CTA = lanes along heads
constexpr int LW = 4;  // lanes along the width (16-byte vectors)
constexpr int TY = 16; // y rows per shared-memory tile
constexpr int NCH = 8; // 16-byte chunks per shared row (both tiles)

template <typename T, int TM, int NWX, int NWW>
__global__ void __launch_bounds__(NWX *NWW * 32, 2)
dense_bwd_kernel(const T *__restrict__ g, const T *__restrict__ q, const T *__restrict__ k,
		 T *__restrict__ d_q, T *__restrict__ d_k, int n_tok, int n_heads, int width, T scale,
		 int vec_ok, int nxt, int nwt, int nhg, int bs)
{
	constexpr int VEC = 16 / sizeof(T);
	constexpr int TX = NWX * TM;       // x tile
	constexpr int WR = NWW * LW * VEC; // width slice per CTA
	constexpr int NT = NWX * NWW * 32;
	static_assert(TX / VEC == NCH && WR / VEC == NCH, "tile rows must be 8 chunks of 16 bytes");
	static_assert(TM % VEC == 0, "TM must be whole vectors");
	using V = Pack<T, VEC>;
	__shared__ __align__(16) V Bt[TY * HG * NCH]; // b[y][h][w chunk], chunk ^= h
	__shared__ __align__(16) V Gt[TY * HG * NCH]; // G[y][h][x chunk], chunk ^= h

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	const int lane_h = lane & 7, lane_w = lane >> 3;
	const int wx = warp % NWX, ww = warp / NWX;
	long long bid = blockIdx.x;
	const int x0 = int(bid % nxt) * TX;
	bid /= nxt;
	const int w0 = int(bid % nwt) * WR;
	bid /= nwt;
	const int h0 = int(bid % nhg) * HG;
	bid /= nhg;
	const int b = int(bid % bs);
	const int pass = int(bid / bs); // 0: d_q, 1: d_k

	const size_t row = size_t(n_heads) * width;
	const T *av = (pass == 0 ? q : k) + size_t(b) * n_tok * row;
	const T *bv = (pass == 0 ? k : q) + size_t(b) * n_tok * row;
	T *out = (pass == 0 ? d_q : d_k) + size_t(b) * n_tok * row;
	const T *gb = g + size_t(b) * n_tok * n_tok * n_heads;
	const size_t gsx = pass == 0 ? size_t(n_heads) : size_t(n_tok) * n_heads;
	const size_t gsy = pass == 0 ? size_t(n_tok) * n_heads : size_t(n_heads);

	const int h = h0 + lane_h;
	const int wv = ww * LW + lane_w; // this thread's 16-byte chunk within the slice
	const int w = w0 + wv * VEC;

	T a[TM][VEC], acc[TM][VEC];
#pragma unroll
	for (int i = 0; i < TM; i++) {
		const int x = x0 + wx * TM + i;
#pragma unroll
		for (int e = 0; e < VEC; e++) {
			const bool ok = x < n_tok && h < n_heads && w + e < width;
			a[i][e] = ok ? av[size_t(x) * row + size_t(h) * width + w + e] : T(0);
			acc[i][e] = T(0);
		}
	}

	for (int y0 = 0; y0 < n_tok; y0 += TY) {
		// b tile: [TY][HG][WR]
		for (int v = tid; v < TY * HG * NCH; v += NT) {
			const int c = v % NCH, hh = (v / NCH) % HG, y = v / (NCH * HG);
			const int gy = y0 + y, gh = h0 + hh, gw = w0 + c * VEC;
			V *dst = &Bt[(y * HG + hh) * NCH + (c ^ hh)];
			const T *src = bv + size_t(gy) * row + size_t(gh) * width + gw;
			const bool ok = gy < n_tok && gh < n_heads;
			if (ok && vec_ok && gw + VEC <= width) {
				*dst = *reinterpret_cast<const V *>(src);
			} else {
				V z;
#pragma unroll
				for (int e = 0; e < VEC; e++)
					z.v[e] = (ok && gw + e < width) ? src[e] : T(0);
				*dst = z;
			}
		}
		// G tile: [TY][HG][TX], heads fastest in global memory
		T *Gs = reinterpret_cast<T *>(Gt);
		for (int idx = tid; idx < TY * HG * TX; idx += NT) {
			const int hh = idx % HG;
			int x, y;
			if (pass == 0) { // x = t is the contiguous token axis of g
				x = (idx / HG) % TX;
				y = idx / (HG * TX);
			} else { // y = t is
				y = (idx / HG) % TY;
				x = idx / (HG * TY);
			}
			const int gx = x0 + x, gy = y0 + y, gh = h0 + hh;
			T val = T(0);
			if (gx < n_tok && gy < n_tok && gh < n_heads)
				val = gb[size_t(gx) * gsx + size_t(gy) * gsy + gh];
			Gs[((y * HG + hh) * NCH + ((x / VEC) ^ hh)) * VEC + (x % VEC)] = val;
		}
		__syncthreads();
#pragma unroll 4
		for (int y = 0; y < TY; y++) {
			const V bvec = Bt[(y * HG + lane_h) * NCH + (wv ^ lane_h)];
			T gv[TM];
#pragma unroll
			for (int m = 0; m < TM / VEC; m++) {
				const V t = Gt[(y * HG + lane_h) * NCH + ((wx * TM / VEC + m) ^ lane_h)];
#pragma unroll
				for (int e = 0; e < VEC; e++)
					gv[m * VEC + e] = t.v[e];
			}
#pragma unroll
			for (int i = 0; i < TM; i++)
#pragma unroll
				for (int e = 0; e < VEC; e++)
					acc[i][e] += sign_apply(a[i][e] - bvec.v[e], gv[i]);
		}
		__syncthreads();
	}

	if (h < n_heads) {
#pragma unroll
		for (int i = 0; i < TM; i++) {
			const int x = x0 + wx * TM + i;
			if (x >= n_tok)
				continue;
			T *dst = out + size_t(x) * row + size_t(h) * width + w;
			if (vec_ok && w + VEC <= width) {
				V o;
#pragma unroll
				for (int e = 0; e < VEC; e++)
					o.v[e] = acc[i][e] * scale;
				*reinterpret_cast<V *>(dst) = o;
			} else {
#pragma unroll
				for (int e = 0; e < VEC; e++)
					if (w + e < width)
						dst[e] = acc[i][e] * scale;
			}
		}
	}
}

template <typename T, int TM, int NWX, int NWW>
int launch(const T *g, const T *q, const T *k, T *d_q, T *d_k, int bs, int n_tok, int n_heads, int width,
	   cudaStream_t st)
{
	constexpr int VEC = 16 / sizeof(T);
	constexpr int TX = NWX * TM, WR = NWW * LW * VEC;
	const int nxt = (n_tok + TX - 1) / TX, nwt = (width + WR - 1) / WR, nhg = (n_heads + HG - 1) / HG;
	const long long nblk = 2LL * bs * nhg * nwt * nxt;
	if (nblk > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	const int vec_ok = (width % VEC == 0) && aligned(q, 16) && aligned(k, 16) && aligned(d_q, 16) && aligned(d_k, 16);
	const T scale = T(-1.0 / sqrt(double(width)));
	dense_bwd_kernel<T, TM, NWX, NWW><<<unsigned(nblk), NWX * NWW * 32, 0, st>>>(
		g, q, k, d_q, d_k, n_tok, n_heads, width, scale, vec_ok, nxt, nwt, nhg, bs);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace

size_t dense_bwd_scratch_bytes(int bs, int n_tok, int n_heads, int width, int dtype)
{
	if (dtype != L1ATTN_F32 || bs <= 0 || n_tok <= 0 || n_heads <= 0 || width <= 0)
		return 16;
	return bwd_scratch_layout(bs, n_tok, n_heads, width).bytes; // tie flags, tie header, tie list, shares of d_k
}

int dense_bwd_launch(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, void *scratch, int bs,
		     int n_tok, int n_heads, int width, int dtype, cudaStream_t st)
{
	if (bs == 0 || n_tok == 0 || n_heads == 0 || width == 0)
		return L1ATTN_OK;
	static const bool no_tma = getenv("L1ATTN_NO_TMA") != nullptr; // debugging aid: force the generic kernel
	static const bool no_sv = getenv("L1ATTN_NO_SV") != nullptr;   // debugging aid: force the two-pass kernel
	if (!no_tma) {
		// With scratch the tie detector runs first: it lists every exact tie q == k (and marks tiles, for the case
		// that the list overflows -- a device-side fact, no host round trip).  Then the single-visit kernel computes
		// both gradients with the compare form and the listed terms are repaired afterwards.  If the list overflowed
		// that kernel returns at once and the two-pass kernel, gated on the same word, runs its exact loop where
		// flagged tiles meet.  Without scratch (or when the detector does not apply) the two-pass kernel runs every
		// tile with the exact loop.
		unsigned char *flags = nullptr;
		const int *tie_hdr = nullptr;
		int sv = 0;
		if (scratch && dtype == L1ATTN_F32 && width % 4 == 0 && n_heads % 4 == 0 && aligned(scratch, 256)) {
			const int trc = dense_ties_launch((const float *)q, (const float *)k, (unsigned char *)scratch, bs, n_tok,
							  n_heads, width, st);
			if (trc < 0)
				return trc;
			if (trc == 0) {
				const BwdScratchLayout sl = bwd_scratch_layout(bs, n_tok, n_heads, width);
				unsigned char *sc = (unsigned char *)scratch;
				flags = sc + sl.flags;
				tie_hdr = (const int *)(sc + sl.hdr);
				// Both fast kernels are persistent with equal-sized work items, so the last wave of items decides how
				// full the GPU stays: the single-visit kernel (4 heads x 32 columns x 128 query rows per item, ~8 %
				// faster per term) runs unless its item count leaves the SMs markedly emptier than the two-pass
				// kernel's (8 heads x 64 columns x 32 rows per item and gradient) would.
				int dev = 0, sms = 148;
				(void)cudaGetDevice(&dev);
				(void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
				auto fill = [&](double items) { return bwd_wave_fill(items, sms); };
				const double it_sv = double(bs) * ((n_heads + 3) / 4) * ((width + 31) / 32) * ((n_tok + 127) / 128) * sl.ns;
				const double it_tp = 2.0 * bs * ((n_heads + 7) / 8) * ((width + 63) / 64) * ((n_tok + 31) / 32);
				// (and an item of either kernel is only as busy as its head group is full: 4 heads leave half of an
				// 8-head item's lanes idle)
				const double hf_sv = double(n_heads) / (4.0 * ((n_heads + 3) / 4)), hf_tp = double(n_heads) / (8.0 * ((n_heads + 7) / 8));
				if (!no_sv && 1.08 * fill(it_sv) * hf_sv >= fill(it_tp) * hf_tp) {
					const int frc = dense_bwd_sv_launch(d_attn, q, k, d_q, d_k, tie_hdr, sc + sl.part, sl.ns > 1 ? sc + sl.dqpart : nullptr,
									    sl.ns, bs, n_tok, n_heads, width, dtype, st);
					if (frc < 0)
						return frc;
					sv = frc == 0;
				}
			}
		}
		const int rc = dense_bwd_tma_launch(d_attn, q, k, d_q, d_k, bs, n_tok, n_heads, width, dtype, flags, tie_hdr, sv, st);
		if (rc < 0)
			return rc;
		if (rc == 0)
			return tie_hdr ? dense_tiefix_launch(d_attn, d_q, d_k, (const unsigned char *)scratch, bs, n_tok, n_heads,
							     width, sv ? -1 : 1, st)
				       : L1ATTN_OK;
		if (sv)
			return L1ATTN_ERR_CUDA; // cannot happen: both fast kernels accept the same shapes and alignments
	}
	if (dtype == L1ATTN_F32)
		return launch<float, 8, 4, 2>((const float *)d_attn, (const float *)q, (const float *)k, (float *)d_q,
					      (float *)d_k, bs, n_tok, n_heads, width, st);
	return launch<double, 4, 4, 2>((const double *)d_attn, (const double *)q, (const double *)k, (double *)d_q,
				       (double *)d_k, bs, n_tok, n_heads, width, st);
}

} // namespace l1b
