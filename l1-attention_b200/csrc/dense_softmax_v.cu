// Fused consumer of the dense L1 scores: softmax over the source tokens and the value product,
// without ever writing the [bs, n_tok, n_tok, n_heads] score tensor.
//
//   x[b][s][t][h]  = scale * sum_w |q[b][t][h][w] - k[b][s][h][w]|          scale = -1/sqrt(width)
//   a              = softmax of x over s                                    (mode SOFTMAX)
//                  | exp(x) / (1 + sum_s exp(x))   "one more all-zero row"  (mode SOFTMAX_PLUS_ONE)
//                  | exp(x)                                                 (mode EXP)
//   vo[b][t][h][:] = sum_s a[b][s][t][h] * v[b][s][h][:]
//
// This is what every dense caller of the reference does right after L1Attn
// (README.md:64-66: F.softmax(a, 1) then einsum 'bsdh,bshw->bdhw'); the "+1" forms are the dense
// equivalents of the sparse operator's normalisation (python/l1attn_sparse.py:491-502).
//
// Two kernels:
//   * softmax_v_kernel: any shape, fp32/fp64.  One CTA per (b, t, h) keeps the n_tok scores of its row
//     in shared memory: scores, max, exp/sum, value product, each in a fixed order.
//   * softmax_v_tma_kernel (fp32, width 32..128 in steps of 32, v_width 32/64/128): one CTA per
//     (b, h, tile of 64 or 128 query rows) streams the keys and values of its head in tiles of 64
//     through a TMA ring and keeps running max / sum / output rows in registers (online softmax).
#include <math.h>
#include <stdlib.h>
#include "common.cuh"
#include "tma.cuh"

namespace l1b {
namespace {

// ------------------------------------------------------------------------------------------------
// generic kernel
// ------------------------------------------------------------------------------------------------
constexpr int GEN_NT = 128;

template <typename T> __device__ __forceinline__ T block_reduce(T v, T *red, bool is_max)
{
	// fixed tree: lanes by shuffle, then warp results in warp order by thread 0
#pragma unroll
	for (int o = 16; o > 0; o >>= 1) {
		const T u = __shfl_xor_sync(0xffffffffu, v, o);
		v = is_max ? (u > v ? u : v) : v + u;
	}
	__syncthreads(); // red may still be read from the previous reduction
	if ((threadIdx.x & 31) == 0)
		red[threadIdx.x >> 5] = v;
	__syncthreads();
	T r = red[0];
	for (int i = 1; i < GEN_NT / 32; i++)
		r = is_max ? (red[i] > r ? red[i] : r) : r + red[i];
	return r;
}

template <typename T>
__global__ void __launch_bounds__(GEN_NT)
softmax_v_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ vo,
		 T *__restrict__ lse, int n_tok, int n_heads, int width, int v_width, T scale, int mode)
{
	extern __shared__ __align__(16) unsigned char gsm[];
	T *sc = reinterpret_cast<T *>(gsm); // [n_tok] scores, then weights
	T *qrow = sc + n_tok;               // [width]
	T *red = qrow + width;              // [GEN_NT / 32]
	unsigned r = blockIdx.x;
	const int h = int(r % unsigned(n_heads));
	r /= unsigned(n_heads);
	const int t = int(r % unsigned(n_tok));
	const int b = int(r / unsigned(n_tok));
	const size_t row = size_t(n_heads) * width, vrow = size_t(n_heads) * v_width;
	const T *qp = q + (size_t(b) * n_tok + t) * row + size_t(h) * width;
	const T *kb = k + size_t(b) * n_tok * row + size_t(h) * width;
	const T *vb = v + size_t(b) * n_tok * vrow + size_t(h) * v_width;
	for (int w = threadIdx.x; w < width; w += GEN_NT)
		qrow[w] = qp[w];
	__syncthreads();
	T lmax = -INFINITY;
	for (int s = threadIdx.x; s < n_tok; s += GEN_NT) {
		const T *kp = kb + size_t(s) * row;
		T acc = T(0);
		for (int w = 0; w < width; w++)
			acc += absdiff(qrow[w], kp[w]);
		const T x = acc * scale;
		sc[s] = x;
		lmax = x > lmax ? x : lmax;
	}
	T m = T(0); // the "+1" and exp forms do not shift (the reference's sparse operator does not either)
	if (mode == L1ATTN_SV_SOFTMAX)
		m = block_reduce(lmax, red, true);
	T lsum = T(0);
	for (int s = threadIdx.x; s < n_tok; s += GEN_NT) {
		const T e = exp_t(sc[s] - m);
		sc[s] = e;
		lsum += e;
	}
	T denom = block_reduce(lsum, red, false); // also publishes sc[] to every thread
	if (mode == L1ATTN_SV_SOFTMAX_PLUS_ONE)
		denom += T(1);
	if (mode == L1ATTN_SV_EXP)
		denom = T(1);
	if (lse && threadIdx.x == 0) // weight of (s, t) = exp(x - lse)
		lse[(size_t(b) * n_tok + t) * n_heads + h] = m + log(denom);
	T *op = vo + (size_t(b) * n_tok + t) * vrow + size_t(h) * v_width;
	for (int c = threadIdx.x; c < v_width; c += GEN_NT) {
		T o = T(0);
		for (int s = 0; s < n_tok; s++)
			o += sc[s] * vb[size_t(s) * vrow + c];
		op[c] = o / denom;
	}
}

template <typename T>
int launch_generic(const T *q, const T *k, const T *v, T *vo, T *lse, int bs, int n_tok, int n_heads, int width,
		   int v_width, int mode, cudaStream_t st)
{
	const long long grid = (long long)bs * n_tok * n_heads;
	const size_t smem = (size_t(n_tok) + width + GEN_NT / 32) * sizeof(T);
	if (grid > 0x7fffffffLL || smem > 200 * 1024)
		return L1ATTN_ERR_SHAPE;
	auto kern = softmax_v_kernel<T>;
	L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	kern<<<unsigned(grid), GEN_NT, smem, st>>>(q, k, v, vo, lse, n_tok, n_heads, width, v_width,
						    T(-1.0 / sqrt(double(width))), mode);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

// ------------------------------------------------------------------------------------------------
// TMA kernel (fp32)
// ------------------------------------------------------------------------------------------------
// CTA = NW warps = 2 NW half-warps.  Half-warp `tg` owns TI query rows (t = i*2*NW + tg) and is
// self-contained: for every key tile its 16 lanes first each compute TI x 4 scores (keys
// s = j*16 + lane), reduce the row maxima and sums by shuffles, park the weights in a private slice
// of shared memory, and then each accumulate TI x NV output values (lane = value columns
// [lane*NV, lane*NV+NV)).  Only the key/value ring is shared by the CTA.
// Shared operand rows are 128 bytes (one 32-float slice of the width per TMA box, 128-byte swizzle),
// so the 16 lanes of a half-warp read 16 different key rows without bank conflicts.
constexpr int TS = 64;     // keys per ring stage
constexpr int PP = TS + 4; // row pitch (floats) of the weight tile: the two half-warps of a warp land on different banks
constexpr int MAX_STAGE = 3;

struct SvShape {
	int n_tok, n_heads, nwb, nstage, ntt, mode;
	float scale;
};

template <int NV, int TI, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
softmax_v_tma_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
		     const __grid_constant__ CUtensorMap vmap, float *__restrict__ vo, float *__restrict__ lse, SvShape sh,
		     int *err)
{
	constexpr int TT = 2 * NW * TI; // query rows of the CTA: a half-warp owns TI of them (t = i*2*NW + tg)
	constexpr int NTH = NW * 32;
	constexpr int VW = 16 * NV; // v_width
	constexpr int V_BYTES = TS * VW * 4;
	extern __shared__ __align__(1024) unsigned char smem_raw[];
	unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
	__shared__ __align__(8) uint64_t q_bar, full_bar[MAX_STAGE], empty_bar[MAX_STAGE];
	const int q_bytes = sh.nwb * TT * 128, k_bytes = sh.nwb * TS * 128, stage_bytes = k_bytes + V_BYTES;
	unsigned char *Qs = base;
	unsigned char *stages = base + q_bytes;
	float *Ps = reinterpret_cast<float *>(stages + size_t(sh.nstage) * stage_bytes);

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	unsigned r = blockIdx.x;
	const int t0 = int(r % unsigned(sh.ntt)) * TT;
	r /= unsigned(sh.ntt);
	const int h = int(r % unsigned(sh.n_heads));
	const int b = int(r / unsigned(sh.n_heads));
	const int ns = (sh.n_tok + TS - 1) / TS;

	if (tid == 0) {
		mbar_init(&q_bar, 1);
		for (int s = 0; s < MAX_STAGE; s++) {
			mbar_init(&full_bar[s], 1);
			mbar_init(&empty_bar[s], NTH / 32);
		}
		mbar_fence_init();
	}
	__syncthreads();

	// key/value tile m goes to stage m % nstage; the caller has made sure the stage is free
	auto load_tile = [&](int m) {
		const int st = m % sh.nstage;
		unsigned char *dst = stages + size_t(st) * stage_bytes;
		mbar_expect_tx(&full_bar[st], uint32_t(stage_bytes));
		for (int wb = 0; wb < sh.nwb; wb++)
			tma_load_4d(dst + wb * TS * 128, &kmap, &full_bar[st], wb * 32, h, m * TS, b);
		tma_load_4d(dst + k_bytes, &vmap, &full_bar[st], 0, h, m * TS, b);
	};
	if (tid == 0) {
		mbar_expect_tx(&q_bar, uint32_t(q_bytes));
		for (int wb = 0; wb < sh.nwb; wb++)
			tma_load_4d(Qs + wb * TT * 128, &qmap, &q_bar, wb * 32, h, t0, b);
		for (int m = 0; m < sh.nstage - 1 && m < ns; m++)
			load_tile(m);
	}

	const int sg = lane & 15, tg = warp * 2 + (lane >> 4);
	const bool softmax = sh.mode == L1ATTN_SV_SOFTMAX;
	float o[TI][NV], mrow[TI], lrow[TI];
#pragma unroll
	for (int i = 0; i < TI; i++) {
		mrow[i] = softmax ? -INFINITY : 0.f;
		lrow[i] = sh.mode == L1ATTN_SV_SOFTMAX_PLUS_ONE ? 1.f : 0.f; // the extra all-zero row weighs exp(0)
#pragma unroll
		for (int e = 0; e < NV; e++)
			o[i][e] = 0.f;
	}
	bool dead = false;
	if (!mbar_wait(&q_bar, 0, err))
		dead = true;
	float *Pw = Ps + tg * PP; // weight rows of this half-warp: row i at Pw + i*16*PP

	for (int m = 0; m < ns; m++) {
		// one lane asks for the tile that will be needed nstage-1 tiles from now; its stage held tile
		// m-1, which every warp must have released (the duty rotates so that no warp is always late)
		if (warp == m % NW && lane == 0 && m + sh.nstage - 1 < ns && !dead) {
			const int mm = m + sh.nstage - 1;
			if (mbar_wait(&empty_bar[mm % sh.nstage], ((unsigned(mm) / unsigned(sh.nstage)) & 1u) ^ 1u, err))
				load_tile(mm);
			else
				dead = true;
		}
		__syncwarp();
		const int st = m % sh.nstage;
		if (!dead && !mbar_wait(&full_bar[st], (unsigned(m) / unsigned(sh.nstage)) & 1u, err))
			dead = true; // keep walking without waiting; the error word reports the failure
		const unsigned char *Ks = stages + size_t(st) * stage_bytes;
		const float *Vs = reinterpret_cast<const float *>(Ks + k_bytes);

		// ---- scores of TI query rows x 4 keys
		float acc[TI][4];
#pragma unroll
		for (int i = 0; i < TI; i++)
#pragma unroll
			for (int j = 0; j < 4; j++)
				acc[i][j] = 0.f;
		for (int wb = 0; wb < sh.nwb; wb++) {
			const ulonglong2 *Qb = reinterpret_cast<const ulonglong2 *>(Qs + wb * TT * 128);
			const ulonglong2 *Kb = reinterpret_cast<const ulonglong2 *>(Ks + wb * TS * 128);
#pragma unroll 2
			for (int c = 0; c < 8; c++) {
				ulonglong2 kv[4];
#pragma unroll
				for (int j = 0; j < 4; j++) // row j*16+sg, chunk c ^ (row & 7)
					kv[j] = Kb[(j * 16 + sg) * 8 + (c ^ (sg & 7))];
#pragma unroll
				for (int i = 0; i < TI; i++) {
					const ulonglong2 qv = Qb[(i * (2 * NW) + tg) * 8 + (c ^ (tg & 7))];
#pragma unroll
					for (int j = 0; j < 4; j++) {
						unsigned long long d0, d1;
						float x0, x1, x2, x3;
						asm("sub.f32x2 %0, %1, %2;" : "=l"(d0) : "l"(qv.x), "l"(kv[j].x));
						asm("sub.f32x2 %0, %1, %2;" : "=l"(d1) : "l"(qv.y), "l"(kv[j].y));
						asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(d0));
						asm("mov.b64 {%0, %1}, %2;" : "=f"(x2), "=f"(x3) : "l"(d1));
						acc[i][j] += fabsf(x0);
						acc[i][j] += fabsf(x1);
						acc[i][j] += fabsf(x2);
						acc[i][j] += fabsf(x3);
					}
				}
			}
		}

		// ---- weights: running max / sum per query row, rescale of the output rows
#pragma unroll
		for (int i = 0; i < TI; i++) {
			float x[4], mx = -INFINITY;
#pragma unroll
			for (int j = 0; j < 4; j++) {
				x[j] = (m * TS + j * 16 + sg < sh.n_tok) ? acc[i][j] * sh.scale : -INFINITY; // keys past the end weigh nothing
				mx = fmaxf(mx, x[j]);
			}
			float mnew = mrow[i];
			if (softmax) {
#pragma unroll
				for (int d = 8; d > 0; d >>= 1)
					mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
				mnew = fmaxf(mrow[i], mx);
			}
			float ps = 0.f;
#pragma unroll
			for (int j = 0; j < 4; j++) {
				const float p = expf(x[j] - mnew);
				Pw[i * (2 * NW) * PP + j * 16 + sg] = p;
				ps += p;
			}
#pragma unroll
			for (int d = 8; d > 0; d >>= 1)
				ps += __shfl_xor_sync(0xffffffffu, ps, d);
			if (softmax) {
				const float alpha = expf(mrow[i] - mnew); // exp(-inf) = 0 on the first tile
				lrow[i] = lrow[i] * alpha + ps;
#pragma unroll
				for (int e = 0; e < NV; e++)
					o[i][e] *= alpha;
				mrow[i] = mnew;
			} else {
				lrow[i] += ps;
			}
		}
		__syncwarp();

		// ---- output rows += weights x values; this lane owns value columns [sg*NV, sg*NV+NV)
#pragma unroll 2
		for (int s4 = 0; s4 < TS / 4; s4++) {
			float4 p[TI];
#pragma unroll
			for (int i = 0; i < TI; i++)
				p[i] = *reinterpret_cast<const float4 *>(Pw + i * (2 * NW) * PP + s4 * 4);
#pragma unroll
			for (int ss = 0; ss < 4; ss++) {
				float vv[NV];
				const float *vp = Vs + (s4 * 4 + ss) * VW + sg * NV;
				if (NV == 2) {
					const float2 t2 = *reinterpret_cast<const float2 *>(vp);
					vv[0] = t2.x;
					vv[1] = t2.y;
				} else {
#pragma unroll
					for (int e = 0; e < NV; e += 4) {
						const float4 t4 = *reinterpret_cast<const float4 *>(vp + e);
						vv[e] = t4.x;
						vv[(e + 1) % NV] = t4.y;
						vv[(e + 2) % NV] = t4.z;
						vv[(e + 3) % NV] = t4.w;
					}
				}
#pragma unroll
				for (int i = 0; i < TI; i++) {
					const float pi = ss == 0 ? p[i].x : ss == 1 ? p[i].y : ss == 2 ? p[i].z : p[i].w;
#pragma unroll
					for (int e = 0; e < NV; e++)
						o[i][e] = fmaf(pi, vv[e], o[i][e]);
				}
			}
		}
		__syncwarp(); // the weight slice is rewritten by the next tile
		if (lane == 0)
			mbar_arrive(&empty_bar[st]);
	}

	const size_t vrow = size_t(sh.n_heads) * VW;
#pragma unroll
	for (int i = 0; i < TI; i++) {
		const int t = t0 + i * (2 * NW) + tg;
		if (t >= sh.n_tok)
			continue;
		const float inv = sh.mode == L1ATTN_SV_EXP ? 1.f : 1.f / lrow[i];
		if (lse && sg == 0) // weight of (s, t) = exp(x - lse)
			lse[(size_t(b) * sh.n_tok + t) * sh.n_heads + h] = sh.mode == L1ATTN_SV_EXP ? 0.f : mrow[i] + logf(lrow[i]);
		float *op = vo + (size_t(b) * sh.n_tok + t) * vrow + size_t(h) * VW + sg * NV;
#pragma unroll
		for (int e = 0; e < NV; e++)
			op[e] = o[i][e] * inv;
	}
}

template <int NV, int TI, int NW>
int launch_tma(const float *q, const float *k, const float *v, float *vo, float *lse, int bs, int n_tok, int n_heads,
	       int width, int mode, int nstage, size_t smem, cudaStream_t st)
{
	constexpr int TT = 2 * NW * TI, VW = 16 * NV, NTH = NW * 32;
	const uint64_t dims[4] = {uint64_t(width), uint64_t(n_heads), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t str[3] = {uint64_t(width) * 4, uint64_t(n_heads) * width * 4, uint64_t(n_tok) * n_heads * width * 4};
	const uint64_t vdims[4] = {uint64_t(VW), uint64_t(n_heads), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t vstr[3] = {uint64_t(VW) * 4, uint64_t(n_heads) * VW * 4, uint64_t(n_tok) * n_heads * VW * 4};
	const uint32_t qbox[4] = {32, 1, TT, 1}, kbox[4] = {32, 1, TS, 1}, vbox[4] = {VW, 1, TS, 1};
	CUtensorMap qmap, kmap, vmap;
	if (!encode_tmap_4d(&qmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, q, dims, str, qbox, CU_TENSOR_MAP_SWIZZLE_128B) ||
	    !encode_tmap_4d(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, k, dims, str, kbox, CU_TENSOR_MAP_SWIZZLE_128B) ||
	    !encode_tmap_4d(&vmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, v, vdims, vstr, vbox, CU_TENSOR_MAP_SWIZZLE_NONE))
		return 1;
	int *err = device_error_word();
	if (!err)
		return 1;
	SvShape sh;
	sh.n_tok = n_tok;
	sh.n_heads = n_heads;
	sh.nwb = width / 32;
	sh.nstage = nstage;
	sh.ntt = (n_tok + TT - 1) / TT;
	sh.mode = mode;
	sh.scale = float(-1.0 / sqrt(double(width)));
	const long long grid = (long long)bs * n_heads * sh.ntt;
	if (grid > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	auto kern = softmax_v_tma_kernel<NV, TI, NW>;
	L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	kern<<<unsigned(grid), NTH, smem, st>>>(qmap, kmap, vmap, vo, lse, sh, err);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

// shared memory of one CTA: query tile + ring + weight tile + alignment slack
size_t sv_smem(int nwb, int nv, int tt_rows, int nstage)
{
	const size_t tt = size_t(tt_rows);
	return size_t(nwb) * tt * 128 + size_t(nstage) * (size_t(nwb) * TS * 128 + size_t(TS) * nv * 64) + tt * PP * 4 + 1024;
}

// Returns L1ATTN_OK, a negative error, or 1 when the shape is outside this kernel's set.
int softmax_v_tma(const float *q, const float *k, const float *v, float *vo, float *lse, int bs, int n_tok, int n_heads,
		  int width, int v_width, int mode, cudaStream_t st)
{
	if (width % 32 != 0 || width > 128 || (v_width != 32 && v_width != 64 && v_width != 128))
		return 1;
	for (const void *p : {(const void *)q, (const void *)k, (const void *)v, (const void *)vo})
		if (!aligned(p, 16))
			return 1;
	const int nwb = width / 32, nv = v_width / 16;
	const size_t limit = 227 * 1024 - 256; // per-CTA maximum minus the static barriers
	// (rows per half-warp, warps): 4 x 16 and 8 x 8 give 128-row CTAs, 4 x 8 a 64-row CTA for the widest rows.
	// Sixteen warps of 128 registers measured 7 % faster than eight of 168 (four warps per scheduler hide
	// the shared-memory and arithmetic latencies); with 128 value columns the thread state does not fit 128 registers.
	const bool nw16 = nv <= 4;
	const int cand[2][2] = {{nw16 ? 4 : 8, nw16 ? 16 : 8}, {4, 8}};
	int ti = 0, nw = 0, nstage = 0;
	for (const auto &c : cand) {
		for (int cand_ns : {3, 2})
			if (!ti && sv_smem(nwb, nv, 2 * c[0] * c[1], cand_ns) <= limit) {
				ti = c[0];
				nw = c[1];
				nstage = cand_ns;
			}
	}
	if (!ti)
		return 1;
	const size_t smem = sv_smem(nwb, nv, 2 * ti * nw, nstage);
#define L1B_SV(NV_, TI_, NW_)                       \
	if (nv == NV_ && ti == TI_ && nw == NW_)    \
		return launch_tma<NV_, TI_, NW_>(q, k, v, vo, lse, bs, n_tok, n_heads, width, mode, nstage, smem, st);
	L1B_SV(2, 8, 8) L1B_SV(4, 8, 8) L1B_SV(8, 8, 8) L1B_SV(2, 4, 8) L1B_SV(4, 4, 8) L1B_SV(8, 4, 8)
	L1B_SV(2, 4, 16) L1B_SV(4, 4, 16) L1B_SV(8, 4, 16)
#undef L1B_SV
	return 1;
}

// ------------------------------------------------------------------------------------------------
// backward, step 1: score gradients dx and value gradients dv
// ------------------------------------------------------------------------------------------------
// With lse[b][t][h] from the forward (weight of (s, t) = exp(x - lse)) and
// delta[b][t][h] = <dvo[b][t][h][:], vo[b][t][h][:]> (zeros for the exp form):
//   p  = exp(x[b][s][t][h] - lse[b][t][h])
//   dx[b][s][t][h] = p * (<v[b][s][h][:], dvo[b][t][h][:]> - delta[b][t][h])
//   dv[b][s][h][:] = sum_t p * dvo[b][t][h][:]
// dx has the layout of the dense operator's d_attn, so l1attn_dense_bwd(dx, q, k) finishes the job
// (d_q, d_k).  Callers bound memory by running a few batch items at a time.

template <typename T>
__global__ void __launch_bounds__(GEN_NT)
softmax_v_bwd_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v, const T *__restrict__ dvo,
		     const T *__restrict__ lse, const T *__restrict__ delta, T *__restrict__ dx, T *__restrict__ dv,
		     int n_tok, int n_heads, int width, int v_width, T scale)
{
	extern __shared__ __align__(16) unsigned char gsm[];
	T *pw = reinterpret_cast<T *>(gsm); // [n_tok] weights of this source row
	T *krow = pw + n_tok;               // [width]
	T *vrow = krow + width;             // [v_width]
	unsigned r = blockIdx.x;
	const int h = int(r % unsigned(n_heads));
	r /= unsigned(n_heads);
	const int s = int(r % unsigned(n_tok));
	const int b = int(r / unsigned(n_tok));
	const size_t row = size_t(n_heads) * width, vr = size_t(n_heads) * v_width;
	const T *kp = k + (size_t(b) * n_tok + s) * row + size_t(h) * width;
	const T *vp = v + (size_t(b) * n_tok + s) * vr + size_t(h) * v_width;
	for (int w = threadIdx.x; w < width; w += GEN_NT)
		krow[w] = kp[w];
	for (int c = threadIdx.x; c < v_width; c += GEN_NT)
		vrow[c] = vp[c];
	__syncthreads();
	const T *qb = q + size_t(b) * n_tok * row + size_t(h) * width;
	const T *gb = dvo + size_t(b) * n_tok * vr + size_t(h) * v_width;
	for (int t = threadIdx.x; t < n_tok; t += GEN_NT) {
		const T *qp = qb + size_t(t) * row, *gp = gb + size_t(t) * vr;
		T acc = T(0), dp = T(0);
		for (int w = 0; w < width; w++)
			acc += absdiff(qp[w], krow[w]);
		for (int c = 0; c < v_width; c++)
			dp += vrow[c] * gp[c];
		const size_t st = (size_t(b) * n_tok + t) * n_heads + h;
		const T p = exp_t(acc * scale - lse[st]);
		pw[t] = p;
		dx[((size_t(b) * n_tok + s) * n_tok + t) * n_heads + h] = p * (dp - delta[st]);
	}
	__syncthreads();
	T *op = dv + (size_t(b) * n_tok + s) * vr + size_t(h) * v_width;
	for (int c = threadIdx.x; c < v_width; c += GEN_NT) {
		T o = T(0);
		for (int t = 0; t < n_tok; t++)
			o += pw[t] * gb[size_t(t) * vr + c];
		op[c] = o;
	}
}

template <typename T>
int launch_bwd_generic(const T *q, const T *k, const T *v, const T *dvo, const T *lse, const T *delta, T *dx, T *dv, int bs,
		       int n_tok, int n_heads, int width, int v_width, cudaStream_t st)
{
	const long long grid = (long long)bs * n_tok * n_heads;
	const size_t smem = (size_t(n_tok) + width + v_width) * sizeof(T);
	if (grid > 0x7fffffffLL || smem > 200 * 1024)
		return L1ATTN_ERR_SHAPE;
	auto kern = softmax_v_bwd_kernel<T>;
	L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	kern<<<unsigned(grid), GEN_NT, smem, st>>>(q, k, v, dvo, lse, delta, dx, dv, n_tok, n_heads, width, v_width,
						    T(-1.0 / sqrt(double(width))));
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

// TMA variant: the forward kernel with the roles swapped.  The CTA owns TT source rows (their key and
// value rows stay in shared memory) and streams the query and dvo rows in tiles of 64; a half-warp
// owns TI source rows, a lane 4 query columns for the scores and the <v, dvo> products, and NV value
// columns for dv.  Every operand row is kept as 128-byte slices with the 128-byte swizzle.
template <int NV, int TI, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
softmax_v_bwd_tma_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
			 const __grid_constant__ CUtensorMap vmap, const __grid_constant__ CUtensorMap gmap,
			 const float *__restrict__ lse, const float *__restrict__ delta, float *__restrict__ dx,
			 float *__restrict__ dv, SvShape sh, int *err)
{
	constexpr int TT = 2 * NW * TI; // source rows of the CTA
	constexpr int NTH = NW * 32;
	constexpr int VW = 16 * NV;
	constexpr int NVB = VW / 32; // 128-byte slices per value row
	extern __shared__ __align__(1024) unsigned char smem_raw[];
	unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
	__shared__ __align__(8) uint64_t own_bar, full_bar[MAX_STAGE], empty_bar[MAX_STAGE];
	const int k_bytes = sh.nwb * TT * 128, v_bytes = NVB * TT * 128;
	const int q_bytes = sh.nwb * TS * 128, g_bytes = NVB * TS * 128, stage_bytes = q_bytes + g_bytes;
	unsigned char *Ks = base, *Vs = base + k_bytes;
	unsigned char *stages = Vs + v_bytes;
	float *Ps = reinterpret_cast<float *>(stages + size_t(sh.nstage) * stage_bytes);

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	unsigned r = blockIdx.x;
	const int s0 = int(r % unsigned(sh.ntt)) * TT;
	r /= unsigned(sh.ntt);
	const int h = int(r % unsigned(sh.n_heads));
	const int b = int(r / unsigned(sh.n_heads));
	const int nt = (sh.n_tok + TS - 1) / TS;

	if (tid == 0) {
		mbar_init(&own_bar, 1);
		for (int s = 0; s < MAX_STAGE; s++) {
			mbar_init(&full_bar[s], 1);
			mbar_init(&empty_bar[s], NTH / 32);
		}
		mbar_fence_init();
	}
	__syncthreads();

	auto load_tile = [&](int m) {
		const int st = m % sh.nstage;
		unsigned char *dst = stages + size_t(st) * stage_bytes;
		mbar_expect_tx(&full_bar[st], uint32_t(stage_bytes));
		for (int wb = 0; wb < sh.nwb; wb++)
			tma_load_4d(dst + wb * TS * 128, &qmap, &full_bar[st], wb * 32, h, m * TS, b);
		for (int vb = 0; vb < NVB; vb++)
			tma_load_4d(dst + q_bytes + vb * TS * 128, &gmap, &full_bar[st], vb * 32, h, m * TS, b);
	};
	if (tid == 0) {
		mbar_expect_tx(&own_bar, uint32_t(k_bytes + v_bytes));
		for (int wb = 0; wb < sh.nwb; wb++)
			tma_load_4d(Ks + wb * TT * 128, &kmap, &own_bar, wb * 32, h, s0, b);
		for (int vb = 0; vb < NVB; vb++)
			tma_load_4d(Vs + vb * TT * 128, &vmap, &own_bar, vb * 32, h, s0, b);
		for (int m = 0; m < sh.nstage - 1 && m < nt; m++)
			load_tile(m);
	}

	const int sg = lane & 15, tg = warp * 2 + (lane >> 4);
	float o[TI][NV];
#pragma unroll
	for (int i = 0; i < TI; i++)
#pragma unroll
		for (int e = 0; e < NV; e++)
			o[i][e] = 0.f;
	bool dead = false;
	if (!mbar_wait(&own_bar, 0, err))
		dead = true;
	float *Pw = Ps + tg * PP;
	const size_t hstride = size_t(sh.n_heads);

	for (int m = 0; m < nt; m++) {
		if (warp == m % NW && lane == 0 && m + sh.nstage - 1 < nt && !dead) {
			const int mm = m + sh.nstage - 1;
			if (mbar_wait(&empty_bar[mm % sh.nstage], ((unsigned(mm) / unsigned(sh.nstage)) & 1u) ^ 1u, err))
				load_tile(mm);
			else
				dead = true;
		}
		__syncwarp();
		// per-query statistics of this lane's 4 columns (global loads issued before the wait)
		float lj[4], dj[4];
#pragma unroll
		for (int j = 0; j < 4; j++) {
			const int t = m * TS + j * 16 + sg;
			const bool ok = t < sh.n_tok;
			const size_t st = (size_t(b) * sh.n_tok + (ok ? t : 0)) * hstride + h;
			lj[j] = ok ? lse[st] : INFINITY; // exp(x - inf) = 0: query rows past the end weigh nothing
			dj[j] = ok ? delta[st] : 0.f;
		}
		const int st = m % sh.nstage;
		if (!dead && !mbar_wait(&full_bar[st], (unsigned(m) / unsigned(sh.nstage)) & 1u, err))
			dead = true;
		const unsigned char *Qs = stages + size_t(st) * stage_bytes;
		const unsigned char *Gs = Qs + q_bytes;

		float acc[TI][4], dp[TI][4];
#pragma unroll
		for (int i = 0; i < TI; i++)
#pragma unroll
			for (int j = 0; j < 4; j++) {
				acc[i][j] = 0.f;
				dp[i][j] = 0.f;
			}
		for (int wb = 0; wb < sh.nwb; wb++) {
			const ulonglong2 *Kb = reinterpret_cast<const ulonglong2 *>(Ks + wb * TT * 128);
			const ulonglong2 *Qb = reinterpret_cast<const ulonglong2 *>(Qs + wb * TS * 128);
#pragma unroll 2
			for (int c = 0; c < 8; c++) {
				ulonglong2 qv[4];
#pragma unroll
				for (int j = 0; j < 4; j++)
					qv[j] = Qb[(j * 16 + sg) * 8 + (c ^ (sg & 7))];
#pragma unroll
				for (int i = 0; i < TI; i++) {
					const ulonglong2 kv = Kb[(i * (2 * NW) + tg) * 8 + (c ^ (tg & 7))];
#pragma unroll
					for (int j = 0; j < 4; j++) {
						unsigned long long d0, d1;
						float x0, x1, x2, x3;
						asm("sub.f32x2 %0, %1, %2;" : "=l"(d0) : "l"(kv.x), "l"(qv[j].x));
						asm("sub.f32x2 %0, %1, %2;" : "=l"(d1) : "l"(kv.y), "l"(qv[j].y));
						asm("mov.b64 {%0, %1}, %2;" : "=f"(x0), "=f"(x1) : "l"(d0));
						asm("mov.b64 {%0, %1}, %2;" : "=f"(x2), "=f"(x3) : "l"(d1));
						acc[i][j] += fabsf(x0);
						acc[i][j] += fabsf(x1);
						acc[i][j] += fabsf(x2);
						acc[i][j] += fabsf(x3);
					}
				}
			}
		}
#pragma unroll
		for (int vb = 0; vb < NVB; vb++) {
			const float4 *Vb = reinterpret_cast<const float4 *>(Vs + vb * TT * 128);
			const float4 *Gb = reinterpret_cast<const float4 *>(Gs + vb * TS * 128);
#pragma unroll 2
			for (int c = 0; c < 8; c++) {
				float4 gv[4];
#pragma unroll
				for (int j = 0; j < 4; j++)
					gv[j] = Gb[(j * 16 + sg) * 8 + (c ^ (sg & 7))];
#pragma unroll
				for (int i = 0; i < TI; i++) {
					const float4 vv = Vb[(i * (2 * NW) + tg) * 8 + (c ^ (tg & 7))];
#pragma unroll
					for (int j = 0; j < 4; j++) {
						dp[i][j] = fmaf(vv.x, gv[j].x, dp[i][j]);
						dp[i][j] = fmaf(vv.y, gv[j].y, dp[i][j]);
						dp[i][j] = fmaf(vv.z, gv[j].z, dp[i][j]);
						dp[i][j] = fmaf(vv.w, gv[j].w, dp[i][j]);
					}
				}
			}
		}

		// weights, score gradients (stored), weights parked for the dv product
#pragma unroll
		for (int i = 0; i < TI; i++) {
			const int s = s0 + i * (2 * NW) + tg;
			float *dxr = dx + ((size_t(b) * sh.n_tok + (s < sh.n_tok ? s : 0)) * sh.n_tok) * hstride + h;
#pragma unroll
			for (int j = 0; j < 4; j++) {
				const int t = m * TS + j * 16 + sg;
				const float p = expf(acc[i][j] * sh.scale - lj[j]);
				Pw[i * (2 * NW) * PP + j * 16 + sg] = p;
				if (s < sh.n_tok && t < sh.n_tok)
					dxr[size_t(t) * hstride] = p * (dp[i][j] - dj[j]);
			}
		}
		__syncwarp();

		// dv rows += weights x dvo rows; this lane owns value columns [sg*NV, sg*NV+NV)
#pragma unroll 2
		for (int t4 = 0; t4 < TS / 4; t4++) {
			float4 p[TI];
#pragma unroll
			for (int i = 0; i < TI; i++)
				p[i] = *reinterpret_cast<const float4 *>(Pw + i * (2 * NW) * PP + t4 * 4);
#pragma unroll
			for (int tt = 0; tt < 4; tt++) {
				const int trow = t4 * 4 + tt;
				float gvv[NV];
#pragma unroll
				for (int e = 0; e < NV; e += (NV < 4 ? NV : 4)) {
					const int col = sg * NV + e; // float column within the value row
					const unsigned char *gp = Gs + (col >> 5) * TS * 128 + trow * 128 + ((((col & 31) >> 2) ^ (trow & 7)) << 4);
					if (NV == 2) {
						const float2 t2 = *reinterpret_cast<const float2 *>(gp + (col & 3) * 4);
						gvv[0] = t2.x;
						gvv[1 % NV] = t2.y;
					} else {
						const float4 t4v = *reinterpret_cast<const float4 *>(gp);
						gvv[e] = t4v.x;
						gvv[(e + 1) % NV] = t4v.y;
						gvv[(e + 2) % NV] = t4v.z;
						gvv[(e + 3) % NV] = t4v.w;
					}
				}
#pragma unroll
				for (int i = 0; i < TI; i++) {
					const float pi = tt == 0 ? p[i].x : tt == 1 ? p[i].y : tt == 2 ? p[i].z : p[i].w;
#pragma unroll
					for (int e = 0; e < NV; e++)
						o[i][e] = fmaf(pi, gvv[e], o[i][e]);
				}
			}
		}
		__syncwarp();
		if (lane == 0)
			mbar_arrive(&empty_bar[st]);
	}

	const size_t vrow = size_t(sh.n_heads) * VW;
#pragma unroll
	for (int i = 0; i < TI; i++) {
		const int s = s0 + i * (2 * NW) + tg;
		if (s >= sh.n_tok)
			continue;
		float *op = dv + (size_t(b) * sh.n_tok + s) * vrow + size_t(h) * VW + sg * NV;
#pragma unroll
		for (int e = 0; e < NV; e++)
			op[e] = o[i][e];
	}
}

size_t sv_bwd_smem(int nwb, int nv, int tt_rows, int nstage)
{
	const size_t tt = size_t(tt_rows), nvb = size_t(nv) / 2;
	return (size_t(nwb) + nvb) * tt * 128 + size_t(nstage) * (size_t(nwb) + nvb) * TS * 128 + tt * PP * 4 + 1024;
}

template <int NV, int TI, int NW>
int launch_bwd_tma(const float *q, const float *k, const float *v, const float *dvo, const float *lse, const float *delta,
		   float *dx, float *dv, int bs, int n_tok, int n_heads, int width, int nstage, size_t smem, cudaStream_t st)
{
	constexpr int TT = 2 * NW * TI, VW = 16 * NV, NTH = NW * 32;
	const uint64_t dims[4] = {uint64_t(width), uint64_t(n_heads), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t str[3] = {uint64_t(width) * 4, uint64_t(n_heads) * width * 4, uint64_t(n_tok) * n_heads * width * 4};
	const uint64_t vdims[4] = {uint64_t(VW), uint64_t(n_heads), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t vstr[3] = {uint64_t(VW) * 4, uint64_t(n_heads) * VW * 4, uint64_t(n_tok) * n_heads * VW * 4};
	const uint32_t own[4] = {32, 1, TT, 1}, stream[4] = {32, 1, TS, 1};
	CUtensorMap qmap, kmap, vmap, gmap;
	const auto f32 = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
	const auto swz = CU_TENSOR_MAP_SWIZZLE_128B;
	if (!encode_tmap_4d(&qmap, f32, q, dims, str, stream, swz) || !encode_tmap_4d(&kmap, f32, k, dims, str, own, swz) ||
	    !encode_tmap_4d(&vmap, f32, v, vdims, vstr, own, swz) || !encode_tmap_4d(&gmap, f32, dvo, vdims, vstr, stream, swz))
		return 1;
	int *err = device_error_word();
	if (!err)
		return 1;
	SvShape sh;
	sh.n_tok = n_tok;
	sh.n_heads = n_heads;
	sh.nwb = width / 32;
	sh.nstage = nstage;
	sh.ntt = (n_tok + TT - 1) / TT;
	sh.mode = 0;
	sh.scale = float(-1.0 / sqrt(double(width)));
	const long long grid = (long long)bs * n_heads * sh.ntt;
	if (grid > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	auto kern = softmax_v_bwd_tma_kernel<NV, TI, NW>;
	L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	kern<<<unsigned(grid), NTH, smem, st>>>(qmap, kmap, vmap, gmap, lse, delta, dx, dv, sh, err);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

int softmax_v_bwd_tma(const float *q, const float *k, const float *v, const float *dvo, const float *lse, const float *delta,
		      float *dx, float *dv, int bs, int n_tok, int n_heads, int width, int v_width, cudaStream_t st)
{
	if (width % 32 != 0 || width > 128 || (v_width != 32 && v_width != 64 && v_width != 128))
		return 1;
	for (const void *p : {(const void *)q, (const void *)k, (const void *)v, (const void *)dvo})
		if (!aligned(p, 16))
			return 1;
	const int nwb = width / 32, nv = v_width / 16;
	const size_t limit = 227 * 1024 - 256;
	const bool nw16 = nv <= 4; // see softmax_v_tma
	const int cand[2][2] = {{nw16 ? 4 : 8, nw16 ? 16 : 8}, {4, 8}};
	int ti = 0, nw = 0, nstage = 0;
	for (const auto &c : cand) {
		for (int cand_ns : {3, 2})
			if (!ti && sv_bwd_smem(nwb, nv, 2 * c[0] * c[1], cand_ns) <= limit) {
				ti = c[0];
				nw = c[1];
				nstage = cand_ns;
			}
	}
	if (!ti)
		return 1;
	const size_t smem = sv_bwd_smem(nwb, nv, 2 * ti * nw, nstage);
#define L1B_SVB(NV_, TI_, NW_)                      \
	if (nv == NV_ && ti == TI_ && nw == NW_)    \
		return launch_bwd_tma<NV_, TI_, NW_>(q, k, v, dvo, lse, delta, dx, dv, bs, n_tok, n_heads, width, nstage, smem, st);
	L1B_SVB(2, 8, 8) L1B_SVB(4, 8, 8) L1B_SVB(8, 8, 8) L1B_SVB(2, 4, 8) L1B_SVB(4, 4, 8) L1B_SVB(8, 4, 8)
	L1B_SVB(2, 4, 16) L1B_SVB(4, 4, 16) L1B_SVB(8, 4, 16)
#undef L1B_SVB
	return 1;
}

} // namespace

int dense_softmax_v_launch(const void *q, const void *k, const void *v, void *vo, void *lse, int bs, int n_tok, int n_heads,
			   int width, int v_width, int mode, int dtype, cudaStream_t st)
{
	if (bs == 0 || n_tok == 0 || n_heads == 0 || v_width == 0)
		return L1ATTN_OK;
	static const bool no_tma = getenv("L1ATTN_NO_TMA") != nullptr; // debugging aid: force the generic kernel
	if (dtype == L1ATTN_F32 && !no_tma && width > 0) {
		const int rc = softmax_v_tma((const float *)q, (const float *)k, (const float *)v, (float *)vo, (float *)lse, bs, n_tok,
					     n_heads, width, v_width, mode, st);
		if (rc <= 0)
			return rc;
	}
	if (dtype == L1ATTN_F32)
		return launch_generic((const float *)q, (const float *)k, (const float *)v, (float *)vo, (float *)lse, bs, n_tok,
				      n_heads, width, v_width, mode, st);
	return launch_generic((const double *)q, (const double *)k, (const double *)v, (double *)vo, (double *)lse, bs, n_tok,
			      n_heads, width, v_width, mode, st);
}

int dense_softmax_v_bwd_dx_launch(const void *q, const void *k, const void *v, const void *dvo, const void *lse,
				  const void *delta, void *dx, void *dv, int bs, int n_tok, int n_heads, int width, int v_width,
				  int dtype, cudaStream_t st)
{
	if (bs == 0 || n_tok == 0 || n_heads == 0 || v_width == 0)
		return L1ATTN_OK;
	static const bool no_tma = getenv("L1ATTN_NO_TMA") != nullptr;
	if (dtype == L1ATTN_F32 && !no_tma && width > 0) {
		const int rc = softmax_v_bwd_tma((const float *)q, (const float *)k, (const float *)v, (const float *)dvo,
						 (const float *)lse, (const float *)delta, (float *)dx, (float *)dv, bs, n_tok, n_heads,
						 width, v_width, st);
		if (rc <= 0)
			return rc;
	}
	if (dtype == L1ATTN_F32)
		return launch_bwd_generic((const float *)q, (const float *)k, (const float *)v, (const float *)dvo,
					  (const float *)lse, (const float *)delta, (float *)dx, (float *)dv, bs, n_tok, n_heads, width,
					  v_width, st);
	return launch_bwd_generic((const double *)q, (const double *)k, (const double *)v, (const double *)dvo,
				  (const double *)lse, (const double *)delta, (double *)dx, (double *)dv, bs, n_tok, n_heads, width,
				  v_width, st);
}

} // namespace l1b
