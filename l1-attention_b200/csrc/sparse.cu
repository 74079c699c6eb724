// Sparse (coordinate-list) L1 attention, forward and backward, one- and bi-directional.
//
// The reference scatters every edge's contribution with atomicAdd
// (cuda/l1attn_sparse_cuda_kernel.cu:148-181,183-254,327-370).  Here every output row has one
// owner: a warp owns a (batch item, token, group of heads) and walks that token's edges, either
//   * the slots (dst, r) of a destination token    ("dst pass": scores, softmax, vo, d_q, d_vb) or
//   * the incoming slots of a source token          ("src pass": d_v, d_k, the bidi part of vo),
// accumulating in registers and storing once.  No atomics, fixed summation order, results are
// bit-reproducible.  Within a warp LPH lanes share a head and split its width; a head's dot
// products / L1 sums are finished with xor-shuffles.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <initializer_list>
#include <type_traits>
#include <mutex>
#include "common.cuh"

namespace l1b {
namespace {

struct SparseArgs {
	int bs, n_tok, n_heads, width, v_width, dm; // dm = dst_mxlen
	int lph;                                     // lanes per head (power of two <= 32)
	int use_softmax, bidi;
	const int32_t *slot_src, *csc_off, *csc_slot;
};

template <typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> ldv(const T *p, bool ok)
{
	Pack<T, VEC> r;
	if (ok) {
		r = *reinterpret_cast<const Pack<T, VEC> *>(p);
	} else {
#pragma unroll
		for (int e = 0; e < VEC; e++)
			r.v[e] = T(0);
	}
	return r;
}

// Storage type S, arithmetic type T.  S == T for float and double; for the 16-bit storage types
// (__half, __nv_bfloat16) the forward loads VEC elements at once, computes in float and rounds on store.
template <typename S> __device__ __forceinline__ float to_f(S x) { return float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename S> __device__ __forceinline__ S from_f(float x) { return S(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename S, typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> ldc(const S *p, bool ok)
{
	if constexpr (std::is_same<S, T>::value) {
		return ldv<T, VEC>(p, ok);
	} else {
		const Pack<S, VEC> raw = ldv<S, VEC>(p, ok);
		Pack<T, VEC> r;
#pragma unroll
		for (int e = 0; e < VEC; e++)
			r.v[e] = to_f<S>(raw.v[e]);
		return r;
	}
}
template <typename S, typename T, int VEC> __device__ __forceinline__ void stc(S *p, const Pack<T, VEC> &x)
{
	if constexpr (std::is_same<S, T>::value) {
		*reinterpret_cast<Pack<T, VEC> *>(p) = x;
	} else {
		Pack<S, VEC> raw;
#pragma unroll
		for (int e = 0; e < VEC; e++)
			raw.v[e] = from_f<S>(x.v[e]);
		*reinterpret_cast<Pack<S, VEC> *>(p) = raw;
	}
}
template <typename S, typename T> __device__ __forceinline__ T ld1(const S *p)
{
	if constexpr (std::is_same<S, T>::value)
		return *p;
	else
		return to_f<S>(*p);
}
template <typename S, typename T> __device__ __forceinline__ void st1(S *p, T x)
{
	if constexpr (std::is_same<S, T>::value)
		*p = x;
	else
		*p = from_f<S>(x);
}

// LPHC > 0: lanes per head known at compile time (the shuffles unroll, index math folds); 0: run-time value
template <int LPHC, typename T> __device__ __forceinline__ T group_sum(T x, int lph)
{
	if (LPHC > 0) {
#pragma unroll
		for (int o = LPHC >> 1; o > 0; o >>= 1)
			x += __shfl_xor_sync(0xffffffffu, x, o);
	} else {
		for (int o = lph >> 1; o > 0; o >>= 1)
			x += __shfl_xor_sync(0xffffffffu, x, o);
	}
	return x;
}

// Which (b, tok, head) this lane works on.  Returns false for warps past the end (whole warp).
struct Who {
	int b, tok, h, li;
	bool head_ok;
};
template <int LPHC> __device__ __forceinline__ bool decode(const SparseArgs &a, Who &w)
{
	const int lane = threadIdx.x & 31;
	const int lph = LPHC > 0 ? LPHC : a.lph;
	const int hpw = 32 / lph;
	const int nhc = (a.n_heads + hpw - 1) / hpw;
	long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
	const int hc = int(gw % nhc);
	gw /= nhc;
	w.tok = int(gw % a.n_tok);
	const long long b = gw / a.n_tok;
	if (b >= a.bs)
		return false;
	w.b = int(b);
	w.li = lane % lph;
	w.h = hc * hpw + lane / lph;
	w.head_ok = w.h < a.n_heads;
	return true;
}

// Edge loops walk the slots / incoming edges U at a time: the U gathered rows are requested before
// any of them is used, so U row fetches (L2 latency each) are in flight per warp instead of one.
constexpr int U = 4;

// Walk of this lane's vectors of a row: x = li*VEC, += lanes-per-head * VEC.  With NX > 0 the trip count
// is a compile-time constant (width == NX * lanes-per-head * VEC) and the walk unrolls completely.
#define L1B_XLOOP(WIDTH) _Pragma("unroll") for (int it_ = 0, x = w.li * VEC; (NX > 0 ? it_ < NX : x < (WIDTH)); it_++, x += step)

// Edge-outer walk for the widths whose vector count per lane is a compile-time constant (NX > 0): every
// list entry (a slot of the destination or an incoming edge of the source) is decoded ONCE -- index,
// weight, row address -- and its NX vectors are fetched at immediate offsets, instead of walking the whole
// list once per vector (which repeated the decoding, and in the source lists an integer division, NX times).
//   MODE 0: acc += weight * row      MODE 1: acc += sign(own - row) * weight      MODE 2: acc += sign(row - own) * weight
// entry(i, ptr, weight) fills the row pointer of entry i (already at this lane's first vector; any valid
// address when the entry is absent: the row is then loaded but not used, which is cheaper than a
// predicated load plus zero fill) and its weight, and returns whether the entry exists.
constexpr int UE = 2; // entries in flight per lane: UE * NX 16-byte loads
template <typename S, typename T, int VEC, int NX, int MODE, typename F>
__device__ __forceinline__ void walk_list(Pack<T, VEC> (&acc)[NX], const Pack<T, VEC> (&own)[NX], int n, int step, F entry)
{
	for (int e0 = 0; e0 < n; e0 += UE) {
		T wgt[UE];
		const S *ptr[UE];
		bool ok[UE];
#pragma unroll
		for (int u = 0; u < UE; u++) {
			wgt[u] = T(0);
			ok[u] = entry(e0 + u < n ? e0 + u : e0, ptr[u], wgt[u]) && e0 + u < n;
			if (!ok[u])
				wgt[u] = T(0);
		}
		Pack<T, VEC> row[UE][NX];
#pragma unroll
		for (int u = 0; u < UE; u++)
#pragma unroll
			for (int it = 0; it < NX; it++)
				row[u][it] = ldc<S, T, VEC>(ptr[u] + it * step, true);
#pragma unroll
		for (int u = 0; u < UE; u++)
			if (ok[u])
#pragma unroll
			for (int it = 0; it < NX; it++)
#pragma unroll
				for (int i = 0; i < VEC; i++) {
					if (MODE == 0)
						acc[it].v[i] += wgt[u] * row[u][it].v[i];
					else if (MODE == 1)
						acc[it].v[i] += sign_apply(own[it].v[i] - row[u][it].v[i], wgt[u]);
					else
						acc[it].v[i] += sign_apply(row[u][it].v[i] - own[it].v[i], wgt[u]);
				}
	}
}
template <typename T, int VEC, int NX> __device__ __forceinline__ void zero_acc(Pack<T, VEC> (&acc)[NX])
{
#pragma unroll
	for (int it = 0; it < NX; it++)
#pragma unroll
		for (int i = 0; i < VEC; i++)
			acc[it].v[i] = T(0);
}

// ---- forward, dst pass: scores -> exp -> (+1)-softmax -> attn, vo[dst] = sum_r a_r v[src_r] ----
template <typename S, typename T, int VEC, int LPHC, int NX>
__global__ void __launch_bounds__(256) sparse_fwd_dst_kernel(SparseArgs a, const S *__restrict__ v,
							      const S *__restrict__ q, const S *__restrict__ k,
							      S *__restrict__ vo, S *attn, T scale)
{
	Who w;
	if (!decode<LPHC>(a, w))
		return;
	const int dst = w.tok, H = a.n_heads, W = a.width, Wv = a.v_width, dm = a.dm;
	const int hh = w.head_ok ? w.h : 0;
	const size_t tokrow = size_t(w.b) * a.n_tok;
	const S *qrow = q + ((tokrow + dst) * H + hh) * W;
	S *arow = attn + ((tokrow + dst) * dm) * H + hh;
	const int32_t *slots = a.slot_src + size_t(dst) * dm;
	const int lph = LPHC > 0 ? LPHC : a.lph;
	const int step = lph * VEC;

	T denom = T(1);
	for (int r0 = 0; r0 < dm; r0 += U) {
		int src[U];
		T part[U];
#pragma unroll
		for (int u = 0; u < U; u++) {
			src[u] = r0 + u < dm ? slots[r0 + u] : -1;
			part[u] = T(0);
		}
		L1B_XLOOP(W) {
			// rows of absent slots / heads past the end are read from a valid address and their
			// scores discarded below: cheaper than predicated loads with zero fill
			const Pack<T, VEC> qv = ldc<S, T, VEC>(qrow + x, true);
			Pack<T, VEC> kv[U];
#pragma unroll
			for (int u = 0; u < U; u++)
				kv[u] = ldc<S, T, VEC>(k + ((tokrow + (src[u] < 0 ? 0 : src[u])) * H + hh) * W + x, true);
#pragma unroll
			for (int u = 0; u < U; u++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					part[u] += absdiff(qv.v[i], kv[u].v[i]);
		}
#pragma unroll
		for (int u = 0; u < U; u++)
			part[u] = group_sum<LPHC>(part[u], lph);
#pragma unroll
		for (int u = 0; u < U; u++) {
			const T e = src[u] >= 0 ? exp_t(part[u] * scale) : T(0);
			denom += e;
			if (w.li == 0 && w.head_ok && r0 + u < dm)
				st1<S, T>(arow + size_t(r0 + u) * H, e);
		}
	}
	__syncwarp();
	if (a.use_softmax && w.head_ok)
		for (int r = w.li; r < dm; r += lph)
			st1<S, T>(arow + size_t(r) * H, ld1<S, T>(arow + size_t(r) * H) / denom);
	__syncwarp();

	S *orow = vo + ((tokrow + dst) * H + hh) * Wv;
	if constexpr (NX > 0) {
		Pack<T, VEC> acc[NX];
		zero_acc(acc);
		const S *vbase = v + (tokrow * H + hh) * Wv + w.li * VEC;
		walk_list<S, T, VEC, NX, 0>(acc, acc, dm, step, [&](int r, const S *&ptr, T &wgt) {
			const int src = slots[r];
			const bool ok = w.head_ok && src >= 0;
			ptr = vbase + size_t(ok ? src : 0) * H * Wv;
			if (ok)
				wgt = ld1<S, T>(arow + size_t(r) * H);
			return ok;
		});
		if (w.head_ok) {
#pragma unroll
			for (int it = 0; it < NX; it++)
				stc<S, T, VEC>(orow + w.li * VEC + it * step, acc[it]);
		}
		return;
	}
	L1B_XLOOP(Wv) {
		Pack<T, VEC> acc = ldv<T, VEC>(nullptr, false);
		for (int r0 = 0; r0 < dm; r0 += U) {
			T ar[U];
			Pack<T, VEC> vv[U];
#pragma unroll
			for (int u = 0; u < U; u++) {
				const int src = r0 + u < dm ? slots[r0 + u] : -1;
				const bool ok = w.head_ok && src >= 0;
				ar[u] = ok ? ld1<S, T>(arow + size_t(r0 + u) * H) : T(0);
				vv[u] = ldc<S, T, VEC>(v + ((tokrow + (src < 0 ? 0 : src)) * H + hh) * Wv + x, ok);
			}
#pragma unroll
			for (int u = 0; u < U; u++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					acc.v[i] += ar[u] * vv[u].v[i];
		}
		if (w.head_ok)
			stc<S, T, VEC>(orow + x, acc);
	}
}

// ---- forward, src pass (bidi only): vo[src] += sum_{incoming (dst,r)} a[dst][r] * vb[dst] ----
template <typename S, typename T, int VEC, int LPHC, int NX>
__global__ void __launch_bounds__(256) sparse_fwd_src_kernel(SparseArgs a, const S *__restrict__ vb,
							      const S *__restrict__ attn, S *vo)
{
	Who w;
	if (!decode<LPHC>(a, w))
		return;
	if (!w.head_ok)
		return;
	const int src = w.tok, H = a.n_heads, Wv = a.v_width, dm = a.dm;
	const size_t tokrow = size_t(w.b) * a.n_tok;
	const int e0 = a.csc_off[src], e1 = a.csc_off[src + 1];
	const int lph = LPHC > 0 ? LPHC : a.lph;
	const int step = lph * VEC;
	S *orow = vo + ((tokrow + src) * H + w.h) * Wv;
	if constexpr (NX > 0) {
		Pack<T, VEC> acc[NX];
		zero_acc(acc);
		const S *bbase = vb + (tokrow * H + w.h) * Wv + w.li * VEC;
		const S *abase = attn + (tokrow * dm) * H + w.h;
		walk_list<S, T, VEC, NX, 0>(acc, acc, e1 - e0, step, [&](int e, const S *&ptr, T &wgt) {
			const int slot = a.csc_slot[e0 + e];
			ptr = bbase + size_t(slot / dm) * H * Wv;
			wgt = ld1<S, T>(abase + size_t(slot) * H);
			return true;
		});
#pragma unroll
		for (int it = 0; it < NX; it++) {
			Pack<T, VEC> cur = ldc<S, T, VEC>(orow + w.li * VEC + it * step, true);
#pragma unroll
			for (int i = 0; i < VEC; i++)
				cur.v[i] += acc[it].v[i];
			stc<S, T, VEC>(orow + w.li * VEC + it * step, cur);
		}
		return;
	}
	L1B_XLOOP(Wv) {
		Pack<T, VEC> acc = ldv<T, VEC>(nullptr, false);
		for (int eb = e0; eb < e1; eb += U) {
			T ar[U];
			Pack<T, VEC> vv[U];
#pragma unroll
			for (int u = 0; u < U; u++) {
				const bool ok = eb + u < e1;
				const int slot = ok ? a.csc_slot[eb + u] : 0;
				ar[u] = ok ? ld1<S, T>(attn + (tokrow * dm + slot) * H + w.h) : T(0);
				vv[u] = ldc<S, T, VEC>(vb + ((tokrow + slot / dm) * H + w.h) * Wv + x, ok);
			}
#pragma unroll
			for (int u = 0; u < U; u++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					acc.v[i] += ar[u] * vv[u].v[i];
		}
		Pack<T, VEC> cur = ldc<S, T, VEC>(orow + x, true);
#pragma unroll
		for (int i = 0; i < VEC; i++)
			cur.v[i] += acc.v[i];
		stc<S, T, VEC>(orow + x, cur);
	}
}

// ---- backward, dst pass: ds_r, softmax Jacobian in closed form, dx_r -> scratch, d_q, (d_vb) ----
//   ds_r = <v[src_r], dvo[dst]>  (+ <vb[dst], dvo[src_r]> when bidi)
//   softmax: dx_r = a_r (ds_r - sum_j a_j ds_j)   [same as the reference's Jacobian product,
//            cuda/l1attn_sparse_cuda_kernel.cu:256-295, without its O(dst_mxlen^2) loop]
//   else:    dx_r = a_r ds_r
// For the common widths ONE walk over the slots does all of it (see the NX > 0 branch): 121 registers, two CTAs
// per SM.  The generic branch walks the list once per quantity and is capped at three CTAs per SM.
template <typename T, int VEC, int LPHC, int NX, bool BIDI>
__global__ void __launch_bounds__(256, NX == 4 ? 2 : 3) sparse_bwd_dst_kernel(SparseArgs a, const T *__restrict__ dvo,
							      const T *__restrict__ v, const T *__restrict__ vb,
							      const T *__restrict__ q, const T *__restrict__ k,
							      const T *__restrict__ attn, T *dx, T *__restrict__ d_q,
							      T *__restrict__ d_vb, T scale)
{
	Who w;
	if (!decode<LPHC>(a, w))
		return;
	const int dst = w.tok, H = a.n_heads, W = a.width, Wv = a.v_width, dm = a.dm;
	const int hh = w.head_ok ? w.h : 0;
	const size_t tokrow = size_t(w.b) * a.n_tok;
	const size_t aoff = ((tokrow + dst) * dm) * H + hh;
	const T *arow = attn + aoff;
	T *xrow = dx + aoff;
	const int32_t *slots = a.slot_src + size_t(dst) * dm;
	const int lph = LPHC > 0 ? LPHC : a.lph;
	const int step = lph * VEC;
	const T *gdst = dvo + ((tokrow + dst) * H + hh) * Wv;
	const T *bdst = a.bidi ? vb + ((tokrow + dst) * H + hh) * Wv : nullptr;

	if constexpr (NX > 0) {
		// One walk over the slots: v[src] and k[src] (and dvo[src] when bidirectional) of a slot are gathered
		// together.  ds_r needs only this slot's rows, but dx_r = a_r (ds_r - S) needs S = sum_j a_j ds_j of the
		// whole list, so d_q is accumulated in two parts and combined at the end:
		//   d_q = scale * sum_r sgn_r dx_r = scale * (sum_r sgn_r a_r ds_r  -  S * sum_r sgn_r a_r),  sgn_r = sign(q - k[src_r]).
		Pack<T, VEC> qv[NX], gd[NX], bd[NX], acc1[NX], acc2[NX], accb[NX];
		const T *qrow = q + ((tokrow + dst) * H + hh) * W + w.li * VEC;
#pragma unroll
		for (int it = 0; it < NX; it++) {
			qv[it] = ldv<T, VEC>(qrow + it * step, w.head_ok);
			gd[it] = ldv<T, VEC>(gdst + w.li * VEC + it * step, true);
			bd[it] = ldv<T, VEC>(BIDI ? bdst + w.li * VEC + it * step : gdst, BIDI);
		}
		zero_acc(acc1);
		zero_acc(acc2);
		zero_acc(accb);
		const T *vbase = v + (tokrow * H + hh) * Wv + w.li * VEC, *kbase = k + (tokrow * H + hh) * W + w.li * VEC;
		const T *gbase = dvo + (tokrow * H + hh) * Wv + w.li * VEC;
		T S = T(0);
		for (int r = 0; r < dm; r++) {
			const int src = slots[r];
			const bool ok = w.head_ok && src >= 0;
			const size_t so = size_t(ok ? src : 0) * H;
			Pack<T, VEC> vr[NX], kr[NX], gr[NX];
#pragma unroll
			for (int it = 0; it < NX; it++) {
				vr[it] = ldv<T, VEC>(vbase + so * Wv + it * step, true);
				kr[it] = ldv<T, VEC>(kbase + so * W + it * step, true);
			}
			if (BIDI) {
#pragma unroll
				for (int it = 0; it < NX; it++)
					gr[it] = ldv<T, VEC>(gbase + so * Wv + it * step, true);
			}
			const T ar = ok ? arow[size_t(r) * H] : T(0);
			T part = T(0);
#pragma unroll
			for (int it = 0; it < NX; it++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					part += vr[it].v[i] * gd[it].v[i];
			if (BIDI) {
#pragma unroll
				for (int it = 0; it < NX; it++)
#pragma unroll
					for (int i = 0; i < VEC; i++)
						part += bd[it].v[i] * gr[it].v[i];
			}
			part = group_sum<LPHC>(part, lph);
			if (!ok)
				continue; // (uniform over the lanes of a head; the shuffles above ran for the whole warp)
			S += ar * part;
			if (w.li == 0)
				xrow[size_t(r) * H] = part;
			const T w1 = ar * part;
#pragma unroll
			for (int it = 0; it < NX; it++)
#pragma unroll
				for (int i = 0; i < VEC; i++) {
					const T sg = sign_apply(qv[it].v[i] - kr[it].v[i], T(1));
					acc1[it].v[i] += sg * w1;
					acc2[it].v[i] += sg * ar;
				}
			if (BIDI) {
#pragma unroll
				for (int it = 0; it < NX; it++)
#pragma unroll
					for (int i = 0; i < VEC; i++)
						accb[it].v[i] += ar * gr[it].v[i];
			}
		}
		__syncwarp();
		if (w.head_ok) {
			for (int r = w.li; r < dm; r += lph) { // ds -> dx for the src pass
				if (slots[r] < 0)
					continue;
				const T ar = arow[size_t(r) * H], ds = xrow[size_t(r) * H];
				xrow[size_t(r) * H] = a.use_softmax ? ar * (ds - S) : ar * ds;
			}
			T *orow = d_q + ((tokrow + dst) * H + hh) * W + w.li * VEC;
			const T sfac = a.use_softmax ? S : T(0);
#pragma unroll
			for (int it = 0; it < NX; it++) {
#pragma unroll
				for (int i = 0; i < VEC; i++)
					acc1[it].v[i] = (acc1[it].v[i] - sfac * acc2[it].v[i]) * scale;
				*reinterpret_cast<Pack<T, VEC> *>(orow + it * step) = acc1[it];
			}
			if (BIDI) { // d_vb[dst] = sum_r a_r dvo[src_r]
				T *brow = d_vb + ((tokrow + dst) * H + hh) * Wv + w.li * VEC;
#pragma unroll
				for (int it = 0; it < NX; it++)
					*reinterpret_cast<Pack<T, VEC> *>(brow + it * step) = accb[it];
			}
		}
		return;
	}
	T S = T(0);
	for (int r0 = 0; r0 < dm; r0 += U) {
		int src[U];
		T part[U];
#pragma unroll
		for (int u = 0; u < U; u++) {
			src[u] = r0 + u < dm ? slots[r0 + u] : -1;
			part[u] = T(0);
		}
		L1B_XLOOP(Wv) {
			// absent slots / heads past the end read a valid address; their sums are discarded below
			const Pack<T, VEC> gv = ldv<T, VEC>(gdst + x, true);
			Pack<T, VEC> vv[U], gs[U];
#pragma unroll
			for (int u = 0; u < U; u++) {
				const size_t off = ((tokrow + (src[u] < 0 ? 0 : src[u])) * H + hh) * Wv + x;
				vv[u] = ldv<T, VEC>(v + off, true);
				gs[u] = ldv<T, VEC>(dvo + off, a.bidi != 0);
			}
#pragma unroll
			for (int u = 0; u < U; u++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					part[u] += vv[u].v[i] * gv.v[i];
			if (a.bidi) {
				const Pack<T, VEC> bv = ldv<T, VEC>(bdst + x, true);
#pragma unroll
				for (int u = 0; u < U; u++)
#pragma unroll
					for (int i = 0; i < VEC; i++)
						part[u] += bv.v[i] * gs[u].v[i];
			}
		}
#pragma unroll
		for (int u = 0; u < U; u++)
			part[u] = group_sum<LPHC>(part[u], lph);
#pragma unroll
		for (int u = 0; u < U; u++) {
			if (src[u] < 0)
				continue;
			const T ar = w.head_ok ? arow[size_t(r0 + u) * H] : T(0);
			S += ar * part[u];
			if (w.li == 0 && w.head_ok)
				xrow[size_t(r0 + u) * H] = part[u];
		}
	}
	__syncwarp();
	if (w.head_ok)
		for (int r = w.li; r < dm; r += lph) {
			if (slots[r] < 0)
				continue;
			const T ar = arow[size_t(r) * H], ds = xrow[size_t(r) * H];
			xrow[size_t(r) * H] = a.use_softmax ? ar * (ds - S) : ar * ds;
		}
	__syncwarp();

	const T *qrow = q + ((tokrow + dst) * H + hh) * W;
	T *orow = d_q + ((tokrow + dst) * H + hh) * W;
	L1B_XLOOP(W) {
		const Pack<T, VEC> qv = ldv<T, VEC>(qrow + x, w.head_ok);
		Pack<T, VEC> acc = ldv<T, VEC>(nullptr, false);
		for (int r0 = 0; r0 < dm; r0 += U) {
			T dxr[U];
			Pack<T, VEC> kv[U];
#pragma unroll
			for (int u = 0; u < U; u++) {
				const int src = r0 + u < dm ? slots[r0 + u] : -1;
				const bool ok = w.head_ok && src >= 0;
				dxr[u] = ok ? xrow[size_t(r0 + u) * H] : T(0);
				// a missing edge reads q itself: difference 0, contributes nothing
				kv[u] = ok ? ldv<T, VEC>(k + ((tokrow + src) * H + hh) * W + x, true) : qv;
			}
#pragma unroll
			for (int u = 0; u < U; u++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					acc.v[i] += sign_apply(qv.v[i] - kv[u].v[i], dxr[u]);
		}
		if (w.head_ok) {
#pragma unroll
			for (int i = 0; i < VEC; i++)
				acc.v[i] *= scale;
			*reinterpret_cast<Pack<T, VEC> *>(orow + x) = acc;
		}
	}
	if (a.bidi) { // d_vb[dst] = sum_r a_r dvo[src_r]
		T *brow = d_vb + ((tokrow + dst) * H + hh) * Wv;
		L1B_XLOOP(Wv) {
			Pack<T, VEC> acc = ldv<T, VEC>(nullptr, false);
			for (int r0 = 0; r0 < dm; r0 += U) {
				T ar[U];
				Pack<T, VEC> gs[U];
#pragma unroll
				for (int u = 0; u < U; u++) {
					const int src = r0 + u < dm ? slots[r0 + u] : -1;
					const bool ok = w.head_ok && src >= 0;
					ar[u] = ok ? arow[size_t(r0 + u) * H] : T(0);
					gs[u] = ldv<T, VEC>(dvo + ((tokrow + (src < 0 ? 0 : src)) * H + hh) * Wv + x, ok);
				}
#pragma unroll
				for (int u = 0; u < U; u++)
#pragma unroll
					for (int i = 0; i < VEC; i++)
						acc.v[i] += ar[u] * gs[u].v[i];
			}
			if (w.head_ok)
				*reinterpret_cast<Pack<T, VEC> *>(brow + x) = acc;
		}
	}
}

// ---- backward, src pass: d_v[src] = sum a dvo[dst];  d_k[src] = -scale sum sign(q[dst]-k[src]) dx ----
template <typename T, int VEC, int LPHC, int NX>
__global__ void __launch_bounds__(256) sparse_bwd_src_kernel(SparseArgs a, const T *__restrict__ dvo,
							      const T *__restrict__ q, const T *__restrict__ k,
							      const T *__restrict__ attn, const T *__restrict__ dx,
							      T *__restrict__ d_v, T *__restrict__ d_k, T scale)
{
	Who w;
	if (!decode<LPHC>(a, w))
		return;
	if (!w.head_ok)
		return;
	const int src = w.tok, H = a.n_heads, W = a.width, Wv = a.v_width, dm = a.dm;
	const size_t tokrow = size_t(w.b) * a.n_tok;
	const int e0 = a.csc_off[src], e1 = a.csc_off[src + 1];
	const int lph = LPHC > 0 ? LPHC : a.lph;
	const int step = lph * VEC;
	T *vrow = d_v + ((tokrow + src) * H + w.h) * Wv;
	if constexpr (NX > 0) {
		// one walk over the incoming edges: dvo[dst] and q[dst] of an edge are gathered together
		Pack<T, VEC> accv[NX], acck[NX], kv[NX];
		zero_acc(accv);
		zero_acc(acck);
		const T *krow = k + ((tokrow + src) * H + w.h) * W + w.li * VEC;
#pragma unroll
		for (int it = 0; it < NX; it++)
			kv[it] = ldv<T, VEC>(krow + it * step, true);
		const T *gbase = dvo + (tokrow * H + w.h) * Wv + w.li * VEC, *qbase = q + (tokrow * H + w.h) * W + w.li * VEC;
		const T *abase = attn + (tokrow * dm) * H + w.h, *xbase = dx + (tokrow * dm) * H + w.h;
		for (int e = e0; e < e1; e++) {
			const int slot = a.csc_slot[e];
			const size_t d = size_t(slot / dm) * H;
			Pack<T, VEC> gr[NX], qr[NX];
#pragma unroll
			for (int it = 0; it < NX; it++) {
				gr[it] = ldv<T, VEC>(gbase + d * Wv + it * step, true);
				qr[it] = ldv<T, VEC>(qbase + d * W + it * step, true);
			}
			const T ar = abase[size_t(slot) * H], dxr = xbase[size_t(slot) * H];
#pragma unroll
			for (int it = 0; it < NX; it++)
#pragma unroll
				for (int i = 0; i < VEC; i++) {
					accv[it].v[i] += ar * gr[it].v[i];
					acck[it].v[i] += sign_apply(qr[it].v[i] - kv[it].v[i], dxr);
				}
		}
		T *orow = d_k + ((tokrow + src) * H + w.h) * W + w.li * VEC;
#pragma unroll
		for (int it = 0; it < NX; it++) {
			*reinterpret_cast<Pack<T, VEC> *>(vrow + w.li * VEC + it * step) = accv[it];
#pragma unroll
			for (int i = 0; i < VEC; i++)
				acck[it].v[i] *= -scale;
			*reinterpret_cast<Pack<T, VEC> *>(orow + it * step) = acck[it];
		}
		return;
	}
	L1B_XLOOP(Wv) {
		Pack<T, VEC> acc = ldv<T, VEC>(nullptr, false);
		for (int eb = e0; eb < e1; eb += U) {
			T ar[U];
			Pack<T, VEC> gv[U];
#pragma unroll
			for (int u = 0; u < U; u++) {
				const bool ok = eb + u < e1;
				const int slot = ok ? a.csc_slot[eb + u] : 0;
				ar[u] = ok ? attn[(tokrow * dm + slot) * H + w.h] : T(0);
				gv[u] = ldv<T, VEC>(dvo + ((tokrow + slot / dm) * H + w.h) * Wv + x, ok);
			}
#pragma unroll
			for (int u = 0; u < U; u++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					acc.v[i] += ar[u] * gv[u].v[i];
		}
		*reinterpret_cast<Pack<T, VEC> *>(vrow + x) = acc;
	}
	const T *krow = k + ((tokrow + src) * H + w.h) * W;
	T *orow = d_k + ((tokrow + src) * H + w.h) * W;
	L1B_XLOOP(W) {
		const Pack<T, VEC> kv = ldv<T, VEC>(krow + x, true);
		Pack<T, VEC> acc = ldv<T, VEC>(nullptr, false);
		for (int eb = e0; eb < e1; eb += U) {
			T dxr[U];
			Pack<T, VEC> qv[U];
#pragma unroll
			for (int u = 0; u < U; u++) {
				const bool ok = eb + u < e1;
				const int slot = ok ? a.csc_slot[eb + u] : 0;
				dxr[u] = ok ? dx[(tokrow * dm + slot) * H + w.h] : T(0);
				// past the end of the list read k itself: difference 0, contributes nothing
				qv[u] = ok ? ldv<T, VEC>(q + ((tokrow + slot / dm) * H + w.h) * W + x, true) : kv;
			}
#pragma unroll
			for (int u = 0; u < U; u++)
#pragma unroll
				for (int i = 0; i < VEC; i++)
					acc.v[i] += sign_apply(qv[u].v[i] - kv.v[i], dxr[u]);
		}
#pragma unroll
		for (int i = 0; i < VEC; i++)
			acc.v[i] *= -scale;
		*reinterpret_cast<Pack<T, VEC> *>(orow + x) = acc;
	}
}

// Lanes per head.  Four 16-byte vectors per lane is the fastest walk (fewer shuffle rounds, less index math per
// term), but a warp then covers 32 / lph heads, and with fewer heads than that (a head-group shard of a multi-GPU
// run, a model with few heads) the other lanes idle.  `idle_den`: more lanes share a head when at least
// (idle_den - 1) / idle_den of them would idle otherwise.  Measured at 4096 tokens, 131072 edges, width 64, one batch item:
// forward 4 heads 0.038 ms against 0.055 ms, 2 heads 0.030 / 0.050; backward 4 heads 0.124 against 0.107 (the
// unrolled four-vector walk wins although half its lanes idle), 2 heads 0.073 / 0.104 -- so the forward asks
// with idle_den 2 and the backward with 4.
int lanes_per_head(int mw, int n_heads, int vec, int idle_den);
int pow2_ceil(int x)
{
	int p = 1;
	while (p < x)
		p <<= 1;
	return p;
}

int lanes_per_head(int mw, int n_heads, int vec, int idle_den)
{
	int lph = pow2_ceil((mw + 4 * vec - 1) / (4 * vec));
	if (lph > 32)
		lph = 32;
	{
		const int hpw = 32 / lph, slots = hpw * ((n_heads + hpw - 1) / hpw);
		if (idle_den * (slots - n_heads) < (idle_den - 1) * slots)
			return lph; // few enough idle lanes as it is
	}
	static const bool no_fill = getenv("L1ATTN_SPARSE_NO_FILL") != nullptr; // debugging aid: keep four vectors per lane
	while (!no_fill && lph < 32 && mw >= 2 * lph * vec) {
		const int hpw = 32 / lph, slots = hpw * ((n_heads + hpw - 1) / hpw);
		if (2 * n_heads > slots)
			break; // more than half the lanes busy
		lph *= 2;
	}
	return lph;
}

struct Grid {
	unsigned blocks;
	bool ok;
};
Grid grid_for(const SparseArgs &a)
{
	const int hpw = 32 / a.lph;
	const long long warps = (long long)a.bs * a.n_tok * ((a.n_heads + hpw - 1) / hpw);
	const long long blocks = (warps + 7) / 8;
	return {unsigned(blocks), blocks <= 0x7fffffffLL};
}

template <typename S, typename T, int VEC>
int fwd_t(SparseArgs a, const S *v, const S *vb, const S *q, const S *k, S *vo, S *attn, cudaStream_t st)
{
	const int mw = a.width > a.v_width ? a.width : a.v_width;
	a.lph = lanes_per_head(mw, a.n_heads, VEC, 2);
	const Grid g = grid_for(a);
	if (!g.ok)
		return L1ATTN_ERR_SHAPE;
	const T scale = T(-1.0 / sqrt(double(a.width)));
	// lanes per head as a compile-time constant for the common widths (16-byte vectors, 32..128+ columns)
#define L1B_FWD(LP, NXV)                                                                                      \
	do {                                                                                             \
		sparse_fwd_dst_kernel<S, T, VEC, LP, NXV><<<g.blocks, 256, 0, st>>>(a, v, q, k, vo, attn, scale); \
		L1B_LAUNCH_CHECK();                                                                      \
		if (a.bidi) {                                                                            \
			sparse_fwd_src_kernel<S, T, VEC, LP, NXV><<<g.blocks, 256, 0, st>>>(a, vb, attn, vo);     \
			L1B_LAUNCH_CHECK();                                                              \
		}                                                                                        \
	} while (0)
	// four vectors per lane exactly (width == v_width == 16 * lanes-per-head elements of 16-byte vectors): unrolled walk
	const bool nx4 = VEC > 1 && a.width == a.v_width && a.width == 4 * a.lph * VEC;
	if (nx4 && a.lph == 4)
		L1B_FWD(4, 4);
	else if (nx4 && a.lph == 8)
		L1B_FWD(8, 4);
	else if (nx4 && a.lph == 16)
		L1B_FWD(16, 4);
	else if (nx4 && a.lph == 32)
		L1B_FWD(32, 4);
	else if (VEC > 1 && a.lph == 4)
		L1B_FWD(4, 0);
	else if (VEC > 1 && a.lph == 8)
		L1B_FWD(8, 0);
	else if (VEC > 1 && a.lph == 16)
		L1B_FWD(16, 0);
	else if (VEC > 1 && a.lph == 32)
		L1B_FWD(32, 0);
	else
		L1B_FWD(0, 0);
#undef L1B_FWD
	return L1ATTN_OK;
}

template <typename T, int VEC>
int bwd_t(SparseArgs a, const T *dvo, const T *v, const T *vb, const T *q, const T *k, const T *attn, T *d_v,
	  T *d_vb, T *d_q, T *d_k, T *dx, cudaStream_t st)
{
	const int mw = a.width > a.v_width ? a.width : a.v_width;
	// (two vectors per lane, twice the warps at ~75 registers, measured 2 % slower than four at 8 heads)
	a.lph = lanes_per_head(mw, a.n_heads, VEC, 4);
	const Grid g = grid_for(a);
	if (!g.ok)
		return L1ATTN_ERR_SHAPE;
	const T scale = T(-1.0 / sqrt(double(a.width)));
#define L1B_BWD(LP, NXV)                                                                                                       \
	do {                                                                                                              \
		if (a.bidi)                                                                                               \
			sparse_bwd_dst_kernel<T, VEC, LP, NXV, true><<<g.blocks, 256, 0, st>>>(a, dvo, v, vb, q, k, attn, dx, d_q, d_vb, scale); \
		else                                                                                                      \
			sparse_bwd_dst_kernel<T, VEC, LP, NXV, false><<<g.blocks, 256, 0, st>>>(a, dvo, v, vb, q, k, attn, dx, d_q, d_vb, scale); \
		L1B_LAUNCH_CHECK();                                                                                       \
		sparse_bwd_src_kernel<T, VEC, LP, NXV><<<g.blocks, 256, 0, st>>>(a, dvo, q, k, attn, dx, d_v, d_k, scale);        \
		L1B_LAUNCH_CHECK();                                                                                       \
	} while (0)
	// four vectors per lane exactly (width == v_width == 16 * lanes-per-head elements of 16-byte vectors): unrolled walk
	const bool nx4 = VEC > 1 && a.width == a.v_width && a.width == 4 * a.lph * VEC;
	if (nx4 && a.lph == 4)
		L1B_BWD(4, 4);
	else if (nx4 && a.lph == 8)
		L1B_BWD(8, 4);
	else if (nx4 && a.lph == 16)
		L1B_BWD(16, 4);
	else if (nx4 && a.lph == 32)
		L1B_BWD(32, 4);
	else if (VEC > 1 && a.lph == 4)
		L1B_BWD(4, 0);
	else if (VEC > 1 && a.lph == 8)
		L1B_BWD(8, 0);
	else if (VEC > 1 && a.lph == 16)
		L1B_BWD(16, 0);
	else if (VEC > 1 && a.lph == 32)
		L1B_BWD(32, 0);
	else
		L1B_BWD(0, 0);
#undef L1B_BWD
	return L1ATTN_OK;
}

bool all_aligned16(std::initializer_list<const void *> ps)
{
	for (const void *p : ps)
		if (p && !aligned(p, 16))
			return false;
	return true;
}

} // namespace
} // namespace l1b

using namespace l1b;

extern "C" size_t l1attn_sparse_bwd_scratch_bytes(int bs, int n_tok, int n_heads, int dst_mxlen, int dtype)
{
	if (bs < 0 || n_tok < 0 || n_heads < 0 || dst_mxlen < 0)
		return 0;
	const size_t n = size_t(bs) * n_tok * dst_mxlen * n_heads * (dtype == L1ATTN_F64 ? 8 : 4);
	return n ? n : 16;
}

static int check_sparse(int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen, int dtype,
			bool allow16 = false)
{
	if (bs < 0 || n_tok < 0 || n_heads < 0 || width < 1 || v_width < 1 || cl < 0 || dst_mxlen < 0)
		return L1ATTN_ERR_ARG;
	const bool is16 = dtype == L1ATTN_F16 || dtype == L1ATTN_BF16;
	if (dtype != L1ATTN_F32 && dtype != L1ATTN_F64 && !(allow16 && is16))
		return L1ATTN_ERR_ARG;
	if ((long long)n_tok * dst_mxlen > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	return L1ATTN_OK;
}

extern "C" int l1attn_sparse_fwd(const void *v, const void *vb, const void *q, const void *k, const void *index,
				  void *vo, void *attn, int bs, int n_tok, int n_heads, int width, int v_width, int cl,
				  int dst_mxlen, int use_softmax, int bidi, int dtype, void *stream)
{
	int rc = check_sparse(bs, n_tok, n_heads, width, v_width, cl, dst_mxlen, dtype, true);
	if (rc)
		return rc;
	if (bs == 0 || n_tok == 0 || n_heads == 0)
		return L1ATTN_OK;
	if (!v || !q || !k || !index || !vo || !attn || (bidi && !vb))
		return L1ATTN_ERR_ARG;
	const size_t es = dtype == L1ATTN_F64 ? 8 : dtype == L1ATTN_F32 ? 4 : 2;
	for (const void *p : {v, vb, q, k, (const void *)vo, (const void *)attn})
		if (p && !aligned(p, es))
			return L1ATTN_ERR_ALIGN;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	SparseIndex ix = sparse_index_view(const_cast<void *>(index), cl, n_tok, dst_mxlen);
	SparseArgs a{bs, n_tok, n_heads, width, v_width, dst_mxlen, 32, use_softmax != 0, bidi != 0,
		     ix.slot_src, ix.csc_off, ix.csc_slot};
	const bool a16 = all_aligned16({v, vb, q, k, vo});
	if (dtype == L1ATTN_F16 || dtype == L1ATTN_BF16) {
		// 16-bit storage, float arithmetic: four elements (8 bytes) per load when rows allow it
		bool a8 = width % 4 == 0 && v_width % 4 == 0;
		for (const void *p : {v, vb, q, k, (const void *)vo})
			a8 = a8 && (!p || aligned(p, 8));
		if (dtype == L1ATTN_F16) {
			using H = __half;
			if (a8)
				return fwd_t<H, float, 4>(a, (const H *)v, (const H *)vb, (const H *)q, (const H *)k, (H *)vo, (H *)attn, st);
			return fwd_t<H, float, 1>(a, (const H *)v, (const H *)vb, (const H *)q, (const H *)k, (H *)vo, (H *)attn, st);
		}
		using B = __nv_bfloat16;
		if (a8)
			return fwd_t<B, float, 4>(a, (const B *)v, (const B *)vb, (const B *)q, (const B *)k, (B *)vo, (B *)attn, st);
		return fwd_t<B, float, 1>(a, (const B *)v, (const B *)vb, (const B *)q, (const B *)k, (B *)vo, (B *)attn, st);
	}
	if (dtype == L1ATTN_F32) {
		if (a16 && width % 4 == 0 && v_width % 4 == 0)
			return fwd_t<float, float, 4>(a, (const float *)v, (const float *)vb, (const float *)q, (const float *)k,
					       (float *)vo, (float *)attn, st);
		return fwd_t<float, float, 1>(a, (const float *)v, (const float *)vb, (const float *)q, (const float *)k,
				       (float *)vo, (float *)attn, st);
	}
	if (a16 && width % 2 == 0 && v_width % 2 == 0)
		return fwd_t<double, double, 2>(a, (const double *)v, (const double *)vb, (const double *)q, (const double *)k,
					(double *)vo, (double *)attn, st);
	return fwd_t<double, double, 1>(a, (const double *)v, (const double *)vb, (const double *)q, (const double *)k,
				(double *)vo, (double *)attn, st);
}

extern "C" int l1attn_sparse_bwd(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
				  const void *index, const void *attn, void *d_v, void *d_vb, void *d_q, void *d_k,
				  void *scratch, int bs, int n_tok, int n_heads, int width, int v_width, int cl,
				  int dst_mxlen, int use_softmax, int bidi, int dtype, void *stream)
{
	int rc = check_sparse(bs, n_tok, n_heads, width, v_width, cl, dst_mxlen, dtype);
	if (rc)
		return rc;
	if (bs == 0 || n_tok == 0 || n_heads == 0)
		return L1ATTN_OK;
	if (!dvo || !v || !q || !k || !index || !attn || !d_v || !d_q || !d_k || !scratch || (bidi && (!vb || !d_vb)))
		return L1ATTN_ERR_ARG;
	const size_t es = dtype == L1ATTN_F64 ? 8 : 4;
	for (const void *p : {dvo, v, vb, q, k, attn, (const void *)d_v, (const void *)d_vb, (const void *)d_q,
			      (const void *)d_k, (const void *)scratch})
		if (p && !aligned(p, es))
			return L1ATTN_ERR_ALIGN;
	cudaStream_t st = static_cast<cudaStream_t>(stream);
	SparseIndex ix = sparse_index_view(const_cast<void *>(index), cl, n_tok, dst_mxlen);
	SparseArgs a{bs, n_tok, n_heads, width, v_width, dst_mxlen, 32, use_softmax != 0, bidi != 0,
		     ix.slot_src, ix.csc_off, ix.csc_slot};
	const bool a16 = all_aligned16({dvo, v, vb, q, k, d_v, d_vb, d_q, d_k});
	if (dtype == L1ATTN_F32) {
		if (a16 && width % 4 == 0 && v_width % 4 == 0)
			return bwd_t<float, 4>(a, (const float *)dvo, (const float *)v, (const float *)vb, (const float *)q,
					       (const float *)k, (const float *)attn, (float *)d_v, (float *)d_vb,
					       (float *)d_q, (float *)d_k, (float *)scratch, st);
		return bwd_t<float, 1>(a, (const float *)dvo, (const float *)v, (const float *)vb, (const float *)q,
				       (const float *)k, (const float *)attn, (float *)d_v, (float *)d_vb, (float *)d_q,
				       (float *)d_k, (float *)scratch, st);
	}
	if (a16 && width % 2 == 0 && v_width % 2 == 0)
		return bwd_t<double, 2>(a, (const double *)dvo, (const double *)v, (const double *)vb, (const double *)q,
					(const double *)k, (const double *)attn, (double *)d_v, (double *)d_vb,
					(double *)d_q, (double *)d_k, (double *)scratch, st);
	return bwd_t<double, 1>(a, (const double *)dvo, (const double *)v, (const double *)vb, (const double *)q,
				(const double *)k, (const double *)attn, (double *)d_v, (double *)d_vb, (double *)d_q,
				(double *)d_k, (double *)scratch, st);
}

// ------------------------------------------------------------------------------------------------
// Sparse backward for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc where they run the backward: a plugin that is
// handed device pointers by an embedding runtime and has no allocator of its own, or code inside a
// region where allocation is forbidden or would synchronise the device.  For them the per-slot
// d(logit) buffer that l1attn_sparse_bwd takes as `scratch` lives here, in a fixed array in the
// library's device image.  Every GPU that loads the library carries these 32 MiB until the process
// exits, and every call on a device shares them, so two such calls that overlap on the GPU (different
// streams) race; calls on one stream are safe.  Nothing in the array has to start at zero: the dst
// pass writes the entry of every real edge slot before the src pass reads it, and entries of empty
// slots are never read, so stale contents of an earlier call are harmless.
constexpr size_t STATIC_SCRATCH_BYTES = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_sparse_bwd_scratch[STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
void *g_scratch_addr[MAX_DEVICES]; // device address of the array, per device, filled on first use
std::mutex g_scratch_mu;

// In host code the array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked for once per device with that device current.
int static_scratch_for_current_device(void **out)
{
	int dev = 0;
	L1B_CUDA(cudaGetDevice(&dev));
	if (dev < 0 || dev >= MAX_DEVICES)
		return L1ATTN_ERR_ARG;
	std::lock_guard<std::mutex> lock(g_scratch_mu);
	if (!g_scratch_addr[dev]) {
		void *p = nullptr;
		L1B_CUDA(cudaGetSymbolAddress(&p, g_sparse_bwd_scratch));
		g_scratch_addr[dev] = p;
	}
	*out = g_scratch_addr[dev];
	return L1ATTN_OK;
}
} // namespace

extern "C" size_t l1attn_sparse_bwd_static_capacity(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int l1attn_sparse_bwd_static(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
					 const void *index, const void *attn, void *d_v, void *d_vb, void *d_q,
					 void *d_k, int bs, int n_tok, int n_heads, int width, int v_width, int cl,
					 int dst_mxlen, int use_softmax, int bidi, int dtype, void *stream)
{
	int rc = check_sparse(bs, n_tok, n_heads, width, v_width, cl, dst_mxlen, dtype);
	if (rc)
		return rc;
	if (l1attn_sparse_bwd_scratch_bytes(bs, n_tok, n_heads, dst_mxlen, dtype) > STATIC_SCRATCH_BYTES)
		return L1ATTN_ERR_SCRATCH;
	void *scratch = nullptr;
	if ((rc = static_scratch_for_current_device(&scratch)))
		return rc;
	return l1attn_sparse_bwd(dvo, v, vb, q, k, index, attn, d_v, d_vb, d_q, d_k, scratch, bs, n_tok, n_heads, width,
				 v_width, cl, dst_mxlen, use_softmax, bidi, dtype, stream);
}
