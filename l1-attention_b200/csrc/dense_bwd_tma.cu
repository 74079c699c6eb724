// Dense L1 scores, backward -- the B200 fast path (fp32).
//
//   d_q[b][t][h][w] =  scale * sum_s sign(q[b][t][h][w] - k[b][s][h][w]) * g[b][s][t][h]
//   d_k[b][s][h][w] = -scale * sum_t sign(q[b][t][h][w] - k[b][s][h][w]) * g[b][s][t][h]     sign(0) = 0
//
// Both are  out[x][h][w] = scale * sum_y sign(a[x][h][w] - b[y][h][w]) * G(x, y, h)
// (pass 0: a=q, b=k, x=t, y=s;  pass 1: a=k, b=q, x=s, y=t;  G(x,y,h) = g[s][t][h] either way).
// Each output element is owned by one thread and summed in a fixed order: no atomics, no scratch
// partials, bit-reproducible.  The price is that every term is visited twice (once per pass); the
// gain is that a visit is two instructions.
//
// Two instructions per term.  With no ties (a != b) in a tile,
//     sum_y sign(a-b) G = 2 * sum_y [a > b] G  -  sum_y G,
// so the inner loop is one compare (FSETP) and one predicated add per term; the row sums
// sum_y G(x,y,h) are a by-product (4 extra adds per 32 terms).  A warp (4 x rows, 8 heads, 32 width
// columns) may use this form on a y tile unless a detector kernel (dense_ties.cu) has found a row among
// its x rows AND one in the y tile that take part in a tie a == b (same batch, head group, width group); such pairs run the
// exact loop (subtract, sign transfer, tie predicate, add) on halved G, so that one accumulator
// serves both forms: out = scale * (2 acc - R), R summed over the compare-form tiles only.
// Exact ties between random floats occur ~1.5e-8 per term (a few hundred per call at 16x1024x16x64),
// zero-padded tokens tie everywhere; both cases stay exact and cost the exact loop only where they occur.
//
// Structure: one persistent launch for both passes, one CTA per SM, work item = (batch, 8 heads, 32 x-rows,
// all 64 width columns of a 64-wide slice).  One thread streams y in tiles of 16 through a 4-stage
// ring of TMA tensor loads (no multicast): the b rows as two [y][head][32 w] boxes with the 128-byte
// swizzle, and the G tile as a [.][.][8 heads] box of the heads-innermost gradient tensor -- 32-byte
// runs, whole sectors, no transposed copy of d_attn (the reference makes one).  16 warps:
// lanes = 8 heads x 4 width chunks, a thread owns 4 x-rows x 8 width columns of one head (32 `a`
// values and 32 accumulators in registers) and per y reads 2 x 16 bytes of b and 4 G scalars.
// (8 warps with 8 x 8 tiles measured half the speed: with two warps per scheduler the
// compare -> predicated-add latency was exposed, "wait" stalls of ~5 cycles per instruction.)
// All mbarrier waits are bounded (tma.cuh).
#include <type_traits>
#include "common.cuh"
#include "tma.cuh"
#include "dense_bwd_tiles.h"

namespace l1b {
namespace {

constexpr int HG = BWD_HG; // heads per work item = lanes along heads (8)
constexpr int TX = BWD_TX; // x rows per work item (32)
constexpr int TY = BWD_TY; // y rows per stage (16)
constexpr int WS = BWD_WS; // width slice per work item (64 = two 32-wide halves)
constexpr int NCW = 16;  // warps: 8 x-groups of XR rows x 2 halves of the chunk range
constexpr int XR = 4;    // x rows per thread
static_assert(XR == BWD_XF && WS == 2 * BWD_WF, "a warp owns one x flag and one width group");
constexpr int NSTAGE = 4;
constexpr int B_BYTES = TY * HG * 32 * 4;  // one 32-wide half of the b tile: 16384
constexpr int G_BYTES = TY * TX * HG * 4;  // 16384
constexpr int STAGE_BYTES = 2 * B_BYTES + G_BYTES; // 49152
constexpr int NTHREADS = NCW * 32; // 512 threads x 128 registers; 4 warps per scheduler hide the compare->add latency

struct BwdWork {
	unsigned nxt, nws, nhg, bs, per_pass, total;
	int ny; // y tiles per item
};
struct BwdItem {
	int b, h0, w0, x0;
};
__device__ __forceinline__ BwdItem decode(const BwdWork &wk, unsigned r)
{
	BwdItem it;
	// width slices of one x tile are neighbours in the item order: the CTAs that work on them at the same
	// time stream the same G tiles, so the second reader finds them in L2 (matters when width > 64)
	it.w0 = int(r % wk.nws) * WS;
	r /= wk.nws;
	it.x0 = int(r % wk.nxt) * TX;
	r /= wk.nxt;
	it.h0 = int(r % wk.nhg) * HG;
	it.b = int(r / wk.nhg);
	return it;
}

// one stage (TY rows of y) of the inner loop for the calling thread
template <int PASS, bool EXACT>
__device__ __forceinline__ void tile_loop(const unsigned char *stage, int h, int c, int wx, int wp, const float (&a)[XR][8],
					  float (&acc)[XR][8], float (&rs)[XR])
{
	const float4 *B0 = reinterpret_cast<const float4 *>(stage);
	const float4 *B1 = reinterpret_cast<const float4 *>(stage + B_BYTES);
	const float *G = reinterpret_cast<const float *>(stage + 2 * B_BYTES);
	// G tile layout: pass 0 [y][x][h], pass 1 [x][y][h]
	const float *gp = G + (PASS == 0 ? (wx * XR) * HG : (wx * XR) * TY * HG) + h;
	constexpr int GI = PASS == 0 ? HG : TY * HG;  // stride between this thread's x rows
	constexpr int GY = PASS == 0 ? TX * HG : HG;  // stride between y rows
	const int boff = h * 8 + (c ^ h); // 128-byte swizzle: chunk ^= (row & 7), row = y*8 + h
#pragma unroll 4
	for (int y = 0; y < TY; y++) {
		const float4 b0 = B0[y * 64 + boff], b1 = B1[y * 64 + boff];
		const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
		float g[XR];
#pragma unroll
		for (int i = 0; i < XR; i++)
			g[i] = gp[y * GY + i * GI];
		if (!EXACT) {
#pragma unroll
			for (int i = 0; i < XR; i++)
				rs[i] += g[i];
		}
		if (EXACT) {
#pragma unroll
			for (int i = 0; i < XR; i++)
#pragma unroll
				for (int e = 0; e < 8; e++) // halves: the epilogue doubles every accumulator (exact in binary fp)
					acc[i][e] += sign_apply(a[i][e] - bv[e], 0.5f * g[i]);
		} else {
			// compare + predicated add, spelled in PTX four terms at a time (four compares, then four
			// adds): left to the compiler the term becomes compare + add + select, two instructions on
			// the half-rate ALU pipe, and single compare/add pairs were scheduled back to back with
			// the compare latency exposed
#pragma unroll
			for (int i = 0; i < XR; i++)
#pragma unroll
				for (int e = 0; e < 8; e += 4)
					asm("{\n\t.reg .pred p0, p1, p2, p3;\n\t"
					    "setp.gt.f32 p0, %4, %8;\n\tsetp.gt.f32 p1, %5, %9;\n\t"
					    "setp.gt.f32 p2, %6, %10;\n\tsetp.gt.f32 p3, %7, %11;\n\t"
					    "@p0 add.f32 %0, %0, %12;\n\t@p1 add.f32 %1, %1, %12;\n\t"
					    "@p2 add.f32 %2, %2, %12;\n\t@p3 add.f32 %3, %3, %12;\n\t}"
					    : "+f"(acc[i][e]), "+f"(acc[i][e + 1]), "+f"(acc[i][e + 2]), "+f"(acc[i][e + 3])
					    : "f"(a[i][e]), "f"(a[i][e + 1]), "f"(a[i][e + 2]), "f"(a[i][e + 3]), "f"(bv[e]),
					      "f"(bv[e + 1]), "f"(bv[e + 2]), "f"(bv[e + 3]), "f"(g[i]));
		}
	}
}

// The hot loop needs the predicate registers (only seven exist) for its compare -> add pairs.  Any
// boolean that stays live across that loop (bounds tests reused by the epilogue, "is thread 0", "has a
// wait timed out") takes one away, and with one or two left the pairs run strictly one after the
// other.  Passing the integers such tests are made from through this no-op makes the compiler
// recompute the test where it is used instead of keeping its result in a predicate.
__device__ __forceinline__ int opaque(int x)
{
	asm volatile("" : "+r"(x));
	return x;
}

// Work items [0, per_pass) are pass 0: d_q (a = q, b = k, x = t, y = s); items [per_pass, 2 per_pass) are
// pass 1: d_k (a = k, b = q, x = s, y = t).  One launch walks both, so the last wave of CTAs is as
// full as the item count allows; the per-item code is compiled once per pass (generic lambda).
__global__ void __launch_bounds__(NTHREADS, 1)
dense_bwd_tma_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
		     const __grid_constant__ CUtensorMap gmap0, const __grid_constant__ CUtensorMap gmap1,
		     const float *__restrict__ q, const float *__restrict__ k, float *__restrict__ d_q,
		     float *__restrict__ d_k, const unsigned char *__restrict__ flags, BwdFlagLayout fl, int n_tok,
		     int n_heads, int width, float scale, BwdWork wk, const int *__restrict__ tie_hdr, int only_on_overflow,
		     int *err)
{
	if (only_on_overflow != 0 && tie_hdr[1] == 0)
		return; // the single-visit kernel (dense_bwd_sv.cu) has computed this call
	// Every tie of this call is in the detector's list (no overflow): all tiles take the compare form and the fix
	// kernel repairs the listed terms afterwards.  Otherwise the per-tile flags choose the exact loop.
	const int listed = (tie_hdr != nullptr && tie_hdr[1] == 0) ? 1 : 0;
	extern __shared__ __align__(1024) unsigned char smem_raw[];
	// 1024-byte alignment by OFFSET into the shared array: a pointer rebuilt from an integer loses its
	// address space and every access through it becomes a generic load, which measured ~2x slower here
	unsigned char *stages = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
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

	// The ring runs NSTAGE-2 tiles ahead of the math.  The n-th tile this CTA consumes (n counts across
	// work items) lives in stage n % NSTAGE.  While the warps work on tile n, ONE lane requests tile
	// n + NSTAGE-2, whose stage every warp released two tiles ago, so the requester normally does not
	// wait.  The duty rotates over the warps (tile n -> warp n % 16): a fixed issuing thread made its
	// warp slower than the others, and the whole CTA ran at that warp's pace.
	// issue_tile(it, yt, m): request y tile `yt` of work item `it` as ring entry m; yt may run past the
	// item's last tile and then names a tile of the CTA's following items.
	auto issue_tile = [&](unsigned it, int yt, unsigned m) -> bool {
		while (yt >= wk.ny) {
			yt -= wk.ny;
			it += gridDim.x;
		}
		if (it >= wk.total)
			return true;
		const int st = int(m % NSTAGE);
		if (!mbar_wait(&empty_bar[st], ((m / NSTAGE) & 1u) ^ 1u, err))
			return false;
		const bool pass1 = it >= wk.per_pass;
		const BwdItem x = decode(wk, pass1 ? it - wk.per_pass : it);
		const CUtensorMap *bm = pass1 ? &qmap : &kmap;
		unsigned char *dst = stages + size_t(st) * STAGE_BYTES;
		const int y0 = yt * TY;
		mbar_expect_tx(&full_bar[st], STAGE_BYTES);
		tma_load_4d(dst, bm, &full_bar[st], x.w0, x.h0, y0, x.b);
		tma_load_4d(dst + B_BYTES, bm, &full_bar[st], x.w0 + 32, x.h0, y0, x.b);
		if (!pass1) // box {8 h, TX t, TY s}
			tma_load_4d(dst + 2 * B_BYTES, &gmap0, &full_bar[st], x.h0, x.x0, y0, x.b);
		else // box {8 h, TY t, TX s}
			tma_load_4d(dst + 2 * B_BYTES, &gmap1, &full_bar[st], x.h0, y0, x.x0, x.b);
		return true;
	};
	if (tid == 0)
		for (int i = 0; i < NSTAGE - 2; i++)
			issue_tile(blockIdx.x, i, unsigned(i));

	const int lh = lane & 7, lw = lane >> 3;
	const int wx = warp & 7, wp = warp >> 3;
	const int c = lw + 4 * wp; // 16-byte chunk (0..7) of each 32-wide half
	static_assert((NSTAGE & (NSTAGE - 1)) == 0, "stage index and parity are bit fields of the tile counter");
	unsigned n = 0; // tiles consumed by this CTA so far
	int dead = 0;
	auto run_item = [&](auto pass_tag, unsigned item) {
		constexpr int PASS = decltype(pass_tag)::value;
		const float *av_base = PASS == 0 ? q : k;
		float *out_base = PASS == 0 ? d_q : d_k;
		float a[XR][8], acc[XR][8], rs[XR] = {0.f, 0.f, 0.f, 0.f};
		{
			const BwdItem x = decode(wk, item);
			const int h = x.h0 + lh;
			const size_t row = size_t(n_heads) * width;
			const float *av = av_base + size_t(x.b) * n_tok * row + size_t(h) * width;
#pragma unroll
			for (int i = 0; i < XR; i++) {
				const int xr = x.x0 + wx * XR + i;
#pragma unroll
				for (int half = 0; half < 2; half++) {
					const int w = x.w0 + half * 32 + c * 4;
					float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
					if (xr < n_tok && h < n_heads && w < width)
						v = *reinterpret_cast<const float4 *>(av + size_t(xr) * row + w);
					a[i][half * 4 + 0] = v.x;
					a[i][half * 4 + 1] = v.y;
					a[i][half * 4 + 2] = v.z;
					a[i][half * 4 + 3] = v.w;
				}
#pragma unroll
				for (int e = 0; e < 8; e++)
					acc[i][e] = 0.f;
			}
		}
		// exact loop where a tile with a tying x row meets a tile with a tying y row (or always, without flags)
		// (this warp's 4 x rows and its 32 width columns; the flag arrays are padded to whole tiles and slices)
		int xflag = 1;
		const unsigned char *yflags = nullptr;
		if (opaque(listed) != 0) {
			xflag = 0;
		} else if (flags != nullptr) {
			const BwdItem x = decode(wk, item);
			const size_t g = fl.group(x.b, x.h0, x.w0 + wp * 16); // this warp's columns: (w % 32) / 16 == wp
			xflag = int(flags[fl.xoff(PASS) + g * fl.nxf + size_t(x.x0 + wx * XR) / BWD_XF]);
			yflags = flags + fl.yoff(PASS) + g * fl.ny;
		}

		// The walk over the y tiles is compiled twice: for the warps whose x rows hold no tie (nearly all
		// of them) the loop contains the compare form only -- with both forms in one loop the compiler
		// spent ~6 % more instructions on the common path.
		auto walk = [&](auto may_tie) {
			constexpr bool MAY_TIE = decltype(may_tie)::value;
			for (int yt = 0; yt < wk.ny; yt++) {
				if (opaque(tid) == int((n % NCW) * 32) && opaque(dead) == 0 &&
				    !issue_tile(item + PASS * wk.per_pass, yt + NSTAGE - 2, n + NSTAGE - 2))
					dead = 1;
				__syncwarp();
				const int st = int(n % NSTAGE);
				if (opaque(dead) == 0 && !mbar_wait(&full_bar[st], (n / NSTAGE) & 1u, err))
					dead = 1; // keep walking without waiting so the warps stay in step
				const unsigned char *stage = stages + size_t(st) * STAGE_BYTES;
				if (MAY_TIE && (yflags == nullptr || yflags[yt] != 0))
					tile_loop<PASS, true>(stage, lh, c, wx, wp, a, acc, rs);
				else
					tile_loop<PASS, false>(stage, lh, c, wx, wp, a, acc, rs);
				__syncwarp();
				if (opaque(lane) == 0)
					mbar_arrive(&empty_bar[st]);
				n++;
			}
		};
		if (xflag != 0)
			walk(std::true_type{});
		else
			walk(std::false_type{});

		const BwdItem x = decode(wk, unsigned(opaque(int(item))));
		const int h = x.h0 + opaque(lh);
		const size_t row = size_t(n_heads) * width;
		float *ov = out_base + size_t(x.b) * n_tok * row + size_t(h) * width;
#pragma unroll
		for (int i = 0; i < XR; i++) {
			const int xr = x.x0 + wx * XR + i;
			const float r = rs[i]; // sum of G(x, y, h) over the y tiles that took the compare form
#pragma unroll
			for (int half = 0; half < 2; half++) {
				const int w = x.w0 + half * 32 + c * 4;
				if (xr < n_tok && h < n_heads && w < width) {
					float4 o;
					float *op = reinterpret_cast<float *>(&o);
#pragma unroll
					for (int e = 0; e < 4; e++)
						op[e] = fmaf(2.f, acc[i][half * 4 + e], -r) * scale;
					*reinterpret_cast<float4 *>(ov + size_t(xr) * row + w) = o;
				}
			}
		}
	};
	for (unsigned item = blockIdx.x; item < wk.total; item += gridDim.x) {
		if (item < wk.per_pass)
			run_item(std::integral_constant<int, 0>{}, item);
		else
			run_item(std::integral_constant<int, 1>{}, item - wk.per_pass);
	}
}

} // namespace

// Returns L1ATTN_OK, a negative error, or 1 when this path does not apply.
// flags: device tie flags laid out by bwd_flag_layout() and filled by dense_ties_launch(), or nullptr = all exact.
int dense_bwd_tma_launch(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, int bs, int n_tok,
			 int n_heads, int width, int dtype, const unsigned char *flags, const int *tie_hdr, int only_on_overflow,
			 cudaStream_t st)
{
	if (dtype != L1ATTN_F32)
		return 1;
	if (width % 4 != 0 || n_heads % 4 != 0)
		return 1; // row pitches of q/k and of d_attn must be multiples of 16 bytes for the tensor maps
	for (const void *p : {d_attn, q, k, (const void *)d_q, (const void *)d_k})
		if (!aligned(p, 16))
			return 1;
	const uint64_t qdims[4] = {uint64_t(width), uint64_t(n_heads), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t qstr[3] = {uint64_t(width) * 4, uint64_t(n_heads) * width * 4, uint64_t(n_tok) * n_heads * width * 4};
	const uint32_t bbox[4] = {32, HG, TY, 1};
	const uint64_t gdims[4] = {uint64_t(n_heads), uint64_t(n_tok), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t gstr[3] = {uint64_t(n_heads) * 4, uint64_t(n_tok) * n_heads * 4, uint64_t(n_tok) * n_tok * n_heads * 4};
	const uint32_t gbox0[4] = {HG, TX, TY, 1}, gbox1[4] = {HG, TY, TX, 1};
	CUtensorMap qmap, kmap, gmap0, gmap1;
	if (!encode_tmap_4d(&qmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, q, qdims, qstr, bbox, CU_TENSOR_MAP_SWIZZLE_128B) ||
	    !encode_tmap_4d(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, k, qdims, qstr, bbox, CU_TENSOR_MAP_SWIZZLE_128B) ||
	    !encode_tmap_4d(&gmap0, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, d_attn, gdims, gstr, gbox0, CU_TENSOR_MAP_SWIZZLE_NONE) ||
	    !encode_tmap_4d(&gmap1, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, d_attn, gdims, gstr, gbox1, CU_TENSOR_MAP_SWIZZLE_NONE))
		return 1;
	int *err = device_error_word();
	if (!err)
		return 1;
	BwdWork wk;
	wk.nxt = (n_tok + TX - 1) / TX;
	wk.nws = (width + WS - 1) / WS;
	wk.nhg = (n_heads + HG - 1) / HG;
	wk.bs = bs;
	const long long per_pass = (long long)bs * wk.nhg * wk.nws * wk.nxt;
	if (2 * per_pass > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	wk.per_pass = unsigned(per_pass);
	wk.total = unsigned(2 * per_pass);
	wk.ny = (n_tok + TY - 1) / TY;
	int dev = 0, sms = 0;
	L1B_CUDA(cudaGetDevice(&dev));
	L1B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
	const unsigned grid = wk.total < unsigned(sms) ? wk.total : unsigned(sms);
	const size_t smem = size_t(NSTAGE) * STAGE_BYTES + 1024;
	L1B_CUDA(cudaFuncSetAttribute(dense_bwd_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	const float scale = float(-1.0 / sqrt(double(width)));
	const BwdFlagLayout fl = bwd_flag_layout(bs, n_tok, n_heads, width);
	dense_bwd_tma_kernel<<<grid, NTHREADS, smem, st>>>(qmap, kmap, gmap0, gmap1, (const float *)q, (const float *)k,
							    (float *)d_q, (float *)d_k, flags, fl, n_tok, n_heads, width, scale,
							    wk, tie_hdr, (tie_hdr != nullptr && only_on_overflow) ? 1 : 0, err);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace l1b
