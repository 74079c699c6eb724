// Dense L1 scores, backward -- the B200 fast path (fp32): both gradients from ONE visit of every term.
//
//   d_q[b][t][h][w] =  scale * sum_s sign(q[b][t][h][w] - k[b][s][h][w]) * g[b][s][t][h]
//   d_k[b][s][h][w] = -scale * sum_t sign(q[b][t][h][w] - k[b][s][h][w]) * g[b][s][t][h]     sign(0) = 0
//
// Per term (b, s, t, h, w) one compare p = [q > k] and two predicated adds of g: into the d_q accumulator of
// (t, w) and into the d_k accumulator of (s, w).  With no ties, sum sign(q - k) g = 2 sum p g - sum g on
// either side; the plain sums of g are by-products.  Three instructions per term for both gradients; the
// two-pass kernel (dense_bwd_tma.cu) spends two per term and gradient.  The kernels are bound by instruction
// issue (one warp instruction per scheduler and clock, whatever the pipe), so that is the number that counts.
// A tie q == k counts as -g here and is repaired afterwards from the detector's list (dense_ties.cu); when
// the list overflows the kernels of this file return at once and the two-pass kernel does the call.
//
// Work item = (batch, 4 heads, 32 width columns, 128 query rows t).  Thread = ONE width column of one head x 32
// query rows: the lanes of a warp are the 32 columns, so for a source row s the k value is one coalesced 4-byte
// shared load and g[s][t..t+3][h] one BROADCAST 16-byte load -- if g lies [s][h][t] in shared memory.  It
// arrives [s][t][h] (heads are innermost in d_attn and a TMA box keeps the tensor's order), so every tile is
// transposed on its way from the raw TMA stage to the stage the math reads: after its share of tile n each of the 16
// warps (4 groups of 32 query rows x 4 heads) transposes one source row of tile n+1 and sums it over t while it is
// at it.  (Two extra warps for that job would push the CTA past 16 warps and with it below the ~105 registers the
// math needs: measured 5.2 instead of 3.7 instructions per term.)  One lane issues the TMA requests.  One mbarrier
// per tile orders all of it (see the kernel); every wait is bounded.
//
// d_q is complete in registers at the end of an item.  d_k is not: per source row a warp holds the sum over
// its 32 query rows.  The four row groups' partials of a tile meet in shared memory (double-buffered, summed in a
// fixed order by the compute warps themselves, one tile behind the math) and the item's share of d_k -- its
// 128 query rows' -- goes to scratch; dense_bwd_sv_partsum_kernel adds the n_tok/128 shares in order.  No
// atomics anywhere: bit-reproducible.
#include "common.cuh"
#include "tma.cuh"
#include "dense_bwd_tiles.h"

namespace l1b {
namespace {

constexpr int SV_HG = 4;          // heads per work item
constexpr int SV_WS = 32;         // width columns per work item = lanes
constexpr int SV_TX = BWD_SV_TX;  // query rows per work item (128)
constexpr int SV_XR = 32;         // query rows per thread
constexpr int SV_TY = 16;         // source rows per tile
constexpr int SV_NCW = 16;        // warps: (SV_TX / SV_XR) row groups x SV_HG heads; also one source row of a tile each to transpose
constexpr int SV_THREADS = SV_NCW * 32;
constexpr int SV_RAW_BYTES = SV_TY * SV_TX * SV_HG * 4;  // 32768: g as it arrives, [s][t][h]
constexpr int SV_GT_BYTES = SV_RAW_BYTES;                 // 32768: g transposed, [s][h][t]
constexpr int SV_B_BYTES = SV_TY * SV_HG * SV_WS * 4;     // 8192: k rows, [s][h][32 w]
constexpr int SV_CS_BYTES = SV_TY * SV_HG * 4;            // 256: sum over the item's t of g, [s][h]
constexpr int SV_GTSTAGE = 41984;                         // GT | B | CS, padded to a multiple of 1024
constexpr int SV_PK_BYTES = SV_NCW * SV_TY * 32 * 4;      // 32768: [warp][s][lane] partial d_k sums of one tile
static_assert(SV_GT_BYTES + SV_B_BYTES + SV_CS_BYTES <= SV_GTSTAGE, "stage layout");
static_assert(SV_TX == (SV_NCW / SV_HG) * SV_XR && SV_TY == 4 * (SV_NCW / SV_HG) && SV_TY == SV_NCW, "row groups, one row per warp");
constexpr size_t SV_SMEM = 2 * SV_RAW_BYTES + 2 * SV_GTSTAGE + 2 * SV_PK_BYTES + SV_NCW * 32 * 4 + 4 * SV_CS_BYTES + 1024;

struct SvWork {
	unsigned nws, ntb, nhg, ns, total;
	int nt; // tiles of SV_TY source rows per item: those of one of the ns ranges of source rows
};
struct SvItem {
	int b, h0, w0, tb, sh; // sh: which range of source rows
};
__device__ __forceinline__ SvItem sv_decode(const SvWork &wk, unsigned r)
{
	SvItem it;
	// the width slices of one (batch, head group, row block) are neighbours in the item order: the CTAs that work on
	// them at the same time stream the same gradient tiles, so all but the first reader find them in L2
	it.w0 = int(r % wk.nws) * SV_WS;
	r /= wk.nws;
	it.sh = int(r % wk.ns);
	r /= wk.ns;
	it.tb = int(r % wk.ntb);
	r /= wk.ntb;
	it.h0 = int(r % wk.nhg) * SV_HG;
	it.b = int(r / wk.nhg);
	return it;
}

// The hot loop needs the predicate registers (seven exist) for its compare -> add groups.  A boolean that stays live
// across that loop (is this the issuing thread, is the column in range, ...) takes one away, and with too few left
// the compiler parks compare results in general registers and serialises the groups (measured: 5.2 instead of 3.7
// instructions per term).  Passing the integers such tests are made from through this no-op makes the compiler
// recompute the test where it is used instead of keeping its result in a predicate.
__device__ __forceinline__ int sv_opaque(int x)
{
	asm volatile("" : "+r"(x));
	return x;
}

__device__ __forceinline__ size_t sv_opaque(size_t x)
{
	asm volatile("" : "+l"(x));
	return x;
}

struct SvBars {
	uint64_t raw_full[2], gt_full[2];
};
// The issuing thread's cursors (next raw gradient tile, next tile of k rows), kept in shared memory: only thread 0
// touches them, and in registers they would cost every thread of the CTA eight registers the hot loop needs.
struct SvCursor {
	unsigned item, m;
	int tile;
	SvItem x;
};

// One tile (SV_TY source rows) for a compute thread: 32 query rows of its column against the tile's k values.
__device__ __forceinline__ void sv_tile_compute(const unsigned char *gts, float *pkw, int xg, int h, int lane,
						const float (&a)[SV_XR], float (&acc)[SV_XR], float &rsq)
{
	const float4 *GT = reinterpret_cast<const float4 *>(gts) + h * (SV_TX / 4) + xg * (SV_XR / 4);
	const float *GL = reinterpret_cast<const float *>(gts) + h * SV_TX + xg * SV_XR + lane;
	const float *B = reinterpret_cast<const float *>(gts + SV_GT_BYTES) + h * SV_WS + lane;
#pragma unroll 4
	for (int s = 0; s < SV_TY; s++) {
		const float bv = B[s * (SV_HG * SV_WS)];
		float pk = 0.f;
#pragma unroll
		for (int i4 = 0; i4 < SV_XR / 4; i4++) {
			const float4 g = GT[s * (SV_HG * SV_TX / 4) + i4];
			// four compares, then the eight predicated adds they feed
			asm("{\n\t.reg .pred p0, p1, p2, p3;\n\t"
			    "setp.gt.f32 p0, %5, %9;\n\tsetp.gt.f32 p1, %6, %9;\n\tsetp.gt.f32 p2, %7, %9;\n\tsetp.gt.f32 p3, %8, %9;\n\t"
			    "@p0 add.f32 %0, %0, %10;\n\t@p1 add.f32 %1, %1, %11;\n\t@p2 add.f32 %2, %2, %12;\n\t@p3 add.f32 %3, %3, %13;\n\t"
			    "@p0 add.f32 %4, %4, %10;\n\t@p1 add.f32 %4, %4, %11;\n\t@p2 add.f32 %4, %4, %12;\n\t@p3 add.f32 %4, %4, %13;\n\t}"
			    : "+f"(acc[i4 * 4]), "+f"(acc[i4 * 4 + 1]), "+f"(acc[i4 * 4 + 2]), "+f"(acc[i4 * 4 + 3]), "+f"(pk)
			    : "f"(a[i4 * 4]), "f"(a[i4 * 4 + 1]), "f"(a[i4 * 4 + 2]), "f"(a[i4 * 4 + 3]), "f"(bv), "f"(g.x), "f"(g.y), "f"(g.z),
			      "f"(g.w));
		}
		pkw[s * 32] = pk; // (one accumulator: its 32 dependent adds are spread over the ~110 instructions of the row)
		rsq += GL[s * (SV_HG * SV_TX)]; // lane l sums g of query row l of the group: the row sums, spread over the lanes
	}
}

// Synchronisation.  Tile n of the CTA's tile sequence lives in slot n & 1 of the raw ring, of the stage ring and of
// the partial-sum ring.  ONE barrier per tile orders everything: gt_full[n & 1] completes when all 16 warps have
// transposed their row of tile n (and the tile's k rows have landed).  A warp transposes tile n at the END of its
// step n - 1, i.e. after its math on tile n - 1 and after it has summed the partials of tile n - 2.  So whoever has
// passed the wait for tile n knows that every warp is done with the math of tile n - 1 (stage (n + 1) & 1 may be
// refilled, the partials of tile n - 1 are complete), with the partials of tile n - 2 (the partial slot n & 1 may be
// overwritten) and with raw slot n & 1 (tile n + 2 may be requested into it).
__global__ void __launch_bounds__(SV_THREADS, 1)
dense_bwd_sv_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap gmap,
		    const float *__restrict__ q, float *__restrict__ d_q, size_t dq_stride, float *__restrict__ part,
		    const int *__restrict__ tie_hdr, int bs, int n_tok, int n_heads, int width, float scale, SvWork wk, int *err)
{ // d_q, dq_stride: the gradient itself and 0, or (source rows split over wk.ns items) the partial sums' buffer and the size of one
	if (tie_hdr[1] != 0)
		return; // too many ties to list: the two-pass kernel computes this call
	extern __shared__ __align__(1024) unsigned char smem_raw[];
	// aligned by OFFSET into the shared array so that the pointers stay in the shared address space
	unsigned char *base = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
	unsigned char *raw = base;
	unsigned char *gts = raw + 2 * SV_RAW_BYTES;
	float *pkbase = reinterpret_cast<float *>(gts + 2 * SV_GTSTAGE);
	float *rowsum = pkbase + 2 * (SV_PK_BYTES / 4); // [warp][lane] row sums on their way to the d_q store
	float *csring = rowsum + SV_NCW * 32;             // [tile & 3][s][h]: sum over the item's query rows of g, for the reducer
	__shared__ __align__(8) SvBars bars;
	__shared__ SvCursor cur_raw, cur_kb;

	const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
	// tiles this CTA walks in all: its items x tiles per item
	const unsigned n_items = blockIdx.x < wk.total ? (wk.total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
	const unsigned n_tiles = n_items * unsigned(wk.nt);
	if (tid == 0) {
		for (int i = 0; i < 2; i++) {
			mbar_init(&bars.raw_full[i], 1);
			mbar_init(&bars.gt_full[i], SV_NCW + 1); // 16 transposed rows + the k rows' copy
		}
		mbar_fence_init();
		cur_raw.item = cur_kb.item = blockIdx.x;
		cur_raw.m = cur_kb.m = 0;
		cur_raw.tile = cur_kb.tile = 0;
		if (n_items > 0)
			cur_raw.x = cur_kb.x = sv_decode(wk, blockIdx.x);
	}
	__syncthreads();
	const size_t row = size_t(n_heads) * width;
	const int xg = warp >> 2, h = warp & 3;
	int dead = 0;

	// thread 0 only: request the next raw gradient tile / the next tile of k rows (no-ops past the last tile)
	auto advance = [&](SvCursor &c) {
		c.m++;
		if (++c.tile == wk.nt) {
			c.tile = 0;
			c.item += gridDim.x;
			if (c.item < wk.total)
				c.x = sv_decode(wk, c.item);
		}
	};
	auto issue_raw = [&]() {
		if (cur_raw.m >= n_tiles)
			return;
		const int st = int(cur_raw.m & 1u);
		mbar_expect_tx(&bars.raw_full[st], SV_RAW_BYTES);
		tma_load_4d(raw + st * SV_RAW_BYTES, &gmap, &bars.raw_full[st], cur_raw.x.h0, cur_raw.x.tb * SV_TX,
			    (cur_raw.x.sh * wk.nt + cur_raw.tile) * SV_TY, cur_raw.x.b); // box {4 h, 128 t, 16 s}; rows past the end read as zeros
		advance(cur_raw);
	};
	auto issue_kb = [&]() {
		const int st = int(cur_kb.m & 1u);
		if (cur_kb.m >= n_tiles) { // the phase after the last tile exists only to order the last partial sums: plain arrival
			mbar_arrive(&bars.gt_full[st]);
			cur_kb.m++;
			return;
		}
		mbar_expect_tx(&bars.gt_full[st], SV_B_BYTES);
		tma_load_4d(gts + st * SV_GTSTAGE + SV_GT_BYTES, &kmap, &bars.gt_full[st], cur_kb.x.w0, cur_kb.x.h0,
			    (cur_kb.x.sh * wk.nt + cur_kb.tile) * SV_TY, cur_kb.x.b); // box {32 w, 4 h, 16 s}
		advance(cur_kb);
	};
	// This warp's row (s = warp) of tile m: g [t][h] -> [h][t] and its sum over t; then the warp's arrival for tile m.
	// Past the last tile only the arrival is left.
	auto transpose_row = [&](unsigned m) {
		const int st = int(m & 1u);
		if (m < n_tiles) {
			if (sv_opaque(dead) == 0 && !mbar_wait(&bars.raw_full[st], (m >> 1) & 1u, err))
				dead = 1;
			const float4 *R = reinterpret_cast<const float4 *>(raw + st * SV_RAW_BYTES) + warp * SV_TX;
			float *GT = reinterpret_cast<float *>(gts + st * SV_GTSTAGE) + (warp * SV_HG) * SV_TX;
			float4 r[4];
#pragma unroll
			for (int j = 0; j < 4; j++)
				r[j] = R[lane + 32 * j]; // query rows lane, lane+32, lane+64, lane+96: consecutive lanes, no bank conflicts
#pragma unroll
			for (int j = 0; j < 4; j++) {
				float *o = GT + lane + 32 * j;
				o[0] = r[j].x;
				o[SV_TX] = r[j].y;
				o[2 * SV_TX] = r[j].z;
				o[3 * SV_TX] = r[j].w;
			}
			// sum over the 128 query rows of each of the four heads: 4 values x 32 lanes -> 4 values.  Halving twice
			// (each lane keeps the two, then the one head it will finish) leaves 3 butterfly steps on one value.
			float cx = r[0].x + r[1].x + r[2].x + r[3].x, cy = r[0].y + r[1].y + r[2].y + r[3].y;
			float cz = r[0].z + r[1].z + r[2].z + r[3].z, cw = r[0].w + r[1].w + r[2].w + r[3].w;
			const int ln = sv_opaque(lane); // (lane-derived predicates are loop-invariant: computed from `lane` itself they would be hoisted)
			const bool hi16 = (ln & 16) != 0, hi8 = (ln & 8) != 0;
			// lanes 0-15 finish heads (0, 1), lanes 16-31 heads (2, 3)
			float ka = hi16 ? cz : cx, kb = hi16 ? cw : cy, sa = hi16 ? cx : cz, sb = hi16 ? cy : cw;
			ka += __shfl_xor_sync(0xffffffffu, sa, 16);
			kb += __shfl_xor_sync(0xffffffffu, sb, 16);
			// within each half: lanes with bit 3 clear finish the first head of the pair, the others the second
			float kc = hi8 ? kb : ka, sc = hi8 ? ka : kb;
			kc += __shfl_xor_sync(0xffffffffu, sc, 8);
			kc += __shfl_xor_sync(0xffffffffu, kc, 4);
			kc += __shfl_xor_sync(0xffffffffu, kc, 2);
			kc += __shfl_xor_sync(0xffffffffu, kc, 1);
			if ((ln & 7) == 0) // lanes 0, 8, 16, 24 hold heads 0, 1, 2, 3
				csring[(m & 3u) * (SV_TY * SV_HG) + warp * SV_HG + (ln >> 3)] = kc; // read two steps later: four slots keep writer and reader apart
		}
		__syncwarp();
		if (sv_opaque(lane) == 0)
			mbar_arrive(&bars.gt_full[st]);
	};

	if (tid == 0 && n_tiles > 0) {
		issue_raw();
		issue_raw();
		issue_kb(); // k rows of tile 0
	}
	if (n_tiles > 0)
		transpose_row(0);

	unsigned n = 0;
	// the tile whose partials are summed next (one behind the math): where its share of d_k goes (nullptr: this
	// thread's column is out of range), and its first source row
	float *red_pp = nullptr;
	int red_s0 = -1, red_rows = 0; // red_rows: source rows of that tile this thread may store (0: column out of range)
	auto reduce_prev = [&](unsigned tile_no) {
		// this warp's four source rows of the tile: s = xg, xg+4, xg+8, xg+12; the four row groups' partials in order;
		// share = 2 sum p g - sum g
		const float *P = pkbase + (tile_no & 1u) * (SV_PK_BYTES / 4) + h * (SV_TY * 32) + lane;
		const float *C = csring + (tile_no & 3u) * (SV_TY * SV_HG) + h;
#pragma unroll
		for (int j = 0; j < 4; j++) {
			const int s = xg + 4 * j;
			const float *ps = P + s * 32;
			float v = ps[0];
			v += ps[SV_HG * SV_TY * 32];
			v += ps[2 * SV_HG * SV_TY * 32];
			v += ps[3 * SV_HG * SV_TY * 32];
			if (s < sv_opaque(red_rows))
				red_pp[size_t(red_s0 + s) * row] = fmaf(2.f, v, -C[s * SV_HG]);
		}
	};
	for (unsigned item = blockIdx.x; item < wk.total; item += gridDim.x) {
		float a[SV_XR], acc[SV_XR], rsq = 0.f;
		float *item_pp;
		size_t qoff;          // offset of this thread's first (query row, head, column) element in q and in d_q
		int src_left, rows_ok; // source rows from the item's first one to the end (0: column out of range); query rows i < rows_ok are in range
		{
			const SvItem x = sv_decode(wk, item);
			const int hh = x.h0 + h, ww = x.w0 + lane, t0 = x.tb * SV_TX + xg * SV_XR;
			const bool col_ok = hh < n_heads && ww < width;
			qoff = (size_t(x.b) * n_tok + t0) * row + size_t(hh) * width + ww;
			rows_ok = col_ok ? n_tok - t0 : 0;
			size_t off = qoff;
#pragma unroll
			for (int i = 0; i < SV_XR; i++) {
				a[i] = i < rows_ok ? q[off] : 0.f;
				off = sv_opaque(off + row);
				acc[i] = 0.f;
			}
			const int s_first = x.sh * wk.nt * SV_TY; // the item's range of source rows starts here
			item_pp = part + ((size_t(x.tb) * bs + x.b) * n_tok + s_first) * row + size_t(hh) * width + ww;
			src_left = col_ok ? n_tok - s_first : 0;
		}
		for (int tile = 0; tile < wk.nt; tile++, n++) {
			const int st = int(n & 1u);
			if (sv_opaque(dead) == 0 && !mbar_wait(&bars.gt_full[st], (n >> 1) & 1u, err))
				dead = 1; // keep walking without waiting so that every warp makes the same number of steps
			if (sv_opaque(tid) == 0 && sv_opaque(dead) == 0) {
				issue_raw(); // tile n + 2 into the raw slot tile n was transposed out of
				issue_kb();  // k rows of tile n + 1 into the stage the math of tile n - 1 has left
			}
			sv_tile_compute(gts + st * SV_GTSTAGE, pkbase + st * (SV_PK_BYTES / 4) + warp * (SV_TY * 32) + lane, xg, h, lane, a, acc, rsq);
			if (sv_opaque(red_s0) >= 0)
				reduce_prev(n - 1u);
			red_pp = item_pp;
			red_s0 = tile * SV_TY;
			red_rows = sv_opaque(src_left) - red_s0;
			transpose_row(n + 1);
		}
		// d_q of this thread's column: out = scale * (2 acc - row sum); the row sum of query row i sits in lane i and
		// reaches the other lanes through shared memory.  The accesses are volatile on purpose: it keeps them in program
		// order (load one row sum, store one result, ...).  Left free, the compiler gathers all 32 row sums first, and the
		// 32 registers that takes come out of the hot loop's budget: measured 3.64 ms against 2.57 ms for the whole
		// backward at [16,1024,16,64].
		{
			volatile float *rs = rowsum + warp * 32;
			rs[lane] = rsq;
			__syncwarp();
			// advanced through the no-op so that the 32 addresses are formed one after the other, not all up front
			size_t off = qoff + size_t(sv_decode(wk, item).sh) * dq_stride;
#pragma unroll
			for (int i = 0; i < SV_XR; i++) {
				if (i < rows_ok)
					*reinterpret_cast<volatile float *>(d_q + off) = scale * fmaf(2.f, acc[i], -rs[i]);
				off = sv_opaque(off + row);
			}
			__syncwarp();
		}
	}
	if (n_tiles > 0) { // the last tile's partials: complete once every warp has made its arrival for the phase after it
		if (dead == 0 && !mbar_wait(&bars.gt_full[n & 1u], (n >> 1) & 1u, err))
			dead = 1;
		reduce_prev(n - 1u);
	}
}

// d_k = -scale * sum over the query-row blocks of their shares, in block order; and, when the source rows were
// split over ns items, d_q = sum of the ns partial d_q (already scaled), in order.  n4 = float4 count of d_k (= of d_q).
__global__ void __launch_bounds__(256)
dense_bwd_sv_partsum_kernel(const float4 *__restrict__ part, float4 *__restrict__ d_k, const float4 *__restrict__ dq_part,
			    float4 *__restrict__ d_q, const int *__restrict__ tie_hdr, size_t n4, int ntb, int ns, float scale)
{
	if (tie_hdr[1] != 0)
		return;
	for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += size_t(gridDim.x) * blockDim.x) {
		float4 s = part[i];
		for (int r = 1; r < ntb; r++) {
			const float4 v = part[size_t(r) * n4 + i];
			s.x += v.x;
			s.y += v.y;
			s.z += v.z;
			s.w += v.w;
		}
		d_k[i] = make_float4(-scale * s.x, -scale * s.y, -scale * s.z, -scale * s.w);
		if (ns > 1) {
			float4 t = dq_part[i];
			for (int r = 1; r < ns; r++) {
				const float4 v = dq_part[size_t(r) * n4 + i];
				t.x += v.x;
				t.y += v.y;
				t.z += v.z;
				t.w += v.w;
			}
			d_q[i] = t;
		}
	}
}

} // namespace

// Returns L1ATTN_OK, a negative error, or 1 when this path does not apply (then nothing was launched).
// tie_hdr: filled by dense_ties_launch() earlier on the same stream; part, dq_part: the d_k shares and the partial
// d_q of bwd_scratch_layout() (dq_part is used only when that layout splits the source rows: ns > 1).
int dense_bwd_sv_launch(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, const int *tie_hdr,
			void *part, void *dq_part, int ns, int bs, int n_tok, int n_heads, int width, int dtype, cudaStream_t st)
{
	if (dtype != L1ATTN_F32 || width % 4 != 0 || n_heads % 4 != 0)
		return 1; // row pitches of k and of d_attn must be multiples of 16 bytes for the tensor maps
	if (ns < 1 || (ns > 1 && !dq_part))
		return 1;
	for (const void *p : {d_attn, q, k, (const void *)d_q, (const void *)d_k, (const void *)part, (const void *)dq_part})
		if (!aligned(p, 16))
			return 1;
	const uint64_t kdims[4] = {uint64_t(width), uint64_t(n_heads), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t kstr[3] = {uint64_t(width) * 4, uint64_t(n_heads) * width * 4, uint64_t(n_tok) * n_heads * width * 4};
	const uint32_t kbox[4] = {SV_WS, SV_HG, SV_TY, 1};
	const uint64_t gdims[4] = {uint64_t(n_heads), uint64_t(n_tok), uint64_t(n_tok), uint64_t(bs)};
	const uint64_t gstr[3] = {uint64_t(n_heads) * 4, uint64_t(n_tok) * n_heads * 4, uint64_t(n_tok) * n_tok * n_heads * 4};
	const uint32_t gbox[4] = {SV_HG, SV_TX, SV_TY, 1};
	CUtensorMap kmap, gmap;
	if (!encode_tmap_4d(&kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, k, kdims, kstr, kbox, CU_TENSOR_MAP_SWIZZLE_NONE) ||
	    !encode_tmap_4d(&gmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, d_attn, gdims, gstr, gbox, CU_TENSOR_MAP_SWIZZLE_NONE))
		return 1;
	int *err = device_error_word();
	if (!err)
		return 1;
	SvWork wk;
	wk.nws = (width + SV_WS - 1) / SV_WS;
	wk.ntb = (n_tok + SV_TX - 1) / SV_TX;
	wk.nhg = (n_heads + SV_HG - 1) / SV_HG;
	wk.ns = unsigned(ns);
	const long long total = (long long)bs * wk.nhg * wk.ntb * wk.nws * ns;
	if (total > 0x7fffffffLL)
		return 1;
	wk.total = unsigned(total);
	wk.nt = ((n_tok + SV_TY - 1) / SV_TY + ns - 1) / ns; // per item; the last range may reach past the end (zero-filled loads, no stores)
	int dev = 0, sms = 0;
	L1B_CUDA(cudaGetDevice(&dev));
	L1B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
	const unsigned grid = wk.total < unsigned(sms) ? wk.total : unsigned(sms);
	L1B_CUDA(cudaFuncSetAttribute(dense_bwd_sv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SV_SMEM)));
	const float scale = float(-1.0 / sqrt(double(width)));
	const size_t n4 = size_t(bs) * n_tok * n_heads * width / 4;
	dense_bwd_sv_kernel<<<grid, SV_THREADS, SV_SMEM, st>>>(kmap, gmap, (const float *)q, ns > 1 ? (float *)dq_part : (float *)d_q,
							       ns > 1 ? n4 * 4 : size_t(0), (float *)part, tie_hdr, bs, n_tok, n_heads,
							       width, scale, wk, err);
	L1B_LAUNCH_CHECK();
	const size_t want = (n4 + 255) / 256;
	const unsigned pgrid = unsigned(want < size_t(sms) * 16 ? want : size_t(sms) * 16);
	dense_bwd_sv_partsum_kernel<<<pgrid, 256, 0, st>>>((const float4 *)part, (float4 *)d_k, (const float4 *)dq_part, (float4 *)d_q,
							   tie_hdr, n4, int(wk.ntb), ns, scale);
	L1B_LAUNCH_CHECK();
	return L1ATTN_OK;
}

} // namespace l1b
