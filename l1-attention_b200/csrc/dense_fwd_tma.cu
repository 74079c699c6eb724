// Dense L1 scores, forward -- the B200 fast path.
//
//   attn[b][s][t][h] = scale * sum_w |q[b][t][h][w] - k[b][s][h][w]|
//
// Persistent, warp-specialised kernel: one CTA per SM walks a list of (batch, head-group of 8,
// query tile of 64, key tile of 32) work items.
//   * warp 8 is the producer: one lane issues TMA tensor copies (cp.async.bulk.tensor, no
//     multicast) -- per stage the 64-byte-wide width chunk of the q tile and of the k tile, as
//     [token][head][16 B chunk] boxes with the 64-byte hardware swizzle -- into a ring of NSTAGE
//     shared-memory stages, each guarded by a full/empty mbarrier pair.  It runs ahead across
//     work items, so the next item's tiles land while the current one is still being reduced;
//   * warps 0..7 compute: lanes = 8 heads x 4 query rows, each thread keeps an 8 x 8 (query, key)
//     register tile of its head, reads operands with conflict-free 16-byte shared loads (the
//     swizzle spreads the 8 head-lanes over 8 bank groups) and spends 1.5 issue slots per
//     term (packed sub.f32x2 for two differences; scalar add with |.| as a source modifier).  Eight compute warps with ~160
//     registers each (no spills) measured faster than sixteen with 128;
//   * results leave through shared memory: the compute warps drop their scaled tiles into a
//     [key][query][head] staging buffer (each warp store is one 128-byte row) and one thread issues
//     a single TMA tensor store of the 32 x 64 x 8 box; scattered 4-byte global stores from the
//     register tiles cost over 20 % of the kernel when measured.  When the head count is not a
//     multiple of 4 (row pitch not 16-byte aligned) the tiles are stored directly instead: the 8
//     head-lanes then write 32 contiguous bytes per (s, t), whole sectors either way;
//   * no [b,h,t,w] copy of q/k is ever made (the reference transposes both first).
// Out-of-range rows/heads/width are zero-filled by TMA (|0-0| adds nothing) and masked at the store.
// Every mbarrier wait is bounded (tma.cuh); on a timeout the CTA stops and the error word is set.
#include "common.cuh"
#include "tma.cuh"

namespace l1b {
namespace {

// A work item is HG heads x TT query rows x TS key rows with HG * TT = 512: HG = 8 (TT = 64) or, for head counts
// that leave fewer idle lanes in groups of four (4, 12, 20 ... heads; a head-group shard of a multi-GPU run),
// HG = 4 (TT = 128).  The lanes of a warp are the 32 consecutive (query row, head) rows of the q tile either way.
constexpr int CH = 4;       // 16-byte chunks per (token, head) row per stage
constexpr int NCW = 8;      // compute warps: 2 (query halves) x 4 (key groups)
constexpr int NSTAGE = 3;
constexpr int TS = 32;
constexpr int TM = 8, TN = 8;
constexpr int Q_BYTES = 512 * CH * 16;           // 32768: TT * HG rows of 64 bytes
constexpr int K_BYTES_MAX = TS * 8 * CH * 16;    // 16384 (HG = 8; half of it with HG = 4)
constexpr int STAGE_BYTES = Q_BYTES + K_BYTES_MAX; // 49152
constexpr int OUT_BYTES = TS * 512 * 4;          // 65536: staging tile [s][t][h] of the TMA store
constexpr int NTHREADS = (NCW + 1) * 32;

struct Work {
	unsigned ntt, nst, nhg, total;
};

struct Item {
	int t0, s0, h0, b;
};
template <int HG> __device__ __forceinline__ Item decode_item(const Work &wk, unsigned r)
{
	constexpr int TT = 512 / HG;
	Item x;
	x.t0 = int(r % wk.ntt) * TT;
	r /= wk.ntt;
	x.s0 = int(r % wk.nst) * TS;
	r /= wk.nst;
	x.h0 = int(r % wk.nhg) * HG;
	x.b = int(r / wk.nhg);
	return x;
}

template <typename T, int HG> // instantiated for float only: the packed subtract below is fp32
__global__ void __launch_bounds__(NTHREADS, 1)
dense_fwd_tma_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
		     const __grid_constant__ CUtensorMap omap, int tma_store, T *__restrict__ attn, int n_tok, int n_heads, int width, T scale, Work wk, int *err)
{
	constexpr int VEC = 16 / sizeof(T);
	constexpr int WC = CH * VEC;
	constexpr int LT = 32 / HG;  // lanes along the query axis
	constexpr int TT = 512 / HG; // query rows per item
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

	const int nchunk = (width + WC - 1) / WC;

	if (warp == NCW) {
		// ---------------- producer warp: one lane feeds the ring
		if (lane == 0) {
			int st = 0;
			uint32_t ph = 1; // a fresh barrier reads as "previous phase (parity 1) complete"
			for (unsigned item = blockIdx.x; item < wk.total; item += gridDim.x) {
				const Item x = decode_item<HG>(wk, item);
				for (int ci = 0; ci < nchunk; ci++) {
					if (!mbar_wait_relaxed(&empty_bar[st], ph, err))
						return;
					unsigned char *dst = stages + size_t(st) * STAGE_BYTES;
					mbar_expect_tx(&full_bar[st], Q_BYTES + TS * HG * CH * 16);
					tma_load_4d(dst, &qmap, &full_bar[st], ci * WC, x.h0, x.t0, x.b);
					tma_load_4d(dst + Q_BYTES, &kmap, &full_bar[st], ci * WC, x.h0, x.s0, x.b);
					if (++st == NSTAGE) {
						st = 0;
						ph ^= 1;
					}
				}
			}
		}
		return;
	}

	// ---------------- compute warps
	const int lane_h = lane & (HG - 1), lane_t = lane / HG;
	const int wt = warp & 1, ws = warp >> 1; // 2 query halves x 4 key groups
	// TMA 64-byte swizzle: chunk ^= address bits 7..8 = (row >> 1) & 3, row = token * HG + head within the box.  The
	// q rows of a warp load are base + lane with base a multiple of 32; the k rows are (ws * TN + j) * HG + head,
	// where j contributes to those bits only when HG = 4
	const int sw = (lane >> 1) & 3;
	const int swk = (lane_h >> 1) & 3;
	const int qoff = ((wt * (TT / 2) + lane_t) * HG + lane_h) * CH;
	const int koff = Q_BYTES / 16 + ((ws * TN) * HG + lane_h) * CH;
	int st = 0;
	uint32_t ph = 0;
	bool dead = false;
	for (unsigned item = blockIdx.x; item < wk.total; item += gridDim.x) {
		T acc[TM][TN];
#pragma unroll
		for (int i = 0; i < TM; i++)
#pragma unroll
			for (int j = 0; j < TN; j++)
				acc[i][j] = T(0);

		for (int ci = 0; ci < nchunk; ci++) {
			// after a timeout the warp keeps walking its items without waiting (results are
			// invalid and the error word says so) so that it still meets the others at the barriers
			if (!dead && !mbar_wait(&full_bar[st], ph, err))
				dead = true;
			const ulonglong2 *S = reinterpret_cast<const ulonglong2 *>(stages + size_t(st) * STAGE_BYTES);
			const ulonglong2 *qp = S + qoff, *kp = S + koff;
#pragma unroll
			for (int c = 0; c < CH; c++) {
				const int pc = c ^ sw, pk0 = c ^ swk;
				// Each 16-byte operand is two register pairs; the subtraction is the packed
				// sub.f32x2 (one issue slot for two differences), the |.|-accumulation stays
				// scalar because its abs is a free source modifier only there.
				ulonglong2 kv[TN];
#pragma unroll
				for (int j = 0; j < TN; j++)
					kv[j] = kp[j * HG * CH + (pk0 ^ (HG == 4 ? (2 * j) & 3 : 0))];
#pragma unroll
				for (int i = 0; i < TM; i++) {
					const ulonglong2 qv = qp[i * LT * HG * CH + pc];
#pragma unroll
					for (int j = 0; j < TN; j++) {
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
			__syncwarp();
			if (lane == 0)
				mbar_arrive(&empty_bar[st]);
			if (++st == NSTAGE) {
				st = 0;
				ph ^= 1;
			}
		}

		const Item x = decode_item<HG>(wk, item);
		if (tma_store) {
			T *stage_out = reinterpret_cast<T *>(stages + size_t(NSTAGE) * STAGE_BYTES);
			if (tid == 0)
				tma_store_wait_read(); // the previous item's store has drained the staging tile
			named_barrier(1, NCW * 32);
			T *o = stage_out + ((ws * TN) * TT + wt * (TT / 2) + lane_t) * HG + lane_h;
#pragma unroll
			for (int j = 0; j < TN; j++)
#pragma unroll
				for (int i = 0; i < TM; i++)
					o[(j * TT + LT * i) * HG] = acc[i][j] * scale;
			fence_proxy_async_smem();
			named_barrier(1, NCW * 32);
			if (tid == 0) {
				tma_store_4d(&omap, stage_out, x.h0, x.t0, x.s0, x.b);
				tma_store_commit();
			}
			continue;
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
					const int t = x.t0 + wt * (TT / 2) + lane_t + LT * i;
					if (t < n_tok)
						row[size_t(t) * n_heads] = acc[i][j] * scale;
				}
			}
		}
	}
	if (tma_store && tid == 0)
		tma_store_wait_read(); // shared memory must outlive the last store's reads
}

template <typename T> CUtensorMapDataType tmap_dtype();
template <> CUtensorMapDataType tmap_dtype<float>() { return CU_TENSOR_MAP_DATA_TYPE_FLOAT32; }

template <typename T, int HG>
int launch(const T *q, const T *k, T *attn, int bs, int n_tok, int n_heads, int width, cudaStream_t st)
{
	constexpr int VEC = 16 / sizeof(T);
	constexpr int TT = 512 / HG;
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
	// output [bs][s][t][h] as a tensor for the TMA store; needs a 16-byte row pitch and base
	CUtensorMap omap = qmap;
	int tma_store = 0;
	if ((size_t(n_heads) * sizeof(T)) % 16 == 0 && aligned(attn, 16)) {
		const uint64_t odims[4] = {uint64_t(n_heads), uint64_t(n_tok), uint64_t(n_tok), uint64_t(bs)};
		const uint64_t ostr[3] = {uint64_t(n_heads) * sizeof(T), uint64_t(n_tok) * n_heads * sizeof(T),
					  uint64_t(n_tok) * n_tok * n_heads * sizeof(T)};
		const uint32_t obox[4] = {HG, TT, TS, 1};
		tma_store = encode_tmap_4d(&omap, tmap_dtype<T>(), attn, odims, ostr, obox, CU_TENSOR_MAP_SWIZZLE_NONE) ? 1 : 0;
	}
	Work wk;
	wk.ntt = (n_tok + TT - 1) / TT;
	wk.nst = (n_tok + TS - 1) / TS;
	wk.nhg = (n_heads + HG - 1) / HG;
	const long long total = (long long)bs * wk.nhg * wk.ntt * wk.nst;
	if (total > 0x7fffffffLL)
		return L1ATTN_ERR_SHAPE;
	wk.total = unsigned(total);
	int dev = 0, sms = 0;
	L1B_CUDA(cudaGetDevice(&dev));
	L1B_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
	const unsigned grid = wk.total < unsigned(sms) ? wk.total : unsigned(sms);
	const size_t smem = size_t(NSTAGE) * STAGE_BYTES + OUT_BYTES + 1024;
	auto kern = dense_fwd_tma_kernel<T, HG>;
	L1B_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
	const T scale = T(-1.0 / sqrt(double(width)));
	kern<<<unsigned(grid), NTHREADS, smem, st>>>(qmap, kmap, omap, tma_store, attn, n_tok, n_heads, width, scale, wk, err);
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
	// groups of four heads (x 128 query rows) where they leave fewer lanes idle than groups of eight (x 64 query rows):
	// 4, 12, 20 ... heads, unless the token count pads badly to 128
	const long long work8 = (long long)((n_heads + 7) / 8 * 8) * ((n_tok + 63) / 64 * 64);
	const long long work4 = (long long)((n_heads + 3) / 4 * 4) * ((n_tok + 127) / 128 * 128);
	if (work4 < work8)
		return launch<float, 4>((const float *)q, (const float *)k, (float *)attn, bs, n_tok, n_heads, width, st);
	return launch<float, 8>((const float *)q, (const float *)k, (float *)attn, bs, n_tok, n_heads, width, st);
}

} // namespace l1b
