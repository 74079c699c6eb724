// Work-item geometry shared by the fast dense backward (dense_bwd_tma.cu) and the tie detector
// (dense_ties.cu): both must number the (pass, batch, head group, width slice, x tile) items alike.
#pragma once
#include <stddef.h>
#include <cuda_runtime.h>
namespace l1b {
constexpr int BWD_HG = 8;  // heads per work item
constexpr int BWD_TX = 32; // x rows (tokens) per work item
constexpr int BWD_WS = 64; // width columns per work item
constexpr int BWD_TY = 16; // y rows (tokens of the other side) per pipeline stage

constexpr int BWD_XF = 4;  // x rows per x flag: the rows one warp of the backward owns
constexpr int BWD_WF = 32; // width columns per flag group: the columns one warp of the backward owns,
                           // i.e. those of a 64-wide slice with the same (w % 32) / 16

// Tie flags, one byte each, for G = bs * head groups * width groups (two per width slice):
//   xflag[pass][G][nxf]  rows [4i, 4i+4) of the x side hold a value that ties with some row of the other side
//   yflag[pass][G][ny]   the y tile holds such a row of the other side
// A warp of the backward (4 x rows, 8 heads, 32 width columns) needs the exact loop for a y tile only
// if both flags are set.
struct BwdFlagLayout {
	size_t groups, nxf, ny, nhg, nwf;
	__host__ __device__ size_t group(int b, int h, int w) const { return (size_t(b) * nhg + size_t(h) / BWD_HG) * nwf + size_t(w) / BWD_WS * 2 + size_t(w) % 32 / 16; }
	__host__ __device__ size_t xoff(int pass) const { return size_t(pass) * groups * nxf; }
	__host__ __device__ size_t yoff(int pass) const { return 2 * groups * nxf + size_t(pass) * groups * ny; }
	__host__ __device__ size_t bytes() const { return 2 * groups * (nxf + ny); }
};
inline BwdFlagLayout bwd_flag_layout(int bs, int n_tok, int n_heads, int width)
{
	BwdFlagLayout l;
	l.nhg = (n_heads + BWD_HG - 1) / BWD_HG;
	l.nwf = size_t((width + BWD_WS - 1) / BWD_WS) * (BWD_WS / BWD_WF); // padded to whole width slices
	l.groups = size_t(bs) * l.nhg * l.nwf;
	l.nxf = size_t((n_tok + BWD_TX - 1) / BWD_TX) * (BWD_TX / BWD_XF); // padded to whole x tiles
	l.ny = (n_tok + BWD_TY - 1) / BWD_TY;
	return l;
}

// ---- listed ties, single-visit backward ----
constexpr int BWD_TIE_CAP = 4096; // listed ties per call; more set the overflow word and the flagged exact loops run
constexpr int BWD_SV_TX = 128;    // query rows per work item of the single-visit kernel: d_k leaves it as ceil(n_tok / 128) shares

// The single-visit kernel's work items are (batch, 4 heads, 32 columns, 128 query rows); each walks all source
// rows, or -- when that many items would leave much of the last wave of SMs empty (long context, small batch, a
// shard of a multi-GPU run) -- one of `ns` equal ranges of them, leaving `ns` partial d_q that the summing kernel
// adds.  The choice depends on the shape alone (the SM count is taken as B200's 148) so that the scratch size can
// be stated without a device.  An item's fixed cost (its q rows in, its d_q rows out) is taken as 0.4 tiles.
constexpr int BWD_SV_SMS = 148;
inline double bwd_wave_fill(double items, int sms)
{
	const double waves = double((long long)((items + sms - 1) / sms));
	return waves > 0 ? items / (waves * sms) : 0.0;
}
inline int bwd_sv_splits(int bs, int n_tok, int n_heads, int width)
{
	const double items = double(bs) * ((n_heads + 3) / 4) * ((width + 31) / 32) * ((n_tok + BWD_SV_TX - 1) / BWD_SV_TX);
	const int tiles = (n_tok + 15) / 16;
	int best = 1;
	double best_eff = bwd_wave_fill(items, BWD_SV_SMS) * tiles / (tiles + 0.4);
	for (int ns = 2; ns <= 8; ns *= 2) {
		const double tp = double((tiles + ns - 1) / ns);
		if (tp < 8)
			break;
		const double eff = bwd_wave_fill(items * ns, BWD_SV_SMS) * tp / (tp + 0.4);
		if (eff > best_eff * 1.02) { // (not for a percent or two: a split costs one more pass over d_q)
			best = ns;
			best_eff = eff;
		}
	}
	return best;
}

// Caller-provided scratch of the dense backward, in this order (every part 256-byte aligned):
//   tie flags | tie header {count, overflow} | tie list uint4[BWD_TIE_CAP] | shares of d_k | partial d_q (if split)
// The flags and the header are adjacent so that one memset clears both.
struct BwdScratchLayout {
	size_t flags, hdr, ties, part, dqpart, bytes; // offsets, total
	int ntb, ns;
};
inline BwdScratchLayout bwd_scratch_layout(int bs, int n_tok, int n_heads, int width)
{
	auto pad = [](size_t n) { return (n + 255) / 256 * 256; };
	BwdScratchLayout l;
	l.flags = 0;
	l.hdr = pad(bwd_flag_layout(bs, n_tok, n_heads, width).bytes());
	l.ties = l.hdr + 256;
	l.part = l.ties + size_t(BWD_TIE_CAP) * 16;
	l.ntb = (n_tok + BWD_SV_TX - 1) / BWD_SV_TX;
	l.ns = bwd_sv_splits(bs, n_tok, n_heads, width);
	const size_t n = size_t(bs) * n_tok * n_heads * width * 4;
	l.dqpart = l.part + pad(size_t(l.ntb) * n);
	l.bytes = l.dqpart + (l.ns > 1 ? pad(size_t(l.ns) * n) : 0);
	return l;
}
} // namespace l1b
