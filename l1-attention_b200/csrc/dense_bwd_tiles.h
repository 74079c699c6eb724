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

// Tie flags, one byte each, for G = bs * head groups * width slices "groups":
//   xflag[pass][G][nxt]  the x tile holds a row that ties with some row of the other side
//   yflag[pass][G][ny]   the y tile holds such a row of the other side
// A (work item, y tile) pair needs the exact loop only if both its flags are set.
struct BwdFlagLayout {
	size_t groups, nxt, ny;
	__host__ __device__ size_t xoff(int pass) const { return size_t(pass) * groups * nxt; }
	__host__ __device__ size_t yoff(int pass) const { return 2 * groups * nxt + size_t(pass) * groups * ny; }
	__host__ __device__ size_t bytes() const { return 2 * groups * (nxt + ny); }
};
inline BwdFlagLayout bwd_flag_layout(int bs, int n_tok, int n_heads, int width)
{
	BwdFlagLayout l;
	l.groups = size_t(bs) * ((n_heads + BWD_HG - 1) / BWD_HG) * ((width + BWD_WS - 1) / BWD_WS);
	l.nxt = (n_tok + BWD_TX - 1) / BWD_TX;
	l.ny = (n_tok + BWD_TY - 1) / BWD_TY;
	return l;
}
} // namespace l1b
