/*
 * l1attn_oracle.c -- CPU oracle for the L1-attention hot path.  TEST INFRASTRUCTURE ONLY:
 * it is linked by the tests, by the smoke check and by the benchmark's CPU-baseline leg, and by
 * nothing the library ships.  The GPU library never falls back to it.
 *
 * Parity status: PINNED.  tests/test_oracle_golden.py checks every function here against
 * (1) the known-answer vectors of the reference's own fixtures (python/l1attn_sparse.py:444-581,
 * testdense.py:20-39), (2) outputs of the reference's pure-PyTorch code and of its compiled CPU
 * extension on seeded inputs (tests/golden/, made by tests/golden/make_golden.py), and (3), when
 * oracle/_ref/ is present, the compiled reference CPU extension directly.
 *
 * Build: `make -C oracle` (gcc -O2; no -ffast-math, the summation order is part of the contract).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define REAL double
#define SFX f64
#define ABS fabs
#define EXP exp
#include "l1attn_oracle_impl.h"
#undef REAL
#undef SFX
#undef ABS
#undef EXP

#define REAL float
#define SFX f32
#define ABS fabsf
#define EXP expf
#include "l1attn_oracle_impl.h"
#undef REAL
#undef SFX
#undef ABS
#undef EXP

/*
 * expandCoo (cuda/l1attn_sparse_cuda.py:58-101; identical copies at
 * cuda/l1attn_sparse_bidi_cuda.py:59-104, cpp/l1attn_sparse_cpp.py:61-106,
 * python/l1attn_sparse.py:382-427).
 *
 * co:  int64 [cl][2] rows {dst, src}.
 * coo: int32 [cl][4] rows {dst, src, dst_rank, src_rank}; a rank is the number of EARLIER rows
 *      with the same dst (resp. src), i.e. the reference's per-key running counter.
 * Returns the largest rank + 1 for each key through *dst_mxlen / *src_mxlen (1 for an empty list,
 * because the reference starts both maxima at 0 and adds 1).
 *
 * The reference keeps its counters in Python dicts; here they are dense arrays over
 * [min key, max key], which gives the same numbers for any integer keys.
 * Returns 0, or -1 if the key range is too large to allocate.
 */
int oracle_expand_coo(const int64_t *co, int cl, int32_t *coo, int *dst_mxlen, int *src_mxlen)
{
	int mx[2] = {0, 0};
	for (int col = 0; col < 2; col++) {
		if (cl == 0)
			break;
		int64_t lo = co[col], hi = co[col];
		for (int i = 0; i < cl; i++) {
			int64_t x = co[2 * (size_t)i + col];
			if (x < lo)
				lo = x;
			if (x > hi)
				hi = x;
		}
		if (hi - lo > ((int64_t)1 << 31))
			return -1;
		int32_t *cnt = (int32_t *)calloc((size_t)(hi - lo + 1), sizeof(int32_t));
		if (!cnt)
			return -1;
		for (int i = 0; i < cl; i++) {
			int64_t x = co[2 * (size_t)i + col];
			int32_t rank = cnt[x - lo]++; /* first occurrence gets 0 (:78-85) */
			coo[4 * (size_t)i + col] = (int32_t)x;
			coo[4 * (size_t)i + 2 + col] = rank;
			if (rank > mx[col])
				mx[col] = rank;
		}
		free(cnt);
	}
	*dst_mxlen = mx[0] + 1;
	*src_mxlen = mx[1] + 1;
	return 0;
}
