/*
 * CPU restatement of the reference's L1-attention arithmetic -- TEST INFRASTRUCTURE ONLY.
 *
 * This header is included twice by l1attn_oracle.c, once with REAL=double / SFX=f64 and once
 * with REAL=float / SFX=f32.  Every function is a plain scalar loop nest in the loop order of the
 * reference's CPU extension, so that results agree with it to the last bit in fp64 (same
 * operations in the same order).  The fp32 instantiation is what the reference's CPU code would
 * compute if its `#define DTYPE double` (cpp/l1attn_drv.cpp:5) read `float`.
 *
 * Layouts (all row-major, contiguous):
 *   q, k, v, vo, dq, dk, dv ... : [bs][n_tok][n_heads][width]
 *   dense attn / d_attn         : [bs][src s][dst t][n_heads]
 *   sparse attn                 : [bs][n_tok][dst_mxlen][n_heads]
 *   coo                         : int32 [cl][4] = {dst, src, dst_rank, src_rank}
 */

#define CAT_(a, b) a##_##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SFX)

/* cpp/l1attn_drv.cpp:7-11 -- sign with sign(0) = 0 */
static REAL FN(sgn)(REAL x)
{
	REAL t = x < 0 ? (REAL)-1 : (REAL)0;
	return x > 0 ? (REAL)1 : t;
}

/* cpp/l1attn_drv.cpp:13-58 (l1attn_forward): attn[b][s][t][h] = scale * sum_w |q[b][t][h][w] - k[b][s][h][w]| */
void FN(oracle_dense_fwd)(const REAL *q, const REAL *k, REAL *attn, int bs, int n_ctx, int n_heads, int width)
{
	const double scale = -1.0 / sqrt((double)width); /* :22, a double in the reference too */
	for (int b = 0; b < bs; b++)
		for (int s = 0; s < n_ctx; s++)
			for (int t = 0; t < n_ctx; t++)
				for (int h = 0; h < n_heads; h++) {
					const REAL *qr = q + (((size_t)b * n_ctx + t) * n_heads + h) * width;
					const REAL *kr = k + (((size_t)b * n_ctx + s) * n_heads + h) * width;
					REAL f = 0;
					for (int w = 0; w < width; w++)
						f += ABS(qr[w] - kr[w]);
					f *= scale; /* REAL *= double, then rounded to REAL, as in :50 */
					attn[(((size_t)b * n_ctx + s) * n_ctx + t) * n_heads + h] = f;
				}
}

/* cpp/l1attn_drv.cpp:60-103 (l1attn_backward) */
void FN(oracle_dense_bwd)(const REAL *d_attn, const REAL *q, const REAL *k, REAL *d_q, REAL *d_k,
			  int bs, int n_ctx, int n_heads, int width)
{
	const double scale = -1.0 / sqrt((double)width);
	size_t n = (size_t)bs * n_ctx * n_heads * width;
	for (size_t i = 0; i < n; i++) {
		d_q[i] = 0;
		d_k[i] = 0;
	}
	for (int b = 0; b < bs; b++)
		for (int s = 0; s < n_ctx; s++)
			for (int t = 0; t < n_ctx; t++)
				for (int h = 0; h < n_heads; h++) {
					REAL d_a = d_attn[(((size_t)b * n_ctx + s) * n_ctx + t) * n_heads + h];
					size_t qo = (((size_t)b * n_ctx + t) * n_heads + h) * width;
					size_t ko = (((size_t)b * n_ctx + s) * n_heads + h) * width;
					for (int w = 0; w < width; w++) {
						REAL ws = q[qo + w] - k[ko + w];
						ws = FN(sgn)(ws) * scale; /* :95 */
						d_q[qo + w] += ws * d_a;
						d_k[ko + w] -= ws * d_a;
					}
				}
}


/*
 * The dense consumer that follows l1attn_forward in every dense caller of the reference
 * (README.md:64-66, testdense.py:14-16): a = F.softmax(attn, 1); vo = einsum('bsdh,bshw->bdhw', a, v).
 * mode 0: softmax over s (max subtracted first, as torch does);
 * mode 1: softmax with one more all-zero source row, the row then dropped
 *         (python/l1attn_sparse.py:491-502: zero-padded `ap`, softmax, strip) = exp(x) / (1 + sum exp(x)),
 *         the maximum being the 0 of the extra row;
 * mode 2: exp(x) (same lines, use_softmax False).
 * `attn` is scratch of n_ctx REALs.
 */
void FN(oracle_dense_softmax_v)(const REAL *q, const REAL *k, const REAL *v, REAL *vo, REAL *attn, int bs, int n_ctx,
				int n_heads, int width, int v_width, int mode)
{
	const double scale = -1.0 / sqrt((double)width);
	for (int b = 0; b < bs; b++)
		for (int t = 0; t < n_ctx; t++)
			for (int h = 0; h < n_heads; h++) {
				const REAL *qr = q + (((size_t)b * n_ctx + t) * n_heads + h) * width;
				REAL mx = 0; /* modes 1, 2: the extra row's 0 / no shift */
				for (int s = 0; s < n_ctx; s++) {
					const REAL *kr = k + (((size_t)b * n_ctx + s) * n_heads + h) * width;
					REAL f = 0;
					for (int w = 0; w < width; w++)
						f += ABS(qr[w] - kr[w]);
					f *= scale;
					attn[s] = f;
					if (mode == 0 && (s == 0 || f > mx))
						mx = f;
				}
				REAL den = mode == 1 ? (REAL)1 : (REAL)0;
				for (int s = 0; s < n_ctx; s++) {
					attn[s] = EXP(attn[s] - mx);
					den += attn[s];
				}
				if (mode == 2)
					den = 1;
				REAL *o = vo + (((size_t)b * n_ctx + t) * n_heads + h) * v_width;
				for (int c = 0; c < v_width; c++) {
					REAL acc = 0;
					for (int s = 0; s < n_ctx; s++)
						acc += attn[s] * v[(((size_t)b * n_ctx + s) * n_heads + h) * v_width + c];
					o[c] = acc / den;
				}
			}
}

/*
 * Sparse forward, one-directional (bidi == 0; cpp/l1attn_sparse_drv.cpp:13-96) or bidirectional
 * (bidi == 1; cpp/l1attn_sparse_bidi_drv.cpp:15-101).  `v` is V (vf for bidi); `vb` is read only
 * when bidi.  v_width may differ from width, as in the reference's GPU launcher
 * (cuda/l1attn_sparse_cuda_kernel.cu:385); the CPU reference only ever uses v_width == width.
 * attn is returned post-softmax (it is the activation the backward consumes).
 */
void FN(oracle_sparse_fwd)(const REAL *v, const REAL *vb, const REAL *q, const REAL *k, const int *coo,
			   REAL *vo, REAL *attn, int bs, int n_tok, int n_heads, int width, int v_width,
			   int cl, int dst_mxlen, int use_softmax, int bidi)
{
	const double scale = -1.0 / sqrt((double)width);
	size_t n_attn = (size_t)bs * n_tok * dst_mxlen * n_heads;
	size_t n_vo = (size_t)bs * n_tok * n_heads * v_width;
	for (size_t i = 0; i < n_attn; i++)
		attn[i] = (REAL)(1 * -1e12); /* ones * -1e12, :40-41 */
	for (size_t i = 0; i < n_vo; i++)
		vo[i] = 0;
#define QK(b, tok, h) ((((size_t)(b) * n_tok + (tok)) * n_heads + (h)) * width)
#define VV(b, tok, h) ((((size_t)(b) * n_tok + (tok)) * n_heads + (h)) * v_width)
#define AT(b, d, r, h) ((((size_t)(b) * n_tok + (d)) * dst_mxlen + (r)) * n_heads + (h))
	for (int b = 0; b < bs; b++)
		for (int h = 0; h < n_heads; h++) {
			for (int c = 0; c < cl; c++) { /* :53-63 */
				int dst = coo[4 * c + 0], src = coo[4 * c + 1], r = coo[4 * c + 2];
				REAL f = 0;
				for (int w = 0; w < width; w++)
					f += ABS(q[QK(b, dst, h) + w] - k[QK(b, src, h) + w]);
				f *= scale;
				attn[AT(b, dst, r, h)] = f;
			}
			if (use_softmax) { /* :64-73: denominator starts at 1, no max subtraction */
				for (int d = 0; d < n_tok; d++) {
					REAL f = 1;
					for (int r = 0; r < dst_mxlen; r++)
						f += EXP(attn[AT(b, d, r, h)]);
					for (int r = 0; r < dst_mxlen; r++)
						attn[AT(b, d, r, h)] = EXP(attn[AT(b, d, r, h)]) / f;
				}
			} else { /* :74-79 */
				for (int d = 0; d < n_tok; d++)
					for (int r = 0; r < dst_mxlen; r++)
						attn[AT(b, d, r, h)] = EXP(attn[AT(b, d, r, h)]);
			}
			for (int c = 0; c < cl; c++) { /* :81-90; bidi :82-95 */
				int dst = coo[4 * c + 0], src = coo[4 * c + 1], r = coo[4 * c + 2];
				for (int w = 0; w < v_width; w++)
					vo[VV(b, dst, h) + w] += attn[AT(b, dst, r, h)] * v[VV(b, src, h) + w];
				if (bidi)
					for (int w = 0; w < v_width; w++)
						vo[VV(b, src, h) + w] += attn[AT(b, dst, r, h)] * vb[VV(b, dst, h) + w];
			}
		}
}

/*
 * Sparse backward (cpp/l1attn_sparse_drv.cpp:98-192; bidi: cpp/l1attn_sparse_bidi_drv.cpp:103-212).
 * Outputs d_v (d_vf for bidi), d_vb (bidi only), d_q, d_k.  The softmax Jacobian product is the
 * reference's O(dst_mxlen^2) double loop, kept literally so the summation order matches.
 */
void FN(oracle_sparse_bwd)(const REAL *dvo, const REAL *v, const REAL *vb, const REAL *q, const REAL *k,
			   const int *coo, const REAL *attn, REAL *d_v, REAL *d_vb, REAL *d_q, REAL *d_k,
			   int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
			   int use_softmax, int bidi)
{
	const double scale = -1.0 / sqrt((double)width);
	size_t n_qk = (size_t)bs * n_tok * n_heads * width;
	size_t n_v = (size_t)bs * n_tok * n_heads * v_width;
	size_t n_attn = (size_t)bs * n_tok * dst_mxlen * n_heads;
	REAL *dattn_sm = (REAL *)calloc(n_attn ? n_attn : 1, sizeof(REAL));
	REAL *dattn = (REAL *)calloc(n_attn ? n_attn : 1, sizeof(REAL));
	for (size_t i = 0; i < n_qk; i++) {
		d_q[i] = 0;
		d_k[i] = 0;
	}
	for (size_t i = 0; i < n_v; i++) {
		d_v[i] = 0;
		if (bidi)
			d_vb[i] = 0;
	}
	for (int b = 0; b < bs; b++)
		for (int h = 0; h < n_heads; h++) {
			for (int c = 0; c < cl; c++) { /* :138-151 */
				int dst = coo[4 * c + 0], src = coo[4 * c + 1], r = coo[4 * c + 2];
				for (int w = 0; w < v_width; w++)
					d_v[VV(b, src, h) + w] += attn[AT(b, dst, r, h)] * dvo[VV(b, dst, h) + w];
				if (bidi)
					for (int w = 0; w < v_width; w++)
						d_vb[VV(b, dst, h) + w] += attn[AT(b, dst, r, h)] * dvo[VV(b, src, h) + w];
				for (int w = 0; w < v_width; w++)
					dattn_sm[AT(b, dst, r, h)] += v[VV(b, src, h) + w] * dvo[VV(b, dst, h) + w];
				if (bidi)
					for (int w = 0; w < v_width; w++)
						dattn_sm[AT(b, dst, r, h)] += vb[VV(b, dst, h) + w] * dvo[VV(b, src, h) + w];
			}
			if (use_softmax) { /* :152-166 */
				for (int d = 0; d < n_tok; d++)
					for (int r = 0; r < dst_mxlen; r++)
						for (int qq = 0; qq < dst_mxlen; qq++) {
							REAL f;
							if (r == qq)
								f = attn[AT(b, d, r, h)] * (1 - attn[AT(b, d, r, h)]);
							else
								f = -1 * attn[AT(b, d, r, h)] * attn[AT(b, d, qq, h)];
							dattn[AT(b, d, r, h)] += f * dattn_sm[AT(b, d, qq, h)];
						}
			} else { /* :167-174 */
				for (int d = 0; d < n_tok; d++)
					for (int r = 0; r < dst_mxlen; r++)
						dattn[AT(b, d, r, h)] += attn[AT(b, d, r, h)] * dattn_sm[AT(b, d, r, h)];
			}
			for (int c = 0; c < cl; c++) { /* :176-187 */
				int dst = coo[4 * c + 0], src = coo[4 * c + 1], r = coo[4 * c + 2];
				for (int w = 0; w < width; w++) {
					REAL ws = q[QK(b, dst, h) + w] - k[QK(b, src, h) + w];
					ws = FN(sgn)(ws) * scale;
					d_q[QK(b, dst, h) + w] += ws * dattn[AT(b, dst, r, h)];
					d_k[QK(b, src, h) + w] += -1 * ws * dattn[AT(b, dst, r, h)];
				}
			}
		}
	free(dattn_sm);
	free(dattn);
#undef QK
#undef VV
#undef AT
}

#undef FN
#undef CAT
#undef CAT_
