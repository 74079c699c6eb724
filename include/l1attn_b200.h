/*
 * l1attn_b200.h -- C ABI of libl1attn_b200.so: L1-distance attention on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes, returns 0 (L1ATTN_OK) or a negative
 * L1ATTN_ERR_* code, and never calls into Python or PyTorch.  There is no CPU fallback: without a
 * CUDA device every compute entry point returns L1ATTN_ERR_CUDA.
 *
 * Two families:
 *   *  device-pointer entry points (l1attn_dense_fwd ...): all tensors already live in the
 *      memory of the CURRENT device; work is enqueued on `stream` (a cudaStream_t passed as
 *      void*, NULL = the legacy default stream) and the call returns without synchronising.
 *      They allocate nothing; scratch and index buffers are passed in by the caller.
 *   *  host-buffer entry points (l1attn_*_host): tensors are in host memory; the call copies
 *      them to the current device, runs, copies results back and synchronises.  The work is
 *      pipelined one batch item at a time over three streams of the library's own, so copies in
 *      both directions overlap the kernels.  The *_host_async forms return once everything is
 *      enqueued; l1attn_host_sync() waits.  Device memory for these calls comes from a
 *      grow-only arena per device that the library keeps until l1attn_host_release() or process exit.
 *
 * Tensor layouts (row-major, contiguous), identical to the reference extension:
 *   q, k, v, vf, vb, vo and their gradients : [bs][n_tok][n_heads][width]   (v*: v_width)
 *   dense attn / d_attn                     : [bs][n_tok (key, s)][n_tok (query, t)][n_heads]
 *   sparse attn                             : [bs][n_tok][dst_mxlen][n_heads]  (post-softmax)
 *   coo                                     : int32 [cl][4] = {dst, src, dst_rank, src_rank}
 * dtype: L1ATTN_F32 or L1ATTN_F64 for every floating tensor of a call.
 *
 * Reference interfaces these replace are cited per function as file:line of tlh24/l1-attention.
 */
#ifndef L1ATTN_B200_H
#define L1ATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define L1ATTN_OK 0
#define L1ATTN_ERR_ARG (-1)      /* NULL pointer, negative size, unknown dtype */
#define L1ATTN_ERR_SHAPE (-2)    /* size beyond what the kernels index (see each function) */
#define L1ATTN_ERR_CUDA (-3)     /* a CUDA runtime call or launch failed; see l1attn_last_cuda_error() */
#define L1ATTN_ERR_INDEX (-4)    /* coo holds a token / rank outside [0,n_tok) / [0,dst_mxlen) */
#define L1ATTN_ERR_NOMEM (-5)    /* host-buffer entry point could not get device memory */
#define L1ATTN_ERR_ALIGN (-6)    /* a floating tensor pointer is not aligned to its element size */
#define L1ATTN_ERR_SCRATCH (-8)  /* problem needs more scratch than the library's built-in buffer holds */
#define L1ATTN_ERR_TIMEOUT (-7)  /* a kernel gave up a bounded wait on an asynchronous copy (its output is invalid) */

#define L1ATTN_F32 0
#define L1ATTN_F64 1
#define L1ATTN_F16 2  /* IEEE half storage, float arithmetic: l1attn_sparse_fwd only */
#define L1ATTN_BF16 3 /* bfloat16 storage, float arithmetic: l1attn_sparse_fwd only */

/* normalisation of l1attn_dense_softmax_v_fwd */
#define L1ATTN_SV_SOFTMAX 0          /* softmax over the source tokens (F.softmax(attn, 1)) */
#define L1ATTN_SV_SOFTMAX_PLUS_ONE 1 /* exp(x) / (1 + sum exp(x)): softmax with one more all-zero source row */
#define L1ATTN_SV_EXP 2              /* exp(x), no normalisation */

/* Library version (major*10000 + minor*100 + patch). */
int l1attn_version(void);
/* Static description of an L1ATTN_ERR_* code. */
const char *l1attn_strerror(int code);
/* cudaError_t (as int) of the last failing CUDA call made by this library on this thread, 0 if none. */
int l1attn_last_cuda_error(void);
/*
 * Synchronises with the device and reports whether any kernel of this library gave up a bounded
 * wait since the last call (L1ATTN_ERR_TIMEOUT, cleared by the call) -- the kernels that stage
 * tiles with asynchronous bulk copies never spin without a limit.  L1ATTN_OK otherwise.
 */
int l1attn_device_status(void);
/*
 * The same word without a synchronisation: enqueues a copy of it to *host_word on `stream` (use pinned host
 * memory) and returns; the word is not cleared.  A caller that launches on one stream can thus look at
 * *host_word before its next call and pay for l1attn_device_status() only when it is non-zero.
 * No counterpart in the reference, whose kernels have no waits and whose launchers check no errors.
 */
int l1attn_device_status_async(int *host_word, void *stream);
/*
 * Test hook, not an operator: launches one warp that waits at most limit_us (1..100000) microseconds on a
 * barrier nothing completes.  The wait gives up, l1attn_device_status() then reports L1ATTN_ERR_TIMEOUT once
 * and L1ATTN_OK after; returned_dev (two device ints) receives {1, number of failed polls} when the kernel
 * has returned from the wait.
 * Nothing faults or hangs.  No counterpart in the reference.
 */
int l1attn_test_wait_timeout(int limit_us, int *returned_dev, void *stream);

/* ------------------------------------------------------------------ dense --------------- */

/*
 * attn[b][s][t][h] = (-1/sqrt(width)) * sum_w |q[b][t][h][w] - k[b][s][h][w]|.
 * Replaces l1attn_cuda_drv.forward (cuda/l1attn_cuda_drv.cpp:42-65) and the three launchers
 * l1attn_cuda_forward{,32,64} (cuda/l1attn_cuda_kernel.cu:457-557).  Any bs, n_tok, n_heads,
 * width >= 1; every element of attn is written (no memset needed).
 */
int l1attn_dense_fwd(const void *q, const void *k, void *attn,
		     int bs, int n_tok, int n_heads, int width, int dtype, void *stream);

/*
 * d_q[b][t][h][w] =  scale * sum_s sign(q[b][t][h][w]-k[b][s][h][w]) * d_attn[b][s][t][h]
 * d_k[b][s][h][w] = -scale * sum_t sign(q[b][t][h][w]-k[b][s][h][w]) * d_attn[b][s][t][h]
 * with scale = -1/sqrt(width) and sign(0) = 0.  Deterministic (no atomics).
 * `scratch`: device buffer of l1attn_dense_bwd_scratch_bytes() bytes (256-byte aligned), or NULL.
 * In fp32 a detector kernel proves every exact tie q == k -- the one case the fast inner loop (compare +
 * predicated adds) gets wrong -- and writes them there as a list, which a fix kernel applies after the
 * backward, plus one flag per tile for the case that the list overflows (zero-padded tokens, q == k:
 * flagged tiles then take an exact loop).  The rest of the buffer receives the shares of d_k that the
 * single-visit kernel leaves per block of 128 query rows: ceil(n_tok / 128) * sizeof(d_k) bytes, i.e.
 * about width / 128 times the size of d_attn (plus 2 or 4 times sizeof(d_q) for shapes whose work items
 * split their source rows: long context with a small batch).  With NULL every tile takes the exact loop and no scratch is
 * needed (same results, about 2.7 times the time in fp32).  Contents need no initialisation and mean
 * nothing after the call; calls that share a scratch buffer must not overlap on the GPU.
 * Replaces l1attn_cuda_drv.backward (cuda/l1attn_cuda_drv.cpp:67-104) and
 * l1attn_cuda_backward{,32,64} (cuda/l1attn_cuda_kernel.cu:559-685).
 */
size_t l1attn_dense_bwd_scratch_bytes(int bs, int n_tok, int n_heads, int width, int dtype);
int l1attn_dense_bwd(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k, void *scratch,
		     int bs, int n_tok, int n_heads, int width, int dtype, void *stream);

/*
 * Dense scores, normalisation and value product in one pass, without the [bs, n_tok, n_tok, n_heads]
 * score tensor:
 *   x[b][s][t][h]  = (-1/sqrt(width)) * sum_w |q[b][t][h][w] - k[b][s][h][w]|
 *   a              = softmax_s(x) | exp(x) / (1 + sum_s exp(x)) | exp(x)        (mode L1ATTN_SV_*)
 *   vo[b][t][h][:] = sum_s a[b][s][t][h] * v[b][s][h][:]                         v, vo: [bs][n_tok][n_heads][v_width]
 * The reference has no single function for this: it is the sequence every dense caller runs right
 * after l1attn_cuda.L1Attn -- F.softmax(a, 1) and einsum('bsdh,bshw->bdhw') (README.md:64-66,
 * testdense.py:14-16) -- and its README (README.md:21) names the fusion as the goal.  The "+1" and
 * exp forms are the dense equivalents of the sparse operator's weights
 * (python/l1attn_sparse.py:491-502).  No scratch memory.
 * lse: NULL, or [bs][n_tok][n_heads] receiving the log of each query row's normaliser (weight of
 * (s, t) = exp(x - lse); zeros for L1ATTN_SV_EXP) -- what l1attn_dense_softmax_v_bwd_dx needs.
 */
int l1attn_dense_softmax_v_fwd(const void *q, const void *k, const void *v, void *vo, void *lse,
			       int bs, int n_tok, int n_heads, int width, int v_width,
			       int mode, int dtype, void *stream);

/*
 * First half of the backward of l1attn_dense_softmax_v_fwd (no counterpart in the reference either):
 *   p              = exp(x[b][s][t][h] - lse[b][t][h])
 *   dx[b][s][t][h] = p * (<v[b][s][h][:], dvo[b][t][h][:]> - delta[b][t][h])
 *   dv[b][s][h][:] = sum_t p * dvo[b][t][h][:]
 * with delta[b][t][h] = <dvo[b][t][h][:], vo[b][t][h][:]> for the two softmax forms and zeros for
 * L1ATTN_SV_EXP (the caller computes it: one elementwise product and a row sum).  dx has the layout
 * of d_attn, so l1attn_dense_bwd(dx, q, k, d_q, d_k, ...) is the second half.  Only dx is of size
 * n_tok x n_tok; callers bound it by passing a few batch items per call (every pointer advanced to
 * the first item of the chunk, bs = items in the chunk).
 */
int l1attn_dense_softmax_v_bwd_dx(const void *q, const void *k, const void *v, const void *dvo,
				  const void *lse, const void *delta, void *dx, void *dv,
				  int bs, int n_tok, int n_heads, int width, int v_width,
				  int dtype, void *stream);

/* ------------------------------------------------------------------ sparse -------------- */

/*
 * Edge index derived from coo, shared by forward and backward of both sparse operators.
 * l1attn_sparse_index_bytes() gives the size of the device buffer the caller provides;
 * l1attn_sparse_build_index() fills it (a few small kernels on `stream`).  The index depends
 * only on (coo, n_tok, dst_mxlen) and can be reused for every call on the same graph.
 * `status` (device int32, may be NULL) receives 0, or L1ATTN_ERR_INDEX if a row of coo is out
 * of range; such rows are skipped, never dereferenced.
 * No counterpart in the reference, whose kernels scatter with atomicAdd per edge
 * (cuda/l1attn_sparse_cuda_kernel.cu:148-181,327-370) and need no index.
 */
size_t l1attn_sparse_index_bytes(int cl, int n_tok, int dst_mxlen);
int l1attn_sparse_build_index(const int32_t *coo, int cl, int n_tok, int dst_mxlen,
			      void *index, int32_t *status, void *stream);

/*
 * Forward of L1AttnSparse (bidi = 0) / L1AttnSparseBidi (bidi = 1):
 *   x[b][dst][r][h] = scale * sum_w |q[b][dst][h][w] - k[b][src][h][w]|      per coo row (dst,src,r)
 *   a = exp(x) / (1 + sum_r exp(x))   (use_softmax)   or   a = exp(x)        (slots without an edge: 0)
 *   vo[b][dst][h][:] += a * v[b][src][h][:]           and, bidi:  vo[b][src][h][:] += a * vb[b][dst][h][:]
 * Writes every element of vo and attn.  vb is ignored unless bidi.
 * Replaces l1attn_sparse_cuda_drv.forward (cuda/l1attn_sparse_cuda_drv.cpp:32-46,
 * cuda/l1attn_sparse_cuda_kernel.cu:373-445) and l1attn_sparse_bidi_cuda_drv.forward
 * (cuda/l1attn_sparse_bidi_cuda_drv.cpp:34-50, cuda/l1attn_sparse_cuda_kernel.cu:651-725).
 * dtype may also be L1ATTN_F16 / L1ATTN_BF16 here (and only here): v, vb, q, k, vo, attn are then
 * 16-bit tensors, the arithmetic is float; the reference dispatches Half in its sparse forward only
 * (cuda/l1attn_sparse_cuda_kernel.cu:405, :483).
 */
int l1attn_sparse_fwd(const void *v, const void *vb, const void *q, const void *k,
		      const void *index, void *vo, void *attn,
		      int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
		      int use_softmax, int bidi, int dtype, void *stream);

/*
 * Backward of the same operators.  `attn` is the tensor the forward returned.  `scratch` is a
 * device buffer of l1attn_sparse_bwd_scratch_bytes() bytes (holds d(logit) per attn slot).
 * Outputs d_v (d_vf when bidi), d_vb (bidi only, else ignored), d_q, d_k; every element written.
 * Replaces l1attn_sparse_cuda_drv.backward (cuda/l1attn_sparse_cuda_drv.cpp:48-69,
 * cuda/l1attn_sparse_cuda_kernel.cu:447-531) and the bidi backward
 * (cuda/l1attn_sparse_bidi_cuda_drv.cpp:52-75, cuda/l1attn_sparse_cuda_kernel.cu:727-815).
 */
size_t l1attn_sparse_bwd_scratch_bytes(int bs, int n_tok, int n_heads, int dst_mxlen, int dtype);
int l1attn_sparse_bwd(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
		      const void *index, const void *attn,
		      void *d_v, void *d_vb, void *d_q, void *d_k, void *scratch,
		      int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
		      int use_softmax, int bidi, int dtype, void *stream);

/*
 * l1attn_sparse_bwd for callers that cannot allocate device memory at the point where they run the
 * backward (a plugin that only receives device pointers from its host runtime, or code in a region
 * where cudaMalloc is forbidden or would stall the device).  Same arguments without `scratch`: the
 * d(logit) buffer is a fixed 32 MiB array inside the library's device image
 * (l1attn_sparse_bwd_static_capacity() bytes), so the call allocates nothing, neither with the CUDA
 * runtime nor through any library.  It fails with L1ATTN_ERR_SCRATCH, before launching anything, when
 * l1attn_sparse_bwd_scratch_bytes(bs, n_tok, n_heads, dst_mxlen, dtype) exceeds that capacity.
 * The first call on each device looks up the array's device address (a CUDA runtime query, no
 * allocation); make that first call outside any stream capture.  All calls on a device share the one
 * array: calls whose kernels can overlap on the GPU (different streams) must not be issued
 * concurrently; on a single stream they are ordered and safe.  The array keeps whatever the last call
 * left; the kernels overwrite every entry they later read, so nothing needs clearing.
 * No counterpart in the reference, whose backward allocates its two scratch tensors with torch
 * on every call (cuda/l1attn_sparse_cuda_kernel.cu:447-531).
 */
size_t l1attn_sparse_bwd_static_capacity(void);
int l1attn_sparse_bwd_static(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
			     const void *index, const void *attn,
			     void *d_v, void *d_vb, void *d_q, void *d_k,
			     int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
			     int use_softmax, int bidi, int dtype, void *stream);

/* ------------------------------------------------------------------ expandCoo ----------- */

/*
 * coo[i] = {dst_i, src_i, #{j<i : dst_j == dst_i}, #{j<i : src_j == src_i}} (int32) from
 * co = int64 [cl][2] rows {dst, src}; mxlen[0] / mxlen[1] (device int32[2]) receive the largest
 * dst / src rank + 1 (1 when cl == 0).  Keys must lie in [key_lo, key_lo + n_keys); `counters`
 * is a device buffer of l1attn_expand_coo_scratch_bytes(n_keys) bytes (may be NULL when that is 0).
 * Bit-exact replacement of expandCoo (cuda/l1attn_sparse_cuda.py:58-101), which is a Python loop.
 * l1attn_i64_minmax writes {min, max} over n int64 values to out (device int64[2]).
 */
size_t l1attn_expand_coo_scratch_bytes(long long n_keys);
int l1attn_expand_coo(const int64_t *co, int cl, int32_t *coo, int32_t *mxlen,
		      long long key_lo, long long n_keys, void *counters, void *stream);
int l1attn_i64_minmax(const int64_t *x, long long n, int64_t *out, void *stream);

/* ------------------------------------------------------------------ host buffers -------- */

/* Same operations with every tensor in HOST memory (pageable or pinned); synchronous.
 * (The reference has no host-buffer form: its callers move tensors with torch's .cuda() / .cpu() around
 * l1attn_cuda_drv.forward / backward, cuda/l1attn_cuda_drv.cpp:42-104.) */
int l1attn_dense_fwd_host(const void *q, const void *k, void *attn,
			  int bs, int n_tok, int n_heads, int width, int dtype);
int l1attn_dense_softmax_v_fwd_host(const void *q, const void *k, const void *v, void *vo,
				    int bs, int n_tok, int n_heads, int width, int v_width, int mode, int dtype);
int l1attn_dense_bwd_host(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k,
			  int bs, int n_tok, int n_heads, int width, int dtype);
int l1attn_sparse_fwd_host(const void *v, const void *vb, const void *q, const void *k, const int32_t *coo,
			   void *vo, void *attn,
			   int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
			   int use_softmax, int bidi, int dtype);
int l1attn_sparse_bwd_host(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
			   const int32_t *coo, const void *attn,
			   void *d_v, void *d_vb, void *d_q, void *d_k,
			   int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
			   int use_softmax, int bidi, int dtype);
/*
 * Asynchronous forms of the four calls above: they enqueue the copies in, the kernels and the copies out and
 * return; outputs are valid after l1attn_host_sync().  Calls enqueued before the sync work on device buffers of
 * their own and run concurrently (a backward whose d_attn does not come from the forward enqueued before it
 * overlaps that forward's copy back).  Host buffers must stay alive and unmodified until the sync; only pinned
 * host memory lets the copies overlap, pageable memory still gives correct results.  A call may wait for
 * earlier ones when the arena has to grow.  l1attn_host_sync() returns the first deferred error of the calls
 * it waited for (L1ATTN_ERR_INDEX for an out-of-range coo row) or L1ATTN_OK.
 */
int l1attn_dense_fwd_host_async(const void *q, const void *k, void *attn,
				int bs, int n_tok, int n_heads, int width, int dtype);
int l1attn_dense_bwd_host_async(const void *d_attn, const void *q, const void *k, void *d_q, void *d_k,
				int bs, int n_tok, int n_heads, int width, int dtype);
int l1attn_sparse_fwd_host_async(const void *v, const void *vb, const void *q, const void *k, const int32_t *coo,
				 void *vo, void *attn,
				 int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
				 int use_softmax, int bidi, int dtype);
int l1attn_sparse_bwd_host_async(const void *dvo, const void *v, const void *vb, const void *q, const void *k,
				 const int32_t *coo, const void *attn,
				 void *d_v, void *d_vb, void *d_q, void *d_k,
				 int bs, int n_tok, int n_heads, int width, int v_width, int cl, int dst_mxlen,
				 int use_softmax, int bidi, int dtype);
int l1attn_host_sync(void);
/* co int64 [cl][2] -> coo int32 [cl][4]; *dst_mxlen, *src_mxlen as expandCoo returns them.  Token ids must fit in
 * int32 (else L1ATTN_ERR_SHAPE) and the counters take memory proportional to max id - min id + 1. */
int l1attn_expand_coo_host(const int64_t *co, int cl, int32_t *coo, int *dst_mxlen, int *src_mxlen);
/* Free the current device's arena used by the *_host entry points. */
int l1attn_host_release(void);

#ifdef __cplusplus
}
#endif
#endif /* L1ATTN_B200_H */
