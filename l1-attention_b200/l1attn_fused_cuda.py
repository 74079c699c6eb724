"""L1 attention with the normalisation and the value product fused in: an ADDITIONAL operator.

The reference has no counterpart module.  Every dense caller of the reference runs

    a = l1attn_cuda.L1Attn()(q, k)                      # [bs, n, n, h] scores
    a_sm = F.softmax(a, 1)
    vo = torch.einsum('bsdh, bshw -> bdhw', a_sm, v)     # README.md:64-66, testdense.py:14-16

and its README (README.md:21) names doing this without the [bs, n, n, h] tensor as the goal.
`L1AttnSoftmaxV()(q, k, v)` returns that `vo`; `mode="softmax_plus_one"` / `"exp"` give the dense
equivalents of the sparse operator's weights (python/l1attn_sparse.py:491-502: softmax with one more
all-zero source row, or plain exp).  `l1attn_cuda.L1Attn` itself is unchanged.

Forward: one kernel (`l1attn_dense_softmax_v_fwd`), nothing of size n x n is stored; it keeps the log
of every query row's normaliser ([bs, n, h]) for the backward.
Backward, a few batch items at a time: `l1attn_dense_softmax_v_bwd_dx` recomputes the weights and
writes the score gradients dx [c, n, n, h] and dv; the library's dense backward turns dx into dq, dk.
The only n x n tensor alive is that one chunk of dx (256 MB by default).
"""
import torch

import l1attn_cabi as _c

MODES = tuple(_c.SV_MODES)
_CHUNK_BYTES = 256 << 20  # score tensor of one backward chunk


class L1AttnSoftmaxVFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mode="softmax"):
        if mode not in _c.SV_MODES:
            raise ValueError("mode must be one of %s" % (MODES,))
        for name, t in (("q", q), ("k", k), ("v", v)):
            if not t.is_cuda:
                raise RuntimeError("%s must be a CUDA tensor" % name)
        if q.shape != k.shape or q.dim() != 4 or v.dim() != 4 or v.shape[:3] != q.shape[:3]:
            raise RuntimeError("q, k must be [bs, n, h, w] and v [bs, n, h, wv]")
        if q.dtype not in (torch.float32, torch.float64) or k.dtype != q.dtype or v.dtype != q.dtype:
            raise RuntimeError("q, k, v must share dtype float32 or float64")
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        lse = torch.empty(q.shape[:3], dtype=q.dtype, device=q.device)
        with torch.cuda.device(q.device):
            vo = _c.dense_softmax_v_fwd(q, k, v, mode, lse=lse)
        ctx.save_for_backward(q, k, v, vo, lse)
        ctx.mode = mode
        return vo

    @staticmethod
    def backward(ctx, dvo):
        q, k, v, vo, lse = ctx.saved_tensors
        dvo = dvo.contiguous()
        bs, n, h, _ = q.shape
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        # delta[b,t,h] = sum_s weight * <v_s, dvo_t> = <vo_t, dvo_t>; the exp form has no normaliser to differentiate
        delta = torch.zeros_like(lse) if ctx.mode == "exp" else (dvo * vo).sum(-1)
        step = max(1, min(bs, _CHUNK_BYTES // max(1, n * n * h * q.element_size())))
        with torch.cuda.device(q.device):
            dx = torch.empty((step, n, n, h), dtype=q.dtype, device=q.device)
            for b0 in range(0, bs, step):
                sl = slice(b0, min(bs, b0 + step))  # leading-dimension slices of contiguous tensors stay contiguous
                c = sl.stop - sl.start
                _c.dense_softmax_v_bwd_dx(q[sl], k[sl], v[sl], dvo[sl], lse[sl], delta[sl], dx[:c], dv[sl])
                _c.dense_bwd(dx[:c], q[sl], k[sl], out=(dq[sl], dk[sl]))
        return dq, dk, dv, None


class L1AttnSoftmaxV(torch.nn.Module):
    """vo[b,t,h,:] = sum_s weight(L1 score of (t, s)) * v[b,s,h,:]; see the module docstring."""

    def __init__(self, mode="softmax"):
        super().__init__()
        if mode not in _c.SV_MODES:
            raise ValueError("mode must be one of %s" % (MODES,))
        self.mode = mode

    def forward(self, q, k, v):
        return L1AttnSoftmaxVFn.apply(q, k, v, self.mode)
