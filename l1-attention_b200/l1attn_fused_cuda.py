"""L1 attention with the normalisation and the value product fused in: an ADDITIONAL operator.

The reference has no counterpart module.  Every dense caller of the reference runs

    a = l1attn_cuda.L1Attn()(q, k)                      # [bs, n, n, h] scores
    a_sm = F.softmax(a, 1)
    vo = torch.einsum('bsdh, bshw -> bdhw', a_sm, v)     # README.md:64-66, testdense.py:14-16

and its README (README.md:21) names doing this without the [bs, n, n, h] tensor as the goal.
`L1AttnSoftmaxV()(q, k, v)` returns that `vo`; `mode="softmax_plus_one"` / `"exp"` give the dense
equivalents of the sparse operator's weights (python/l1attn_sparse.py:491-502: softmax with one more
all-zero source row, or plain exp).  `l1attn_cuda.L1Attn` itself is unchanged.

Forward: one kernel (`l1attn_dense_softmax_v_fwd`), nothing of size n x n is stored.
Backward: recomputes the scores a few batch items at a time with the library's dense forward,
applies the softmax/value-product derivatives with torch ops on that chunk and feeds the result to
the library's dense backward, so the peak extra memory is a few chunk-sized [c, n, n, h] tensors
instead of four full ones.
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
        with torch.cuda.device(q.device):
            vo = _c.dense_softmax_v_fwd(q, k, v, mode)
        ctx.save_for_backward(q, k, v)
        ctx.mode = mode
        return vo

    @staticmethod
    def backward(ctx, dvo):
        q, k, v = ctx.saved_tensors
        mode = ctx.mode
        dvo = dvo.contiguous()
        bs, n, h, _ = q.shape
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        step = max(1, _CHUNK_BYTES // max(1, n * n * h * q.element_size()))
        with torch.cuda.device(q.device):
            for b0 in range(0, bs, step):
                sl = slice(b0, min(bs, b0 + step))
                qb, kb = q[sl], k[sl]  # leading-dimension slices of contiguous tensors stay contiguous
                x = _c.dense_fwd(qb, kb)  # [c, s, t, h]
                if mode == "softmax":
                    a = torch.softmax(x, 1)
                else:
                    a = torch.exp(x)
                    if mode == "softmax_plus_one":
                        a = a / (1 + a.sum(1, keepdim=True))
                del x
                dv[sl] = torch.einsum("bsdh,bdhw->bshw", a, dvo[sl])
                da = torch.einsum("bdhw,bshw->bsdh", dvo[sl], v[sl])
                if mode == "exp":
                    dx = a * da
                else:  # the extra row of "+1" has a zero value vector, so the same Jacobian applies
                    dx = a * (da - (a * da).sum(1, keepdim=True))
                del a, da
                _c.dense_bwd(dx.contiguous(), qb, kb, out=(dq[sl], dk[sl]))
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
