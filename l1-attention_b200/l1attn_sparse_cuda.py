"""Sparse (coordinate-list) L1 attention on B200 -- drop-in for the reference's
`l1attn_sparse_cuda` module (cuda/l1attn_sparse_cuda.py:8-101).

    coo, dst_mxlen, src_mxlen = expandCoo(co)           # co: [n_edges, 2] rows of (dst, src)
    vo = L1AttnSparse()(v, q, k, coo.cuda(), dst_mxlen, use_softmax)

Per edge (dst, src, r):  x = -(1/sqrt(width)) * sum_w |q[b,dst,h,w] - k[b,src,h,w]|,
a = exp(x) / (1 + sum_r exp(x))  (or exp(x) when use_softmax is False),  vo[b,dst,h,:] += a * v[b,src,h,:].

The reference's forward takes use_softmax as a required sixth positional argument; here it is
also accepted as a keyword and defaults to True, so both m(v,q,k,coo,dst_mxlen) and the
six-argument form work.  No CPU path.
"""
import torch
from torch import nn
from torch.autograd import Function

import l1attn_sparse_cuda_drv


class L1AttnSparseFn(Function):
    @staticmethod
    def forward(ctx, v, q, k, coo, dst_mxlen, *rest):
        use_softmax = rest[0] if rest else True
        ctx.n_rest = len(rest)
        v = v.contiguous()
        q = q.contiguous()
        k = k.contiguous()
        dst_mxlen, use_softmax = int(dst_mxlen), bool(use_softmax)
        vo, attn = l1attn_sparse_cuda_drv.forward(v, q, k, coo, dst_mxlen, use_softmax)
        ctx.save_for_backward(v, q, k, coo, attn)
        ctx.dst_mxlen, ctx.use_softmax = dst_mxlen, use_softmax
        return vo

    @staticmethod
    def backward(ctx, dvo):
        dvo = dvo.contiguous()
        v, q, k, coo, attn = ctx.saved_tensors[:5]
        d_v, d_q, d_k = l1attn_sparse_cuda_drv.backward(dvo, v, q, k, coo, attn, ctx.dst_mxlen, ctx.use_softmax)
        return (d_v, d_q, d_k, None, None) + (None,) * ctx.n_rest


class L1AttnSparse(nn.Module):
    def __init__(self):
        super(L1AttnSparse, self).__init__()

    def forward(self, v, q, k, coo, dst_mxlen, use_softmax=True):
        return L1AttnSparseFn.apply(v, q, k, coo, dst_mxlen, use_softmax)


def expandCoo(co):
    """[n_edges, 2] rows of (dst, src)  ->  (coo int32 [n_edges, 4], dst_mxlen, src_mxlen).

    coo[i] = [dst, src, dst_rank, src_rank]: the rank is the number of earlier rows with the same
    dst (resp. src); dst_rank is the softmax slot of the edge.  dst_mxlen / src_mxlen are the
    largest rank + 1.  Same values, dtype and device placement as the reference's Python loop
    (cuda/l1attn_sparse_cuda.py:58-101), computed by a GPU kernel.
    """
    return l1attn_sparse_cuda_drv.expand_coo(torch.as_tensor(co))


class SparseGraph:
    """One graph, preprocessed once and reused by every layer and step (not in the reference, whose
    callers redo `expandCoo(co)` + `.to(device)` by hand and whose kernels need no index).

    `co` is the [n_edges, 2] list of (dst, src) pairs.  Construction runs expandCoo on the GPU and keeps
    the expanded list on `device`; the kernels' edge index is built on first use and cached by the
    driver for as long as this object keeps the list alive.

        g = SparseGraph(co, device="cuda")
        vo = g.attend(v, q, k)                      # L1AttnSparse
        vo = g.attend_bidi(vf, vb, q, k)            # L1AttnSparseBidi
    """

    def __init__(self, co, device="cuda"):
        co = torch.as_tensor(co).to(device)
        self.coo, self.dst_mxlen, self.src_mxlen = expandCoo(co)
        self.n_edges = int(self.coo.shape[0])

    def attend(self, v, q, k, use_softmax=True):
        return L1AttnSparseFn.apply(v, q, k, self.coo, self.dst_mxlen, use_softmax)

    def attend_bidi(self, vf, vb, q, k, use_softmax=True):
        import l1attn_sparse_bidi_cuda
        return l1attn_sparse_bidi_cuda.L1AttnSparseBidiFn.apply(vf, vb, q, k, self.coo, self.dst_mxlen, use_softmax)
