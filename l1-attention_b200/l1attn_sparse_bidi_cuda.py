"""Bidirectional sparse L1 attention on B200 -- drop-in for the reference's
`l1attn_sparse_bidi_cuda` module (cuda/l1attn_sparse_bidi_cuda.py:8-104).

    vo = L1AttnSparseBidi()(vf, vb, q, k, coo, dst_mxlen, use_softmax)

As L1AttnSparse, and every edge also carries the reverse message:
    vo[b,dst,h,:] += a * vf[b,src,h,:]        vo[b,src,h,:] += a * vb[b,dst,h,:]
use_softmax may be omitted (defaults to True).  No CPU path.
"""
import torch
from torch import nn
from torch.autograd import Function

import l1attn_sparse_bidi_cuda_drv


class L1AttnSparseBidiFn(Function):
    @staticmethod
    def forward(ctx, vf, vb, q, k, coo, dst_mxlen, *rest):
        use_softmax = rest[0] if rest else True
        ctx.n_rest = len(rest)
        vf = vf.contiguous()
        vb = vb.contiguous()
        q = q.contiguous()
        k = k.contiguous()
        dst_mxlen, use_softmax = int(dst_mxlen), bool(use_softmax)
        vo, attn = l1attn_sparse_bidi_cuda_drv.forward(vf, vb, q, k, coo, dst_mxlen, use_softmax)
        ctx.save_for_backward(vf, vb, q, k, coo, attn)
        ctx.dst_mxlen, ctx.use_softmax = dst_mxlen, use_softmax
        return vo

    @staticmethod
    def backward(ctx, dvo):
        dvo = dvo.contiguous()
        vf, vb, q, k, coo, attn = ctx.saved_tensors[:6]
        d_vf, d_vb, d_q, d_k = l1attn_sparse_bidi_cuda_drv.backward(
            dvo, vf, vb, q, k, coo, attn, ctx.dst_mxlen, ctx.use_softmax)
        return (d_vf, d_vb, d_q, d_k, None, None) + (None,) * ctx.n_rest


class L1AttnSparseBidi(nn.Module):
    def __init__(self):
        super(L1AttnSparseBidi, self).__init__()

    def forward(self, vf, vb, q, k, coo, dst_mxlen, use_softmax=True):
        return L1AttnSparseBidiFn.apply(vf, vb, q, k, coo, dst_mxlen, use_softmax)


def expandCoo(co):
    """See l1attn_sparse_cuda.expandCoo; the reference ships an identical copy in this module
    (cuda/l1attn_sparse_bidi_cuda.py:59-104)."""
    return l1attn_sparse_bidi_cuda_drv.expand_coo(torch.as_tensor(co))
