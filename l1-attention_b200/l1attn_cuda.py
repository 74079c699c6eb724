"""Dense L1 attention scores on B200 -- drop-in for the reference's `l1attn_cuda` module
(cuda/l1attn_cuda.py:7-32): same class names, same call signatures, same tensor layouts.

    attn = L1Attn()(q, k)        # q, k: [batch, n_tokens, heads, width], float32 or float64, CUDA
    attn[b, s, t, h] = -(1/sqrt(width)) * sum_w |q[b, t, h, w] - k[b, s, h, w]|

`attn` is indexed [batch, src (key), dst (query), heads]: take the softmax over dim 1 and apply V
with einsum('bsdh,bshw->bdhw').  The backward gives d_q and d_k with sign(0) = 0.

There is no CPU path: the compiled driver (l1attn_cuda_drv, built by build.py in this
directory) must be present and the tensors must live on a CUDA device.
"""
import torch
from torch import nn
from torch.autograd import Function

import l1attn_cuda_drv  # torch must be imported first: the driver links against libtorch


class L1AttnFn(Function):
    @staticmethod
    def forward(ctx, q, k):
        q = q.contiguous()
        k = k.contiguous()
        attn = l1attn_cuda_drv.forward(q, k)
        ctx.save_for_backward(q, k)
        return attn[0]

    @staticmethod
    def backward(ctx, d_attn):
        q, k = ctx.saved_tensors[:2]
        # autograd may hand over an expanded / strided gradient (e.g. from .sum()); the reference
        # driver rejects those (cuda/l1attn_cuda_drv.cpp:71), here they are made contiguous.
        d_q, d_k = l1attn_cuda_drv.backward(d_attn.contiguous(), q, k)
        return d_q, d_k


class L1Attn(nn.Module):
    def __init__(self):
        super(L1Attn, self).__init__()

    def forward(self, q, k):
        return L1AttnFn.apply(q, k)
