"""ctypes/numpy front end of the CPU oracle (oracle/l1attn_oracle.c).

TEST INFRASTRUCTURE ONLY -- imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg; the GPU library never imports it and has no CPU
fallback.

Function names and argument order follow the reference's driver entry points
(cpp/l1attn_drv.cpp:13,60; cpp/l1attn_sparse_drv.cpp:13,98;
cpp/l1attn_sparse_bidi_drv.cpp:15,103) and expandCoo
(cuda/l1attn_sparse_cuda.py:58).  Inputs are numpy arrays (float64 or float32,
C-contiguous); outputs are fresh numpy arrays of the same dtype.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    """Compile liboracle with the Makefile beside this file (gcc -O2)."""
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libl1attn_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def _sfx(a):
    if a.dtype == np.float64:
        return "f64"
    if a.dtype == np.float32:
        return "f32"
    raise TypeError("oracle works in float64 or float32, got %s" % a.dtype)


def _c(a, dtype=None):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def dense_fwd(q, k):
    q, k = _c(q), _c(k, q.dtype)
    bs, n, h, w = q.shape
    attn = np.empty((bs, n, n, h), dtype=q.dtype)
    getattr(lib(), "oracle_dense_fwd_" + _sfx(q))(_p(q), _p(k), _p(attn), bs, n, h, w)
    return attn


def dense_bwd(d_attn, q, k):
    q = _c(q)
    k, d_attn = _c(k, q.dtype), _c(d_attn, q.dtype)
    bs, n, h, w = q.shape
    dq, dk = np.empty_like(q), np.empty_like(q)
    getattr(lib(), "oracle_dense_bwd_" + _sfx(q))(_p(d_attn), _p(q), _p(k), _p(dq), _p(dk), bs, n, h, w)
    return dq, dk


SV_MODES = {"softmax": 0, "softmax_plus_one": 1, "exp": 2}


def dense_softmax_v(q, k, v, mode="softmax"):
    """vo[b,t,h,:] = sum_s a[b,s,t,h] v[b,s,h,:], a = softmax / "+1" softmax / exp of the dense L1 scores."""
    q = _c(q)
    k, v = _c(k, q.dtype), _c(v, q.dtype)
    bs, n, h, w = q.shape
    vo, scratch = np.empty_like(v), np.empty(max(n, 1), dtype=q.dtype)
    getattr(lib(), "oracle_dense_softmax_v_" + _sfx(q))(_p(q), _p(k), _p(v), _p(vo), _p(scratch), bs, n, h, w,
                                                        v.shape[3], SV_MODES[mode])
    return vo


def _coo(coo):
    coo = _c(coo, np.int32)
    assert coo.ndim == 2 and coo.shape[1] == 4, "coo must be [cl,4] (output of expandCoo)"
    return coo


def _sparse_fwd(v, vb, q, k, coo, dst_mxlen, use_softmax, bidi):
    q = _c(q)
    k, v = _c(k, q.dtype), _c(v, q.dtype)
    vb = _c(vb, q.dtype) if bidi else v
    coo = _coo(coo)
    bs, n, h, w = q.shape
    wv = v.shape[3]
    vo = np.empty((bs, n, h, wv), dtype=q.dtype)
    attn = np.empty((bs, n, int(dst_mxlen), h), dtype=q.dtype)
    getattr(lib(), "oracle_sparse_fwd_" + _sfx(q))(
        _p(v), _p(vb), _p(q), _p(k), _p(coo), _p(vo), _p(attn),
        bs, n, h, w, wv, coo.shape[0], int(dst_mxlen), int(bool(use_softmax)), int(bidi))
    return vo, attn


def _sparse_bwd(dvo, v, vb, q, k, coo, attn, dst_mxlen, use_softmax, bidi):
    q = _c(q)
    k, v, dvo, attn = _c(k, q.dtype), _c(v, q.dtype), _c(dvo, q.dtype), _c(attn, q.dtype)
    vb = _c(vb, q.dtype) if bidi else v
    coo = _coo(coo)
    bs, n, h, w = q.shape
    wv = v.shape[3]
    dv, dvb = np.empty_like(v), np.empty_like(v)
    dq, dk = np.empty_like(q), np.empty_like(q)
    getattr(lib(), "oracle_sparse_bwd_" + _sfx(q))(
        _p(dvo), _p(v), _p(vb), _p(q), _p(k), _p(coo), _p(attn), _p(dv), _p(dvb), _p(dq), _p(dk),
        bs, n, h, w, wv, coo.shape[0], int(dst_mxlen), int(bool(use_softmax)), int(bidi))
    return (dv, dvb, dq, dk) if bidi else (dv, dq, dk)


def sparse_fwd(v, q, k, coo, dst_mxlen, use_softmax=True):
    """-> (vo, attn), as l1attnSparse_forward."""
    return _sparse_fwd(v, None, q, k, coo, dst_mxlen, use_softmax, 0)


def sparse_bwd(dvo, v, q, k, coo, attn, dst_mxlen, use_softmax=True):
    """-> (d_v, d_q, d_k), as l1attnSparse_backward."""
    return _sparse_bwd(dvo, v, None, q, k, coo, attn, dst_mxlen, use_softmax, 0)


def sparse_bidi_fwd(vf, vb, q, k, coo, dst_mxlen, use_softmax=True):
    """-> (vo, attn), as l1attnSparseBidi_forward."""
    return _sparse_fwd(vf, vb, q, k, coo, dst_mxlen, use_softmax, 1)


def sparse_bidi_bwd(dvo, vf, vb, q, k, coo, attn, dst_mxlen, use_softmax=True):
    """-> (d_vf, d_vb, d_q, d_k), as l1attnSparseBidi_backward."""
    return _sparse_bwd(dvo, vf, vb, q, k, coo, attn, dst_mxlen, use_softmax, 1)


def expand_coo(co):
    """co: integer [cl,2] rows (dst, src) -> (coo int32 [cl,4], dst_mxlen, src_mxlen)."""
    co = _c(co, np.int64).reshape(-1, 2)
    cl = co.shape[0]
    coo = np.zeros((cl, 4), dtype=np.int32)
    dm, sm = ctypes.c_int(0), ctypes.c_int(0)
    rc = lib().oracle_expand_coo(_p(co), cl, _p(coo), ctypes.byref(dm), ctypes.byref(sm))
    if rc != 0:
        raise MemoryError("oracle_expand_coo: key range too large")
    return coo, dm.value, sm.value
