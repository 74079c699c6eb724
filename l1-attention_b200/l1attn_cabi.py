"""ctypes binding of libl1attn_b200.so (the C ABI declared in include/l1attn_b200.h).

Two layers:
  * `lib()` -- the loaded library with argument types set; raises if it has not been built.
  * thin helpers that take numpy arrays in HOST memory (the *_host entry points: copies in,
    runs on the current CUDA device, copies out) or torch CUDA tensors (device-pointer entry
    points, enqueued on the current torch stream, no synchronisation).

Nothing here computes on the CPU: without the library or without a GPU the calls fail.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libl1attn_b200.so")
F32, F64, F16, BF16 = 0, 1, 2, 3  # F16 / BF16: storage types of the sparse forward only

_c = ctypes
_vp, _i, _ll, _sz = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_size_t
# name -> (restype, argtypes); one entry per declaration in include/l1attn_b200.h
SIGNATURES = {
    "l1attn_version": (_i, []),
    "l1attn_strerror": (_c.c_char_p, [_i]),
    "l1attn_last_cuda_error": (_i, []),
    "l1attn_device_status": (_i, []),
    "l1attn_device_status_async": (_i, [_vp, _vp]),
    "l1attn_test_wait_timeout": (_i, [_i, _vp, _vp]),
    "l1attn_dense_fwd": (_i, [_vp] * 3 + [_i] * 5 + [_vp]),
    "l1attn_dense_softmax_v_fwd": (_i, [_vp] * 5 + [_i] * 7 + [_vp]),
    "l1attn_dense_softmax_v_bwd_dx": (_i, [_vp] * 8 + [_i] * 6 + [_vp]),
    "l1attn_dense_bwd_scratch_bytes": (_sz, [_i] * 5),
    "l1attn_dense_bwd": (_i, [_vp] * 6 + [_i] * 5 + [_vp]),
    "l1attn_sparse_index_bytes": (_sz, [_i] * 3),
    "l1attn_sparse_build_index": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "l1attn_sparse_fwd": (_i, [_vp] * 7 + [_i] * 10 + [_vp]),
    "l1attn_sparse_bwd_scratch_bytes": (_sz, [_i] * 5),
    "l1attn_sparse_bwd": (_i, [_vp] * 12 + [_i] * 10 + [_vp]),
    "l1attn_sparse_bwd_static_capacity": (_sz, []),
    "l1attn_sparse_bwd_static": (_i, [_vp] * 11 + [_i] * 10 + [_vp]),
    "l1attn_expand_coo_scratch_bytes": (_sz, [_ll]),
    "l1attn_expand_coo": (_i, [_vp, _i, _vp, _vp, _ll, _ll, _vp, _vp]),
    "l1attn_i64_minmax": (_i, [_vp, _ll, _vp, _vp]),
    "l1attn_dense_fwd_host": (_i, [_vp] * 3 + [_i] * 5),
    "l1attn_dense_softmax_v_fwd_host": (_i, [_vp] * 4 + [_i] * 7),
    "l1attn_dense_bwd_host": (_i, [_vp] * 5 + [_i] * 5),
    "l1attn_sparse_fwd_host": (_i, [_vp] * 7 + [_i] * 10),
    "l1attn_sparse_bwd_host": (_i, [_vp] * 11 + [_i] * 10),
    "l1attn_dense_fwd_host_async": (_i, [_vp] * 3 + [_i] * 5),
    "l1attn_dense_bwd_host_async": (_i, [_vp] * 5 + [_i] * 5),
    "l1attn_sparse_fwd_host_async": (_i, [_vp] * 7 + [_i] * 10),
    "l1attn_sparse_bwd_host_async": (_i, [_vp] * 11 + [_i] * 10),
    "l1attn_host_sync": (_i, []),
    "l1attn_expand_coo_host": (_i, [_vp, _i, _vp, _c.POINTER(_i), _c.POINTER(_i)]),
    "l1attn_host_release": (_i, []),
}

_LIB = None


class L1AttnError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        msg = lib().l1attn_strerror(code).decode()
        super().__init__("%s: %s (code %d, cuda error %d)" % (where, msg, code, lib().l1attn_last_cuda_error()))


def lib():
    """Load libl1attn_b200.so.  There is no fallback: a missing library is an error."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s not built -- run `python build.py` in %s" % (LIB_PATH, _HERE))
        l = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            f = getattr(l, name)
            f.restype, f.argtypes = res, args
        _LIB = l
    return _LIB


def _check(rc, where):
    if rc != 0:
        raise L1AttnError(rc, where)


# ------------------------------------------------------------------ host (numpy) helpers

def _np(a, dtype=None):
    return np.ascontiguousarray(a, dtype=dtype)


def _dt(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float64:
        return F64
    raise TypeError("float32 or float64 expected, got %s" % a.dtype)


def _ptr(a):
    return None if a is None else a.ctypes.data


def dense_fwd_host(q, k, out=None, wait=True):
    """wait=False: only enqueue (l1attn_dense_fwd_host_async); the result is valid after host_sync() and the
    arrays passed in must stay alive and unchanged until then."""
    q = _np(q)
    k = _np(k, q.dtype)
    bs, n, h, w = q.shape
    attn = np.empty((bs, n, n, h), dtype=q.dtype) if out is None else out
    f = lib().l1attn_dense_fwd_host if wait else lib().l1attn_dense_fwd_host_async
    _hold(wait, q, k, attn)
    _check(f(_ptr(q), _ptr(k), _ptr(attn), bs, n, h, w, _dt(q)), "l1attn_dense_fwd_host")
    return attn


_PENDING = []  # arrays of calls enqueued with wait=False: kept alive until host_sync()


def _hold(wait, *arrays):
    if not wait:
        _PENDING.append(arrays)


def host_sync():
    """Wait for every *_host call enqueued with wait=False; raises the first deferred error."""
    rc = lib().l1attn_host_sync()
    del _PENDING[:]
    _check(rc, "l1attn_host_sync")


SV_MODES = {"softmax": 0, "softmax_plus_one": 1, "exp": 2}


def dense_softmax_v_fwd_host(q, k, v, mode="softmax"):
    """vo = sum_s a[b,s,t,h] v[b,s,h,:] with a = the chosen normalisation of the L1 scores (numpy in/out)."""
    q = _np(q)
    k, v = _np(k, q.dtype), _np(v, q.dtype)
    bs, n, h, w = q.shape
    vo = np.empty_like(v)
    _check(lib().l1attn_dense_softmax_v_fwd_host(_ptr(q), _ptr(k), _ptr(v), _ptr(vo), bs, n, h, w, v.shape[3],
                                                 SV_MODES[mode], _dt(q)), "l1attn_dense_softmax_v_fwd_host")
    return vo


def dense_bwd_host(d_attn, q, k, out=None, wait=True):
    q = _np(q)
    k, d_attn = _np(k, q.dtype), _np(d_attn, q.dtype)
    bs, n, h, w = q.shape
    dq, dk = (np.empty_like(q), np.empty_like(q)) if out is None else out
    f = lib().l1attn_dense_bwd_host if wait else lib().l1attn_dense_bwd_host_async
    _hold(wait, d_attn, q, k, dq, dk)
    _check(f(_ptr(d_attn), _ptr(q), _ptr(k), _ptr(dq), _ptr(dk), bs, n, h, w, _dt(q)), "l1attn_dense_bwd_host")
    return dq, dk


def sparse_fwd_host(v, q, k, coo, dst_mxlen, use_softmax=True, vb=None, out=None, wait=True):
    """vb given -> bidirectional operator.  Returns (vo, attn); out=(vo, attn) reuses caller arrays
    (pinned ones make the copies back run at full PCIe rate)."""
    q = _np(q)
    k, v = _np(k, q.dtype), _np(v, q.dtype)
    vb = None if vb is None else _np(vb, q.dtype)
    coo = _np(coo, np.int32)
    bs, n, h, w = q.shape
    wv = v.shape[3]
    if out is None:
        vo = np.empty((bs, n, h, wv), dtype=q.dtype)
        attn = np.empty((bs, n, int(dst_mxlen), h), dtype=q.dtype)
    else:
        vo, attn = out
    f = lib().l1attn_sparse_fwd_host if wait else lib().l1attn_sparse_fwd_host_async
    _hold(wait, v, vb, q, k, coo, vo, attn)
    _check(f(_ptr(v), _ptr(vb), _ptr(q), _ptr(k), _ptr(coo), _ptr(vo), _ptr(attn),
             bs, n, h, w, wv, coo.shape[0], int(dst_mxlen), int(bool(use_softmax)),
             int(vb is not None), _dt(q)), "l1attn_sparse_fwd_host")
    return vo, attn


def sparse_bwd_host(dvo, v, q, k, coo, attn, dst_mxlen, use_softmax=True, vb=None, out=None, wait=True):
    """Returns (d_v, d_q, d_k) or, with vb, (d_vf, d_vb, d_q, d_k); out=(d_v, d_vb or None, d_q, d_k) reuses caller arrays."""
    q = _np(q)
    k, v, dvo, attn = _np(k, q.dtype), _np(v, q.dtype), _np(dvo, q.dtype), _np(attn, q.dtype)
    vb = None if vb is None else _np(vb, q.dtype)
    coo = _np(coo, np.int32)
    bs, n, h, w = q.shape
    wv = v.shape[3]
    if out is None:
        dv, dq, dk = np.empty_like(v), np.empty_like(q), np.empty_like(q)
        dvb = np.empty_like(v) if vb is not None else None
    else:
        dv, dvb, dq, dk = out
    f = lib().l1attn_sparse_bwd_host if wait else lib().l1attn_sparse_bwd_host_async
    _hold(wait, dvo, v, vb, q, k, coo, attn, dv, dvb, dq, dk)
    _check(f(_ptr(dvo), _ptr(v), _ptr(vb), _ptr(q), _ptr(k), _ptr(coo), _ptr(attn),
             _ptr(dv), _ptr(dvb), _ptr(dq), _ptr(dk), bs, n, h, w, wv, coo.shape[0],
             int(dst_mxlen), int(bool(use_softmax)), int(vb is not None), _dt(q)),
           "l1attn_sparse_bwd_host")
    return (dv, dq, dk) if vb is None else (dv, dvb, dq, dk)


def expand_coo_host(co):
    co = _np(co, np.int64).reshape(-1, 2)
    cl = co.shape[0]
    coo = np.zeros((cl, 4), dtype=np.int32)
    dm, sm = _c.c_int(0), _c.c_int(0)
    _check(lib().l1attn_expand_coo_host(_ptr(co), cl, _ptr(coo), _c.byref(dm), _c.byref(sm)),
           "l1attn_expand_coo_host")
    return coo, dm.value, sm.value


# ------------------------------------------------------------------ device (torch) helpers

def _tdt(t, allow16=False):
    import torch
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.float64:
        return F64
    if allow16 and t.dtype == torch.float16:
        return F16
    if allow16 and t.dtype == torch.bfloat16:
        return BF16
    raise TypeError("float32 or float64 expected, got %s" % t.dtype)


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def _dp(t):
    return None if t is None else t.data_ptr()


def dense_fwd(q, k, out=None):
    """q, k: contiguous CUDA tensors [bs, n, h, w].  Enqueues on the current stream."""
    import torch
    assert q.is_cuda and q.is_contiguous() and k.is_contiguous() and q.shape == k.shape
    bs, n, h, w = q.shape
    attn = torch.empty((bs, n, n, h), dtype=q.dtype, device=q.device) if out is None else out
    _check(lib().l1attn_dense_fwd(_dp(q), _dp(k), _dp(attn), bs, n, h, w, _tdt(q), _stream()), "l1attn_dense_fwd")
    return attn


def dense_softmax_v_fwd(q, k, v, mode="softmax", out=None, lse=None):
    """q, k: [bs, n, h, w], v: [bs, n, h, wv], contiguous CUDA tensors.  Enqueues on the current stream.
    lse: optional [bs, n, h] tensor receiving the log-normalisers (needed by dense_softmax_v_bwd_dx)."""
    import torch
    assert q.is_cuda and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    assert k.shape == q.shape and v.shape[:3] == q.shape[:3] and k.dtype == q.dtype and v.dtype == q.dtype
    bs, n, h, w = q.shape
    vo = torch.empty_like(v) if out is None else out
    assert lse is None or (lse.is_contiguous() and lse.shape == q.shape[:3] and lse.dtype == q.dtype)
    _check(lib().l1attn_dense_softmax_v_fwd(_dp(q), _dp(k), _dp(v), _dp(vo), _dp(lse), bs, n, h, w, v.shape[3],
                                            SV_MODES[mode], _tdt(q), _stream()), "l1attn_dense_softmax_v_fwd")
    return vo


def dense_softmax_v_bwd_dx(q, k, v, dvo, lse, delta, dx, dv):
    """Fills dx [bs, n, n, h] (layout of d_attn) and dv [bs, n, h, wv]; all tensors contiguous, same dtype."""
    for t in (q, k, v, dvo, lse, delta, dx, dv):
        assert t.is_cuda and t.is_contiguous() and t.dtype == q.dtype
    bs, n, h, w = q.shape
    assert dx.shape == (bs, n, n, h) and dv.shape == v.shape and lse.shape == (bs, n, h) and delta.shape == (bs, n, h)
    _check(lib().l1attn_dense_softmax_v_bwd_dx(_dp(q), _dp(k), _dp(v), _dp(dvo), _dp(lse), _dp(delta), _dp(dx), _dp(dv),
                                               bs, n, h, w, v.shape[3], _tdt(q), _stream()), "l1attn_dense_softmax_v_bwd_dx")


def dense_bwd(d_attn, q, k, out=None, scratch="auto"):
    """scratch: "auto" allocates l1attn_dense_bwd_scratch_bytes() with torch, None passes NULL
    (every tile then runs the exact loop), or a uint8 CUDA tensor of at least that size."""
    import torch
    assert q.is_cuda and q.is_contiguous() and k.is_contiguous() and d_attn.is_contiguous()
    bs, n, h, w = q.shape
    dq, dk = (torch.empty_like(q), torch.empty_like(k)) if out is None else out
    if isinstance(scratch, str):
        scratch = torch.empty(lib().l1attn_dense_bwd_scratch_bytes(bs, n, h, w, _tdt(q)), dtype=torch.uint8,
                              device=q.device)
    _check(lib().l1attn_dense_bwd(_dp(d_attn), _dp(q), _dp(k), _dp(dq), _dp(dk), _dp(scratch), bs, n, h, w, _tdt(q),
                                  _stream()), "l1attn_dense_bwd")
    return dq, dk


class SparseIndex:
    """Device-resident edge index of one coo tensor (see l1attn_sparse_build_index)."""

    def __init__(self, coo, n_tok, dst_mxlen):
        import torch
        assert coo.is_cuda and coo.dtype == torch.int32 and coo.is_contiguous() and coo.shape[1] == 4
        self.cl, self.n_tok, self.dst_mxlen = int(coo.shape[0]), int(n_tok), int(dst_mxlen)
        nbytes = lib().l1attn_sparse_index_bytes(self.cl, self.n_tok, self.dst_mxlen)
        self.buf = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=coo.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=coo.device)
        _check(lib().l1attn_sparse_build_index(_dp(coo), self.cl, self.n_tok, self.dst_mxlen, _dp(self.buf),
                                               _dp(self.status), _stream()), "l1attn_sparse_build_index")

    def check(self):
        """Synchronises; raises if coo held an out-of-range row."""
        _check(int(self.status.item()), "coo")


def sparse_fwd(v, q, k, index, use_softmax=True, vb=None, out=None):
    import torch
    bs, n, h, w = q.shape
    wv = v.shape[3]
    if out is None:
        vo = torch.empty((bs, n, h, wv), dtype=q.dtype, device=q.device)
        attn = torch.empty((bs, n, index.dst_mxlen, h), dtype=q.dtype, device=q.device)
    else:
        vo, attn = out
    _check(lib().l1attn_sparse_fwd(_dp(v), _dp(vb), _dp(q), _dp(k), _dp(index.buf), _dp(vo), _dp(attn), bs, n, h, w,
                                   wv, index.cl, index.dst_mxlen, int(bool(use_softmax)), int(vb is not None),
                                   _tdt(q, allow16=True), _stream()), "l1attn_sparse_fwd")
    return vo, attn


def sparse_bwd(dvo, v, q, k, index, attn, use_softmax=True, vb=None, out=None, scratch=None):
    import torch
    bs, n, h, w = q.shape
    wv = v.shape[3]
    if out is None:
        out = (torch.empty_like(v), torch.empty_like(v) if vb is not None else None,
               torch.empty_like(q), torch.empty_like(k))
    dv, dvb, dq, dk = out
    if scratch is None:
        scratch = torch.empty_like(attn)
    _check(lib().l1attn_sparse_bwd(_dp(dvo), _dp(v), _dp(vb), _dp(q), _dp(k), _dp(index.buf), _dp(attn), _dp(dv),
                                   _dp(dvb), _dp(dq), _dp(dk), _dp(scratch), bs, n, h, w, wv, index.cl,
                                   index.dst_mxlen, int(bool(use_softmax)), int(vb is not None), _tdt(q), _stream()),
           "l1attn_sparse_bwd")
    return (dv, dq, dk) if vb is None else (dv, dvb, dq, dk)


def sparse_bwd_static(dvo, v, q, k, index, attn, use_softmax=True, vb=None, out=None):
    """As sparse_bwd, through l1attn_sparse_bwd_static: the d(logit) scratch is the library's own
    fixed device array, so neither this helper nor the library allocates scratch for the call
    (the gradient tensors are allocated here only when `out` is not given)."""
    import torch
    bs, n, h, w = q.shape
    wv = v.shape[3]
    if out is None:
        out = (torch.empty_like(v), torch.empty_like(v) if vb is not None else None,
               torch.empty_like(q), torch.empty_like(k))
    dv, dvb, dq, dk = out
    _check(lib().l1attn_sparse_bwd_static(_dp(dvo), _dp(v), _dp(vb), _dp(q), _dp(k), _dp(index.buf), _dp(attn),
                                          _dp(dv), _dp(dvb), _dp(dq), _dp(dk), bs, n, h, w, wv, index.cl,
                                          index.dst_mxlen, int(bool(use_softmax)), int(vb is not None), _tdt(q),
                                          _stream()), "l1attn_sparse_bwd_static")
    return (dv, dq, dk) if vb is None else (dv, dvb, dq, dk)
