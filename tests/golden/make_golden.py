"""Generate the committed golden vectors under tests/golden/ by RUNNING THE REFERENCE.

Run where a checkout of the reference is available:

    python tests/golden/make_golden.py --ref <path to tlh24/l1-attention checkout>

It imports the reference's pure-PyTorch implementations (python/l1attn.py,
python/l1attn_baseline.py, python/l1attn_sparse.py) and, when oracle/_ref/ has been
built with oracle/build_ref.py, the reference's compiled CPU extension, runs them on
(a) the reference's own hand-written fixtures and (b) seeded random inputs, and
stores inputs and outputs as .npz files.  The tests then need neither the reference
checkout nor torch-side reference code.

Files written:
  kat.npz      known-answer fixtures of python/l1attn_sparse.py:444-581 and testdense.py:20-39
  dense.npz    seeded dense cases (incl. ties and zero-padded tokens), fwd + grads
  sparse.npz   seeded sparse / bidi cases (cartesian, permuted, rows dropped, ragged), fwd + grads
  expandcoo.npz  expandCoo inputs and outputs
  fused.npz    dense consumer chain (scores -> softmax / "+1" softmax / exp -> value product)
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def load_reference(ref):
    sys.path.insert(0, os.path.join(ref, "python"))
    import l1attn as ref_dense_naive  # python/l1attn.py
    import l1attn_baseline as ref_dense_fn  # python/l1attn_baseline.py
    import l1attn_sparse as ref_sparse  # python/l1attn_sparse.py
    cpp = {}
    refdir = os.path.join(ROOT, "oracle", "_ref")
    if os.path.exists(os.path.join(refdir, "l1attn_drv_cpp.so")):
        sys.path.insert(0, refdir)
        import l1attn_drv_cpp
        import l1attn_sparse_drv
        import l1attn_sparse_bidi_drv
        cpp = dict(dense=l1attn_drv_cpp, sparse=l1attn_sparse_drv, bidi=l1attn_sparse_bidi_drv)
    return ref_dense_naive, ref_dense_fn, ref_sparse, cpp


def np_(t):
    return t.detach().cpu().numpy().copy()


def kat(ref_dense_naive, ref_sparse):
    out = {}
    # fixture of sparseNonsparseTest / bidiTest (python/l1attn_sparse.py:450-482, :522-543)
    q = torch.tensor([[0, 1, 2], [2, 1, 0], [0, 0, 0]], dtype=torch.float32).reshape(1, 3, 1, 3)
    k = torch.tensor([[2, 1, 0], [0, 1, 2], [0, 1, 2]], dtype=torch.float32).reshape(1, 3, 1, 3)
    v = torch.tensor([[-2, 2, 3], [2, -2, 2], [3, 2, -2]], dtype=torch.float32).reshape(1, 3, 1, 3)
    out["f1_q"], out["f1_k"], out["f1_v"] = np_(q), np_(k), np_(v)
    out["f1_dense_attn"] = np_(ref_dense_naive.L1Attn()(q, k))
    for tag, co in (("co5", [[0, 0], [0, 1], [1, 0], [1, 1], [2, 2]]),
                    ("co9", [[d, s] for d in range(3) for s in range(3)])):
        co = torch.tensor(co)
        coo, dm, sm = ref_sparse.expandCoo(co)
        out["f1_%s_co" % tag] = np_(co)
        out["f1_%s_coo" % tag] = np_(coo)
        out["f1_%s_mxlen" % tag] = np.array([dm, sm])
        for usm in (True, False):
            vo = ref_sparse.L1AttnSparse()(v, q, k, coo, dm, sm, usm)
            out["f1_%s_vo_sm%d" % (tag, usm)] = np_(vo)
    # bidiTest (python/l1attn_sparse.py:516-581)
    vf = torch.diag(torch.tensor([1.0, 2.0, 3.0])).reshape(1, 3, 1, 3)
    vb = torch.diag(torch.tensor([-1.0, -2.0, -3.0])).reshape(1, 3, 1, 3)
    co = torch.tensor([[0, 0], [0, 1], [0, 2], [1, 0], [1, 1], [2, 0], [2, 1]])
    coo, dm, sm = ref_sparse.expandCoo(co)
    out["f2_vf"], out["f2_vb"], out["f2_co"], out["f2_coo"] = np_(vf), np_(vb), np_(co), np_(coo)
    out["f2_mxlen"] = np.array([dm, sm])
    for usm in (True, False):
        out["f2_vo_sm%d" % usm] = np_(ref_sparse.L1AttnSparseBidi()(vf, vb, q, k, coo, dm, sm, usm))
    # testdense.py:20-39 one-hot fixture
    q3 = torch.zeros(1, 4, 1, 4)
    k3 = torch.zeros(1, 4, 1, 4)
    v3 = torch.zeros(1, 4, 1, 4)
    q3[0, 0, 0, :] = torch.tensor([0.0, 1, 0, 0])
    q3[0, 1, 0, :] = torch.tensor([0.0, 0, 1, 0])
    q3[0, 2, 0, :] = torch.tensor([1.0, 0, 0, 0])
    k3[0, 0, 0, :] = torch.tensor([1.0, 0, 0, 0])
    k3[0, 1, 0, :] = torch.tensor([0.0, 1, 0, 0])
    k3[0, 2, 0, :] = torch.tensor([0.0, 0, 1, 0])
    v3[0, 0, 0, :] = torch.tensor([1.0, 0, 0, 1])
    v3[0, 1, 0, :] = torch.tensor([0.0, 1, 0, 2])
    v3[0, 2, 0, :] = torch.tensor([0.0, 0, 1, 3])
    a3 = ref_dense_naive.L1Attn()(q3, k3)
    out["f3_q"], out["f3_k"], out["f3_v"], out["f3_attn"] = np_(q3), np_(k3), np_(v3), np_(a3)
    out["f3_vo"] = np_(torch.einsum("bsdh, bshw -> bdhw", torch.softmax(a3, 1), v3))
    return out


def dense_cases(ref_dense_naive, ref_dense_fn, cpp):
    out = {}
    cases = [  # name, shape, kind
        ("check", (1, 16, 8, 64), "randn"),  # check.py:17-22 shape
        ("odd", (2, 5, 3, 7), "randn"),
        ("w33", (1, 9, 2, 33), "randn"),
        ("t17", (2, 17, 5, 16), "randn"),
        ("ties", (2, 12, 4, 8), "quant"),  # values on a grid of 1/2: many exact ties q==k
        ("padded", (1, 16, 2, 8), "padded"),  # last 6 tokens all-zero in q and k (setfind.py:124-128)
    ]
    g = torch.Generator().manual_seed(20241)
    names = []
    for name, shape, kind in cases:
        q = torch.randn(shape, generator=g, dtype=torch.float64)
        k = torch.randn(shape, generator=g, dtype=torch.float64)
        if kind == "quant":
            q, k = torch.round(q * 2) / 2, torch.round(k * 2) / 2
        if kind == "padded":
            q[:, 10:] = 0
            k[:, 10:] = 0
        bs, n, h, w = shape
        d_attn = torch.randn((bs, n, n, h), generator=g, dtype=torch.float64)
        attn = ref_dense_naive.L1Attn()(q, k)
        qq, kk = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
        ref_dense_fn.L1AttnFn.apply(qq, kk).backward(d_attn)
        out["%s_q" % name], out["%s_k" % name], out["%s_dattn" % name] = np_(q), np_(k), np_(d_attn)
        out["%s_attn_py" % name] = np_(attn)
        out["%s_dq_py" % name], out["%s_dk_py" % name] = np_(qq.grad), np_(kk.grad)
        if cpp:
            out["%s_attn_cpp" % name] = np_(cpp["dense"].forward(q, k)[0])
            dq, dk = cpp["dense"].backward(d_attn, q, k)
            out["%s_dq_cpp" % name], out["%s_dk_cpp" % name] = np_(dq), np_(dk)
        names.append(name)
    out["names"] = np.array(names)
    return out


def sparse_cases(ref_sparse, cpp):
    out = {}
    g = torch.Generator().manual_seed(20242)
    names = []

    def graph(kind, n):
        if kind == "cart":  # check_sparse.py: full cartesian product
            return torch.cartesian_prod(torch.arange(n), torch.arange(n))
        if kind == "perm":
            co = torch.cartesian_prod(torch.arange(n), torch.arange(n))
            return co[torch.randperm(co.shape[0], generator=g)]
        if kind == "drop":  # permuted with 4 rows dropped (check_sparse.py:58-60)
            co = torch.cartesian_prod(torch.arange(n), torch.arange(n))
            return co[torch.randperm(co.shape[0], generator=g)][:-4]
        if kind == "ragged":  # random degrees, duplicates allowed, some tokens never dst / never src
            rows = []
            for d in range(n):
                deg = int(torch.randint(0, 6, (1,), generator=g))
                for _ in range(deg):
                    rows.append([d, int(torch.randint(0, n - 1, (1,), generator=g))])
            co = torch.tensor(rows)
            return co[torch.randperm(co.shape[0], generator=g)]
        raise ValueError(kind)

    cases = [  # name, (bs, n, h, w), graph
        ("cart", (2, 3, 16, 7), "cart"),  # check_sparse.py:18-21 shape
        ("perm", (2, 3, 16, 7), "perm"),
        ("drop", (2, 3, 16, 7), "drop"),
        ("ragged", (2, 12, 3, 5), "ragged"),
        ("w64", (1, 10, 8, 64), "ragged"),
    ]
    for name, shape, kind in cases:
        bs, n, h, w = shape
        co = graph(kind, n)
        coo, dm, sm = ref_sparse.expandCoo(co)
        t = {x: torch.randn(shape, generator=g, dtype=torch.float64) for x in ("q", "k", "v", "vb", "dvo")}
        if name == "ragged":  # put exact ties into the sign() path
            t["q"], t["k"] = torch.round(t["q"] * 2) / 2, torch.round(t["k"] * 2) / 2
        out["%s_co" % name], out["%s_coo" % name] = np_(co), np_(coo)
        out["%s_mxlen" % name] = np.array([dm, sm])
        for x in t:
            out["%s_%s" % (name, x)] = np_(t[x])
        for usm in (True, False):
            tag = "%s_sm%d" % (name, usm)
            # one-directional, reference pure-PyTorch module + autograd
            leaf = {x: t[x].clone().requires_grad_(True) for x in ("v", "q", "k")}
            vo = ref_sparse.L1AttnSparse()(leaf["v"], leaf["q"], leaf["k"], coo, dm, sm, usm)
            vo.backward(t["dvo"])
            out[tag + "_vo_py"] = np_(vo)
            for x in leaf:
                out[tag + "_d%s_py" % x] = np_(leaf[x].grad)
            # bidirectional
            leaf = {x: t[x].clone().requires_grad_(True) for x in ("v", "vb", "q", "k")}
            vo = ref_sparse.L1AttnSparseBidi()(leaf["v"], leaf["vb"], leaf["q"], leaf["k"], coo, dm, sm, usm)
            vo.backward(t["dvo"])
            out[tag + "_bidi_vo_py"] = np_(vo)
            for x in leaf:
                out[tag + "_bidi_d%s_py" % x] = np_(leaf[x].grad)
            if cpp:
                vo, attn = cpp["sparse"].forward(t["v"], t["q"], t["k"], coo, dm, usm)
                dv, dq, dk = cpp["sparse"].backward(t["dvo"], t["v"], t["q"], t["k"], coo, attn, dm, usm)
                out[tag + "_vo_cpp"], out[tag + "_attn_cpp"] = np_(vo), np_(attn)
                out[tag + "_dv_cpp"], out[tag + "_dq_cpp"], out[tag + "_dk_cpp"] = np_(dv), np_(dq), np_(dk)
                vo, attn = cpp["bidi"].forward(t["v"], t["vb"], t["q"], t["k"], coo, dm, usm)
                dvf, dvb, dq, dk = cpp["bidi"].backward(t["dvo"], t["v"], t["vb"], t["q"], t["k"], coo, attn, dm, usm)
                out[tag + "_bidi_vo_cpp"], out[tag + "_bidi_attn_cpp"] = np_(vo), np_(attn)
                out[tag + "_bidi_dv_cpp"], out[tag + "_bidi_dvb_cpp"] = np_(dvf), np_(dvb)
                out[tag + "_bidi_dq_cpp"], out[tag + "_bidi_dk_cpp"] = np_(dq), np_(dk)
        names.append(name)
    out["names"] = np.array(names)
    return out


def fused_cases(ref_dense_naive):
    """Dense consumer chain run with the reference's own L1Attn module (python/l1attn.py):
    README.md:64-66 (softmax over dim 1, then einsum) and the zero-padded "+1" variant of
    python/l1attn_sparse.py:491-502 (with and without softmax)."""
    import torch.nn.functional as F
    out, names = {}, []
    g = torch.Generator().manual_seed(20243)
    for name, shape, wv in [("readme", (2, 3, 4, 8), 8), ("w32", (1, 70, 2, 32), 32), ("odd", (1, 9, 2, 7), 5),
                            ("far", (1, 20, 2, 64), 64)]:
        bs, n, h, w = shape
        q = torch.randn(shape, generator=g, dtype=torch.float64)
        k = torch.randn(shape, generator=g, dtype=torch.float64)
        if name == "far":  # every score far below zero: the plain softmax must shift by the maximum
            k = k + 40.0
        v = torch.randn((bs, n, h, wv), generator=g, dtype=torch.float64)
        a = ref_dense_naive.L1Attn()(q, k)
        out[name + "_q"], out[name + "_k"], out[name + "_v"] = np_(q), np_(k), np_(v)
        out[name + "_softmax"] = np_(torch.einsum("bsdh, bshw -> bdhw", F.softmax(a, 1), v))
        ap = torch.zeros(bs, n + 1, n + 1, h, dtype=torch.float64)
        ap[:, :-1, :-1, :] = a
        out[name + "_softmax_plus_one"] = np_(torch.einsum("bsdh, bshw -> bdhw", F.softmax(ap, 1)[:, :-1, :-1, :], v))
        out[name + "_exp"] = np_(torch.einsum("bsdh, bshw -> bdhw", torch.exp(ap)[:, :-1, :-1, :], v))
        names.append(name)
    out["names"] = np.array(names)
    return out


def expandcoo_cases(ref_sparse):
    out = {}
    g = torch.Generator().manual_seed(20243)
    cos = {
        "readme": torch.cartesian_prod(torch.arange(3), torch.arange(3)),  # README.md:89
        "single": torch.tensor([[5, 2]]),
        "dups": torch.tensor([[1, 1], [1, 1], [0, 1], [1, 1], [7, 0], [0, 1]]),
        "rand": torch.randint(0, 50, (700, 2), generator=g),
        "hub": torch.stack([torch.randint(0, 40, (300,), generator=g), torch.full((300,), 3)], 1),
    }
    # the benchmark's graph recipe at a reduced size: self edge + 7 distinct other srcs per dst, permuted
    n = 64
    r = torch.rand(n, n, generator=g)
    r.fill_diagonal_(2)
    src = r.argsort(1)[:, :7]
    rows = torch.cat([torch.stack([torch.arange(n).repeat_interleave(7), src.reshape(-1)], 1),
                      torch.stack([torch.arange(n), torch.arange(n)], 1)])
    cos["bench64"] = rows[torch.randperm(rows.shape[0], generator=g)]
    for name, co in cos.items():
        coo, dm, sm = ref_sparse.expandCoo(co)
        out[name + "_co"], out[name + "_coo"], out[name + "_mxlen"] = np_(co), np_(coo), np.array([dm, sm])
    out["names"] = np.array(list(cos))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True)
    ap.add_argument("--only", default="", help="comma-separated fixture names (default: all)")
    a = ap.parse_args()
    ref_dense_naive, ref_dense_fn, ref_sparse, cpp = load_reference(a.ref)
    if not cpp:
        print("note: oracle/_ref not built -- *_cpp arrays are omitted (tests then skip the bit-exact checks)")
    torch.manual_seed(0)
    makers = {
        "kat": lambda: kat(ref_dense_naive, ref_sparse),
        "dense": lambda: dense_cases(ref_dense_naive, ref_dense_fn, cpp),
        "sparse": lambda: sparse_cases(ref_sparse, cpp),
        "expandcoo": lambda: expandcoo_cases(ref_sparse),
        "fused": lambda: fused_cases(ref_dense_naive),
    }
    for f in (a.only.split(",") if a.only else makers):
        np.savez_compressed(os.path.join(HERE, f + ".npz"), **makers[f]())
        print(f, os.path.getsize(os.path.join(HERE, f + ".npz")), "bytes")


if __name__ == "__main__":
    main()
