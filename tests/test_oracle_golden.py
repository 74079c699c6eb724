"""Pins the CPU oracle (oracle/l1attn_oracle.c) to the reference.

Three anchors, strongest first:
  * arrays named *_cpp in tests/golden/ are outputs of the reference's compiled CPU extension
    (cpp/l1attn_drv.cpp, cpp/l1attn_sparse_drv.cpp, cpp/l1attn_sparse_bidi_drv.cpp): the oracle
    restates the same loops in the same order, so fp64 results must be BIT-EXACT;
  * arrays named *_py come from the reference's pure-PyTorch code (different summation order):
    fp64 within 1e-12, norm-wise;
  * the known-answer fixtures of the reference's own tests (kat.npz).
"""
import numpy as np
import pytest

from conftest import assert_close
from oracle import oracle

TOL64 = 1e-12


def test_kat_dense(golden):
    g = golden["kat"]
    assert_close(oracle.dense_fwd(g["f1_q"], g["f1_k"]), g["f1_dense_attn"], 1e-6, "f1 dense")
    attn = oracle.dense_fwd(g["f3_q"], g["f3_k"])
    assert_close(attn, g["f3_attn"], 1e-6, "f3 dense")
    # the one-hot fixture has exact answers: -L1/sqrt(4)
    expect = np.array([[-1, -1, 0, -.5], [0, -1, -1, -.5], [-1, 0, -1, -.5], [-.5, -.5, -.5, 0]], dtype=np.float32)
    assert np.array_equal(attn[0, :, :, 0], expect)
    e = np.exp(attn.astype(np.float64))
    sm = e / e.sum(1, keepdims=True)
    vo = np.einsum("bsdh,bshw->bdhw", sm, g["f3_v"].astype(np.float64))
    assert_close(vo, g["f3_vo"], 1e-6, "f3 softmax+einsum")


@pytest.mark.parametrize("tag", ["co5", "co9"])
@pytest.mark.parametrize("usm", [1, 0])
def test_kat_sparse(golden, tag, usm):
    g = golden["kat"]
    coo, dm, sm = oracle.expand_coo(g["f1_%s_co" % tag])
    assert np.array_equal(coo, g["f1_%s_coo" % tag]) and coo.dtype == np.int32
    assert [dm, sm] == list(g["f1_%s_mxlen" % tag])
    vo, _ = oracle.sparse_fwd(g["f1_v"], g["f1_q"], g["f1_k"], coo, dm, usm)
    assert_close(vo, g["f1_%s_vo_sm%d" % (tag, usm)], 1e-6, "f1 sparse")
    # row permutation must not change the result (python/l1attn_sparse.py:508-512)
    perm = np.random.RandomState(3).permutation(coo.shape[0])
    coo2, dm2, _ = oracle.expand_coo(g["f1_%s_co" % tag][perm])
    vo2, _ = oracle.sparse_fwd(g["f1_v"], g["f1_q"], g["f1_k"], coo2, dm2, usm)
    assert_close(vo2, vo, 1e-6, "f1 permuted")


@pytest.mark.parametrize("usm", [1, 0])
def test_kat_sparse_equals_dense(golden, usm):
    """sparse(full cartesian COO) == dense scores + softmax with an extra zero logit + V einsum
    (python/l1attn_sparse.py:491-506)."""
    g = golden["kat"]
    q, k, v = (g[x].astype(np.float64) for x in ("f1_q", "f1_k", "f1_v"))
    coo, dm, _ = oracle.expand_coo(g["f1_co9_co"])
    vo, _ = oracle.sparse_fwd(v, q, k, coo, dm, usm)
    a = oracle.dense_fwd(q, k)  # [b, s, t, h]
    e = np.exp(a)
    w = e / (1.0 + e.sum(1, keepdims=True)) if usm else e
    assert_close(vo, np.einsum("bsdh,bshw->bdhw", w, v), 1e-12, "sparse==dense")


@pytest.mark.parametrize("usm", [1, 0])
def test_kat_bidi(golden, usm):
    g = golden["kat"]
    coo, dm, sm = oracle.expand_coo(g["f2_co"])
    assert np.array_equal(coo, g["f2_coo"]) and [dm, sm] == list(g["f2_mxlen"])
    vo, _ = oracle.sparse_bidi_fwd(g["f2_vf"], g["f2_vb"], g["f1_q"], g["f1_k"], coo, dm, usm)
    assert_close(vo, g["f2_vo_sm%d" % usm], 1e-6, "f2 bidi")


def test_dense_seeded(golden):
    g = golden["dense"]
    for name in g["names"]:
        q, k, da = g[name + "_q"], g[name + "_k"], g[name + "_dattn"]
        attn = oracle.dense_fwd(q, k)
        dq, dk = oracle.dense_bwd(da, q, k)
        assert_close(attn, g[name + "_attn_py"], TOL64, name + " attn vs py")
        assert_close(dq, g[name + "_dq_py"], TOL64, name + " dq vs py")
        assert_close(dk, g[name + "_dk_py"], TOL64, name + " dk vs py")
        if name + "_attn_cpp" in g:
            assert np.array_equal(attn, g[name + "_attn_cpp"]), name
            assert np.array_equal(dq, g[name + "_dq_cpp"]), name
            assert np.array_equal(dk, g[name + "_dk_cpp"]), name
        # fp32 instantiation of the same loops stays within fp32 rounding of the fp64 result
        a32 = oracle.dense_fwd(q.astype(np.float32), k.astype(np.float32))
        assert_close(a32, attn, 2e-6, name + " f32")


def test_dense_ties_are_zero(golden):
    """sign(0) = 0: with q == k everywhere both gradients vanish (cpp/l1attn_drv.cpp:7-11)."""
    g = golden["dense"]
    q = g["ties_q"]
    dq, dk = oracle.dense_bwd(g["ties_dattn"], q, q[:, ::-1][:, ::-1])
    bs, n, h, w = q.shape
    # token t against itself contributes nothing; compare against an explicit formula
    s = np.sign(q[:, None, :, :, :] - q[:, :, None, :, :])  # [b, s, t, h, w]
    ref_dq = np.einsum("bsthw,bsth->bthw", s, g["ties_dattn"]) * (-1.0 / np.sqrt(w))
    assert_close(dq, ref_dq, TOL64, "ties dq")
    assert (s == 0).sum() > bs * n * h * w  # the case really has off-diagonal ties


@pytest.mark.parametrize("usm", [1, 0])
def test_sparse_seeded(golden, usm):
    g = golden["sparse"]
    for name in g["names"]:
        coo, dm, sm = oracle.expand_coo(g[name + "_co"])
        assert np.array_equal(coo, g[name + "_coo"]) and [dm, sm] == list(g[name + "_mxlen"])
        v, vb, q, k, dvo = (g["%s_%s" % (name, x)] for x in ("v", "vb", "q", "k", "dvo"))
        tag = "%s_sm%d" % (name, usm)
        vo, attn = oracle.sparse_fwd(v, q, k, coo, dm, usm)
        dv, dq, dk = oracle.sparse_bwd(dvo, v, q, k, coo, attn, dm, usm)
        for x, y in ((vo, "vo"), (dv, "dv"), (dq, "dq"), (dk, "dk")):
            assert_close(x, g["%s_%s_py" % (tag, y)], TOL64, "%s %s vs py" % (tag, y))
        bvo, battn = oracle.sparse_bidi_fwd(v, vb, q, k, coo, dm, usm)
        bdv, bdvb, bdq, bdk = oracle.sparse_bidi_bwd(dvo, v, vb, q, k, coo, battn, dm, usm)
        for x, y in ((bvo, "vo"), (bdv, "dv"), (bdvb, "dvb"), (bdq, "dq"), (bdk, "dk")):
            assert_close(x, g["%s_bidi_%s_py" % (tag, y)], TOL64, "%s bidi %s vs py" % (tag, y))
        if tag + "_vo_cpp" in g:
            for x, y in ((vo, "vo"), (attn, "attn"), (dv, "dv"), (dq, "dq"), (dk, "dk")):
                assert np.array_equal(x, g["%s_%s_cpp" % (tag, y)]), (tag, y)
            for x, y in ((bvo, "vo"), (battn, "attn"), (bdv, "dv"), (bdvb, "dvb"), (bdq, "dq"), (bdk, "dk")):
                assert np.array_equal(x, g["%s_bidi_%s_cpp" % (tag, y)]), (tag, "bidi", y)


def test_expandcoo_golden(golden):
    g = golden["expandcoo"]
    for name in g["names"]:
        coo, dm, sm = oracle.expand_coo(g[name + "_co"])
        assert coo.dtype == np.int32 and np.array_equal(coo, g[name + "_coo"]), name
        assert [dm, sm] == list(g[name + "_mxlen"]), name


def test_expandcoo_empty():
    coo, dm, sm = oracle.expand_coo(np.zeros((0, 2), dtype=np.int64))
    assert coo.shape == (0, 4) and (dm, sm) == (1, 1)


@pytest.mark.parametrize("mode", ["softmax", "softmax_plus_one", "exp"])
def test_dense_softmax_v_golden(golden, mode):
    """Scores -> normalisation -> value product as the reference's own modules compute it
    (README.md:64-66 and the zero-padded "+1" forms of python/l1attn_sparse.py:491-502)."""
    g = golden["fused"]
    for name in g["names"]:
        q, k, v = g[name + "_q"], g[name + "_k"], g[name + "_v"]
        # 'far' holds scores near -320: exp() there amplifies the last-bit differences of the scores
        assert_close(oracle.dense_softmax_v(q, k, v, mode), g["%s_%s" % (name, mode)],
                     1e-11 if name == "far" else TOL64, "%s %s" % (name, mode))
    # testdense.py:20-39 one-hot fixture, softmax form
    k3 = golden["kat"]
    if mode == "softmax":
        assert_close(oracle.dense_softmax_v(k3["f3_q"], k3["f3_k"], k3["f3_v"], mode), k3["f3_vo"], 1e-6, "testdense fixture")
