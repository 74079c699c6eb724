"""Sparse / bidirectional sparse L1 attention and expandCoo on the GPU, through the C ABI,
against the CPU oracle and the committed reference outputs.  fp64 1e-12, fp32 1e-5, integer
outputs bit-exact."""
import numpy as np
import pytest

from conftest import assert_close

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = {np.float32: 1e-5, np.float64: 1e-12}


def _cabi():
    import l1attn_cabi
    return l1attn_cabi


def _dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _host(t):
    return None if t is None else t.cpu().numpy()


def run_gpu(v, vb, q, k, dvo, coo, dm, usm):
    """forward + backward through the device-pointer C ABI; numpy in, numpy out."""
    cabi = _cabi()
    ix = cabi.SparseIndex(_dev(coo.astype(np.int32)), q.shape[1], dm)
    ix.check()
    dv_, dvb_, dq_, dk_, dvo_ = _dev(v), _dev(vb), _dev(q), _dev(k), _dev(dvo)
    vo, attn = cabi.sparse_fwd(dv_, dq_, dk_, ix, usm, vb=dvb_)
    grads = cabi.sparse_bwd(dvo_, dv_, dq_, dk_, ix, attn, usm, vb=dvb_)
    return _host(vo), _host(attn), [_host(x) for x in grads]


def run_oracle(v, vb, q, k, dvo, coo, dm, usm):
    from oracle import oracle
    f = lambda a: None if a is None else a.astype(np.float64)
    v, vb, q, k, dvo = f(v), f(vb), f(q), f(k), f(dvo)
    if vb is None:
        vo, attn = oracle.sparse_fwd(v, q, k, coo, dm, usm)
        return vo, attn, list(oracle.sparse_bwd(dvo, v, q, k, coo, attn, dm, usm))
    vo, attn = oracle.sparse_bidi_fwd(v, vb, q, k, coo, dm, usm)
    return vo, attn, list(oracle.sparse_bidi_bwd(dvo, v, vb, q, k, coo, attn, dm, usm))


def random_graph(rng, n, max_deg, self_edges=True):
    rows = []
    for d in range(n):
        deg = rng.randint(0, max_deg + 1)
        srcs = rng.choice(n, size=min(deg, n), replace=False)
        rows += [[d, s] for s in srcs]
        if self_edges and d % 3:
            rows.append([d, d])
    co = np.array(rows, dtype=np.int64).reshape(-1, 2)
    return co[rng.permutation(co.shape[0])]


CASES = [  # bs, n, h, w, wv, max_deg
    (2, 3, 16, 7, 7, 3), (1, 12, 3, 5, 5, 5), (2, 40, 8, 64, 64, 9), (1, 64, 8, 64, 32, 20),
    (2, 33, 5, 33, 12, 6), (1, 50, 2, 128, 128, 12), (1, 20, 1, 256, 64, 4), (3, 17, 12, 16, 16, 17),
    (1, 30, 40, 4, 4, 5), (1, 25, 3, 130, 2, 5),
]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("bidi", [False, True])
@pytest.mark.parametrize("usm", [True, False])
@pytest.mark.parametrize("case", CASES)
def test_vs_oracle(case, usm, bidi, dtype):
    from oracle import oracle
    bs, n, h, w, wv, deg = case
    rng = np.random.RandomState(sum(case) + 17 * usm + 31 * bidi)
    co = random_graph(rng, n, deg)
    coo, dm, _ = oracle.expand_coo(co)
    q, k = (0.3 * rng.standard_normal((bs, n, h, w)).astype(dtype) for _ in range(2))
    v, vbb, dvo = (rng.standard_normal((bs, n, h, wv)).astype(dtype) for _ in range(3))
    vb = vbb if bidi else None
    vo, attn, grads = run_gpu(v, vb, q, k, dvo, coo, dm, usm)
    rvo, rattn, rgrads = run_oracle(v, vb, q, k, dvo, coo, dm, usm)
    tol = TOL[dtype]
    assert_close(vo, rvo, tol, "vo")
    assert_close(attn, rattn, tol, "attn")
    for name, x, r in zip(("dv", "dvb", "dq", "dk") if bidi else ("dv", "dq", "dk"), grads, rgrads):
        assert_close(x, r, tol, name)


@pytest.mark.parametrize("tdtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("bidi", [False, True])
@pytest.mark.parametrize("usm", [True, False])
@pytest.mark.parametrize("case", CASES)
def test_forward_16bit_storage(case, usm, bidi, tdtype):
    """float16 / bfloat16 tensors in the forward (the reference dispatches Half there,
    cuda/l1attn_sparse_cuda_kernel.cu:405): storage is 16-bit, arithmetic float, so the result is the
    float64 oracle on the same (16-bit representable) inputs up to the rounding of the outputs:
    2^-11 relative for float16, 2^-8 for bfloat16, plus the same rounding of the stored weights."""
    from oracle import oracle
    cabi = _cabi()
    tdt = getattr(torch, tdtype)
    bs, n, h, w, wv, deg = case
    rng = np.random.RandomState(sum(case) + 5 * usm + 3 * bidi)
    co = random_graph(rng, n, deg)
    coo, dm, _ = oracle.expand_coo(co)
    mk = lambda shape, sc: (sc * torch.from_numpy(rng.standard_normal(shape))).to(tdt).cuda()
    q, k = mk((bs, n, h, w), 0.3), mk((bs, n, h, w), 0.3)
    v, vb = mk((bs, n, h, wv), 1.0), (mk((bs, n, h, wv), 1.0) if bidi else None)
    ix = cabi.SparseIndex(_dev(coo.astype(np.int32)), n, dm)
    vo, attn = cabi.sparse_fwd(v, q, k, ix, usm, vb=vb)
    assert vo.dtype == tdt and attn.dtype == tdt
    f64 = lambda t: None if t is None else t.double().cpu().numpy()
    if bidi:
        rvo, rattn = oracle.sparse_bidi_fwd(f64(v), f64(vb), f64(q), f64(k), coo, dm, usm)
    else:
        rvo, rattn = oracle.sparse_fwd(f64(v), f64(q), f64(k), coo, dm, usm)
    tol = 2e-3 if tdtype == "float16" else 1.6e-2
    assert_close(f64(vo), rvo, tol, "vo " + tdtype)
    assert_close(f64(attn), rattn, tol, "attn " + tdtype)


def test_16bit_module_forward_and_backward_error():
    """Through the module: float16 forward works, backward is refused as in the reference (whose backward
    dispatches float32 / float64 only, cuda/l1attn_sparse_cuda_kernel.cu:483)."""
    import l1attn_sparse_cuda
    co = torch.tensor([[0, 0], [0, 1], [1, 0], [2, 2], [2, 1]])
    coo, dm, _ = l1attn_sparse_cuda.expandCoo(co)
    v, q, k = (torch.randn(1, 3, 2, 32, device="cuda", dtype=torch.float16, requires_grad=True) for _ in range(3))
    vo = l1attn_sparse_cuda.L1AttnSparse()(v, q, k, coo.cuda(), dm, True)
    assert vo.dtype == torch.float16 and bool(torch.isfinite(vo).all())
    with pytest.raises(RuntimeError, match="float32 or float64"):
        vo.sum().backward()
    # the dense operator does not take 16-bit tensors at all
    import l1attn_cuda
    with pytest.raises(RuntimeError, match="float32 or float64"):
        l1attn_cuda.L1Attn()(q, k)


@pytest.mark.parametrize("usm", [1, 0])
def test_golden_fixtures(golden, usm):
    g = golden["sparse"]
    for name in g["names"]:
        coo, (dm, _) = g[name + "_coo"], g[name + "_mxlen"]
        v, vb, q, k, dvo = (g["%s_%s" % (name, x)] for x in ("v", "vb", "q", "k", "dvo"))
        tag = "%s_sm%d" % (name, usm)
        vo, attn, (dv, dq, dk) = run_gpu(v, None, q, k, dvo, coo, int(dm), usm)
        bvo, battn, (bdv, bdvb, bdq, bdk) = run_gpu(v, vb, q, k, dvo, coo, int(dm), usm)
        for ref in ("py", "cpp"):
            if tag + "_vo_" + ref not in g:
                continue
            for x, y in ((vo, "vo"), (dv, "dv"), (dq, "dq"), (dk, "dk")):
                assert_close(x, g["%s_%s_%s" % (tag, y, ref)], 1e-12, "%s %s vs %s" % (tag, y, ref))
            for x, y in ((bvo, "vo"), (bdv, "dv"), (bdvb, "dvb"), (bdq, "dq"), (bdk, "dk")):
                assert_close(x, g["%s_bidi_%s_%s" % (tag, y, ref)], 1e-12, "%s bidi %s vs %s" % (tag, y, ref))
        if tag + "_attn_cpp" in g:
            assert_close(attn, g[tag + "_attn_cpp"], 1e-12, tag + " attn")


@pytest.mark.parametrize("usm", [1, 0])
def test_kat(golden, usm):
    g = golden["kat"]
    for tag in ("co5", "co9"):
        coo, (dm, _) = g["f1_%s_coo" % tag], g["f1_%s_mxlen" % tag]
        vo, _, _ = run_gpu(g["f1_v"], None, g["f1_q"], g["f1_k"], g["f1_v"], coo, int(dm), usm)
        assert_close(vo, g["f1_%s_vo_sm%d" % (tag, usm)], 1e-6, "f1 " + tag)
    coo, (dm, _) = g["f2_coo"], g["f2_mxlen"]
    vo, _, _ = run_gpu(g["f2_vf"], g["f2_vb"], g["f1_q"], g["f1_k"], g["f2_vf"], coo, int(dm), usm)
    assert_close(vo, g["f2_vo_sm%d" % usm], 1e-6, "f2 bidi")


def test_sparse_equals_dense_and_permutation_invariance():
    """Full cartesian COO == dense scores + softmax with an extra zero logit + V einsum
    (python/l1attn_sparse.py:491-506), for any row order of the COO."""
    from oracle import oracle
    cabi = _cabi()
    rng = np.random.RandomState(9)
    bs, n, h, w = 2, 24, 4, 32
    q, k, v, dvo = (0.2 * rng.standard_normal((bs, n, h, w)) for _ in range(4))
    co = np.array([[d, s] for d in range(n) for s in range(n)], dtype=np.int64)
    a = cabi.dense_fwd(_dev(q), _dev(k)).cpu().numpy()
    e = np.exp(a)
    ref = np.einsum("bsdh,bshw->bdhw", e / (1 + e.sum(1, keepdims=True)), v)
    outs = []
    for perm in (np.arange(n * n), rng.permutation(n * n)):
        coo, dm, _ = oracle.expand_coo(co[perm])
        vo, _, grads = run_gpu(v, None, q, k, dvo, coo, dm, True)
        assert_close(vo, ref, 1e-12, "sparse == dense")
        outs.append([vo] + grads)
    for x, y in zip(*outs):
        assert_close(x, y, 1e-12, "row permutation")


def test_unfilled_slots_and_isolated_tokens():
    """dst_mxlen larger than any degree, tokens without edges: attn slots read 0, vo rows 0,
    gradients of untouched rows 0."""
    rng = np.random.RandomState(2)
    bs, n, h, w = 1, 10, 2, 8
    co = np.array([[1, 2], [1, 3], [4, 4]], dtype=np.int64)
    coo = np.array([[1, 2, 0, 0], [1, 3, 2, 0], [4, 4, 5, 0]], dtype=np.int32)  # ranks with gaps
    q, k, v, dvo = (rng.standard_normal((bs, n, h, w)).astype(np.float32) for _ in range(4))
    vo, attn, (dv, dq, dk) = run_gpu(v, None, q, k, dvo, coo, 7, True)
    rvo, rattn, (rdv, rdq, rdk) = run_oracle(v, None, q, k, dvo, coo, 7, True)
    assert_close(vo, rvo, 1e-5)
    assert_close(attn, rattn, 1e-5)
    assert np.count_nonzero(attn) == 3 * h
    assert np.count_nonzero(vo[0, [0, 2, 3, 5, 6, 7, 8, 9]]) == 0
    for x, r in ((dv, rdv), (dq, rdq), (dk, rdk)):
        assert_close(x, r, 1e-5)
    assert np.count_nonzero(dk[0, [0, 1, 5, 6, 7, 8, 9]]) == 0


def test_empty_edge_list():
    q = np.ones((1, 4, 2, 8), dtype=np.float32)
    coo = np.zeros((0, 4), dtype=np.int32)
    vo, attn, (dv, dq, dk) = run_gpu(q, None, q, q, q, coo, 1, True)
    assert not vo.any() and not attn.any() and not dv.any() and not dq.any() and not dk.any()


def test_out_of_range_rows_are_reported_not_dereferenced():
    cabi = _cabi()
    coo = torch.tensor([[0, 1, 0, 0], [9, 1, 0, 0], [1, 1, 5, 0]], dtype=torch.int32).cuda()
    ix = cabi.SparseIndex(coo, 4, 2)
    with pytest.raises(cabi.L1AttnError) as e:
        ix.check()
    assert e.value.code == -4


def test_host_buffer_entry_points():
    from oracle import oracle
    cabi = _cabi()
    rng = np.random.RandomState(4)
    bs, n, h, w = 2, 30, 4, 16
    co = random_graph(rng, n, 6)
    coo, dm, _ = oracle.expand_coo(co)
    q, k, v, vb, dvo = (0.5 * rng.standard_normal((bs, n, h, w)).astype(np.float32) for _ in range(5))
    for b in (None, vb):
        vo, attn = cabi.sparse_fwd_host(v, q, k, coo, dm, True, vb=b)
        grads = cabi.sparse_bwd_host(dvo, v, q, k, coo, attn, dm, True, vb=b)
        rvo, rattn, rgrads = run_oracle(v, b, q, k, dvo, coo, dm, True)
        assert_close(vo, rvo, 1e-5)
        assert_close(attn, rattn, 1e-5)
        for x, r in zip(grads, rgrads):
            assert_close(x, r, 1e-5)


def test_host_entry_point_reports_out_of_range_rows():
    """The index build's verdict comes back through the copy-out stream and is reported by the synchronisation."""
    cabi = _cabi()
    rng = np.random.RandomState(6)
    bs, n, h, w = 2, 12, 4, 16
    q, k, v = (rng.standard_normal((bs, n, h, w)).astype(np.float32) for _ in range(3))
    coo = np.array([[0, 1, 0, 0], [40, 1, 0, 0], [1, 1, 0, 1]], dtype=np.int32)  # dst 40 of 12 tokens
    with pytest.raises(cabi.L1AttnError) as e:
        cabi.sparse_fwd_host(v, q, k, coo, 2, True)
    assert e.value.code == -4
    # and the library is usable afterwards
    good = np.array([[0, 1, 0, 0], [1, 1, 0, 1]], dtype=np.int32)
    vo, attn = cabi.sparse_fwd_host(v, q, k, good, 1, True)
    assert np.isfinite(vo).all()


def test_deterministic():
    rng = np.random.RandomState(8)
    from oracle import oracle
    bs, n, h, w = 2, 128, 8, 64
    co = random_graph(rng, n, 24)
    coo, dm, _ = oracle.expand_coo(co)
    q, k, v, vb, dvo = (rng.standard_normal((bs, n, h, w)).astype(np.float32) for _ in range(5))
    a = run_gpu(v, vb, q, k, dvo, coo, dm, True)
    b = run_gpu(v, vb, q, k, dvo, coo, dm, True)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    for x, y in zip(a[2], b[2]):
        assert np.array_equal(x, y)


def bench_graph(n, fan, seed):
    """The sparse benchmark graph: every dst gets its self edge plus `fan` distinct other srcs,
    rows randomly permuted."""
    g = torch.Generator().manual_seed(seed)
    r = torch.rand(n, n, generator=g)
    r.fill_diagonal_(2)
    src = r.argsort(1)[:, :fan]
    rows = torch.cat([torch.stack([torch.arange(n).repeat_interleave(fan), src.reshape(-1)], 1),
                      torch.stack([torch.arange(n), torch.arange(n)], 1)])
    return rows[torch.randperm(rows.shape[0], generator=g)].numpy()


@pytest.mark.parametrize("qk_scale", [1.0, 0.25])
@pytest.mark.parametrize("bidi", [False, True])
def test_full_size_config(bidi, qk_scale):
    """The sparse benchmark config (n_ctx 4096, 8 heads, width 64, 131072 edges): one batch item is
    checked in full against the oracle; the batch-of-8 run must reproduce that item bit for bit
    (batch items are independent) and keep sum_r attn <= 1.  q,k ~ N(0,1) as the config states (logits
    near -9, weights ~1e-4) and 0.25 N(0,1) (weights ~1/32, so the normalisation matters)."""
    from oracle import oracle
    n, h, w = 4096, 8, 64
    co = bench_graph(n, 31, 4001)
    coo, dm, sm = oracle.expand_coo(co)
    assert co.shape[0] == 131072 and dm == 32
    gen = torch.Generator().manual_seed(4100)
    t = [qk_scale * torch.randn((8, n, h, w), generator=gen) for _ in range(2)] + \
        [torch.randn((8, n, h, w), generator=gen) for _ in range(3)]
    q, k, v, vb, dvo = (x.numpy() for x in t)
    vb_ = vb if bidi else None
    vo8, attn8, g8 = run_gpu(v, vb_, q, k, dvo, coo, dm, True)
    one = lambda a: None if a is None else a[:1]
    vo1, attn1, g1 = run_gpu(one(v), one(vb_), one(q), one(k), one(dvo), coo, dm, True)
    assert np.array_equal(vo8[:1], vo1) and np.array_equal(attn8[:1], attn1)
    for x, y in zip(g8, g1):
        assert np.array_equal(x[:1], y)
    assert attn8.sum(2).max() <= 1.0 + 1e-5 and attn8.min() >= 0
    rvo, rattn, rg = run_oracle(one(v), one(vb_), one(q), one(k), one(dvo), coo, dm, True)
    assert_close(vo1, rvo, 1e-5, "vo")
    assert_close(attn1, rattn, 1e-5, "attn")
    for x, r in zip(g1, rg):
        assert_close(x, r, 1e-5, "grad")


# ------------------------------------------------------------------ expandCoo

def test_expandcoo_golden(golden):
    cabi = _cabi()
    g = golden["expandcoo"]
    for name in g["names"]:
        coo, dm, sm = cabi.expand_coo_host(g[name + "_co"])
        assert coo.dtype == np.int32 and np.array_equal(coo, g[name + "_coo"]), name
        assert [dm, sm] == list(g[name + "_mxlen"]), name


def test_expandcoo_bench_graph_bit_exact():
    from oracle import oracle
    cabi = _cabi()
    co = bench_graph(4096, 31, 4001)
    coo, dm, sm = cabi.expand_coo_host(co)
    rcoo, rdm, rsm = oracle.expand_coo(co)
    assert np.array_equal(coo, rcoo) and (dm, sm) == (rdm, rsm)


def test_expandcoo_edge_cases():
    from oracle import oracle
    cabi = _cabi()
    coo, dm, sm = cabi.expand_coo_host(np.zeros((0, 2), dtype=np.int64))
    assert coo.shape == (0, 4) and (dm, sm) == (1, 1)
    rng = np.random.RandomState(1)
    for co in (np.array([[7, 7]]), np.full((1000, 2), 3),               # one row; one hub
               rng.randint(0, 200000, size=(5000, 2)),                   # more keys than fit in shared memory
               rng.randint(-50, 50, size=(777, 2)),                      # negative ids
               rng.randint(0, 33, size=(33, 2))):
        coo, dm, sm = cabi.expand_coo_host(co)
        rcoo, rdm, rsm = oracle.expand_coo(co)
        assert np.array_equal(coo, rcoo) and (dm, sm) == (rdm, rsm)
