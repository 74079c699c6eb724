"""Dense L1Attn forward/backward on the GPU, through the C ABI, against the CPU oracle.

Tolerances (norm-wise, see conftest.rel_err): fp64 1e-12, fp32 1e-5 -- the bars the task states.
"""
import numpy as np
import pytest

from conftest import assert_close

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

TOL = {np.float32: 1e-5, np.float64: 1e-12}

SHAPES = [(1, 1, 1, 1), (1, 16, 8, 64), (2, 5, 3, 7), (1, 9, 2, 33), (2, 17, 5, 16), (1, 33, 9, 65),
          (3, 70, 12, 32), (1, 130, 16, 64), (2, 64, 1, 128), (1, 3, 16, 7), (2, 40, 8, 97), (1, 65, 24, 64),
          (2, 150, 4, 64), (1, 140, 20, 48),   # (head counts that take the forward's four-head work items)
          (1, 300, 4, 32), (1, 600, 4, 32), (1, 1040, 4, 32), (1, 2050, 4, 32)]  # (few work items: the backward splits the source rows in 2, 4, 8 and 8)


def _cabi():
    import l1attn_cabi
    return l1attn_cabi


def _rand(shape, dtype, seed):
    rng = np.random.RandomState(seed)
    bs, n, h, w = shape
    return (rng.standard_normal(shape).astype(dtype), rng.standard_normal(shape).astype(dtype),
            rng.standard_normal((bs, n, n, h)).astype(dtype))


def _dev(a):
    return torch.from_numpy(a).cuda()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("shape", SHAPES)
def test_fwd_bwd_vs_oracle(shape, dtype):
    from oracle import oracle
    cabi = _cabi()
    q, k, g = _rand(shape, dtype, hash(shape) % 1000)
    attn = cabi.dense_fwd(_dev(q), _dev(k)).cpu().numpy()
    dq, dk = (x.cpu().numpy() for x in cabi.dense_bwd(_dev(g), _dev(q), _dev(k)))
    # the oracle runs in fp64 on the same (fp32-representable) inputs
    q64, k64, g64 = q.astype(np.float64), k.astype(np.float64), g.astype(np.float64)
    assert_close(attn, oracle.dense_fwd(q64, k64), TOL[dtype], "attn %s" % (shape,))
    rq, rk = oracle.dense_bwd(g64, q64, k64)
    assert_close(dq, rq, TOL[dtype], "dq %s" % (shape,))
    assert_close(dk, rk, TOL[dtype], "dk %s" % (shape,))


def test_golden_fixtures(golden):
    """Reference outputs (pure-PyTorch and compiled CPU extension) on seeded inputs, incl. the
    tie-heavy and zero-padded cases: sign(0) must be exactly 0."""
    cabi = _cabi()
    g = golden["dense"]
    for name in g["names"]:
        q, k, da = g[name + "_q"], g[name + "_k"], g[name + "_dattn"]
        attn = cabi.dense_fwd(_dev(q), _dev(k)).cpu().numpy()
        dq, dk = (x.cpu().numpy() for x in cabi.dense_bwd(_dev(da), _dev(q), _dev(k)))
        for ref in ("py", "cpp"):
            if "%s_attn_%s" % (name, ref) not in g:
                continue
            assert_close(attn, g["%s_attn_%s" % (name, ref)], 1e-12, "%s attn vs %s" % (name, ref))
            assert_close(dq, g["%s_dq_%s" % (name, ref)], 1e-12, "%s dq vs %s" % (name, ref))
            assert_close(dk, g["%s_dk_%s" % (name, ref)], 1e-12, "%s dk vs %s" % (name, ref))
        # fp32 on the same inputs
        a32 = cabi.dense_fwd(_dev(q.astype(np.float32)), _dev(k.astype(np.float32))).cpu().numpy()
        assert_close(a32, g[name + "_attn_py"], 1e-5, name + " attn fp32")


def test_kat(golden):
    cabi = _cabi()
    g = golden["kat"]
    a = cabi.dense_fwd(_dev(g["f3_q"]), _dev(g["f3_k"])).cpu().numpy()
    expect = np.array([[-1, -1, 0, -.5], [0, -1, -1, -.5], [-1, 0, -1, -.5], [-.5, -.5, -.5, 0]], dtype=np.float32)
    assert np.array_equal(a[0, :, :, 0], expect)
    a1 = cabi.dense_fwd(_dev(g["f1_q"]), _dev(g["f1_k"])).cpu().numpy()
    assert_close(a1, g["f1_dense_attn"], 1e-6, "f1")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_ties_exact(dtype):
    """Inputs on a coarse grid: every difference and every sum is exact in fp32, so the GPU
    result must equal the oracle bit for bit up to the final scale multiply, and rows with
    q == k must contribute exactly nothing."""
    from oracle import oracle
    cabi = _cabi()
    rng = np.random.RandomState(5)
    shape = (2, 48, 8, 64)
    q = (np.round(rng.standard_normal(shape) * 2) / 2).astype(dtype)
    k = (np.round(rng.standard_normal(shape) * 2) / 2).astype(dtype)
    k[:, 40:] = q[:, 40:]  # identical rows
    q[:, 44:] = 0
    k[:, 44:] = 0  # zero padding
    g = np.round(rng.standard_normal((2, 48, 48, 8)) * 4).astype(dtype) / 4
    dq, dk = (x.cpu().numpy() for x in cabi.dense_bwd(_dev(g), _dev(q), _dev(k)))
    rq, rk = oracle.dense_bwd(g.astype(np.float64), q.astype(np.float64), k.astype(np.float64))
    assert_close(dq, rq, 2e-7 if dtype == np.float32 else 1e-14, "dq ties")
    assert_close(dk, rk, 2e-7 if dtype == np.float32 else 1e-14, "dk ties")


@pytest.mark.parametrize("shape", [(2, 200, 8, 64), (1, 1040, 4, 32)])  # (the second: work items split their source rows)
@pytest.mark.parametrize("kind", ["sparse_ties", "padded", "q_is_k", "grid"])
def test_fast_backward_tie_handling(kind, shape):
    """fp32 shapes that take the compare-form backward (16-byte rows): a handful of planted ties, many
    zero-padded tokens (more candidates than the detector lists), q == k, and values on a coarse grid
    (ties everywhere).  The result must match the oracle as if every term had used sign(0) = 0."""
    from oracle import oracle
    cabi = _cabi()
    rng = np.random.RandomState(21)
    bs, n, nh, nw = shape
    q = rng.standard_normal(shape).astype(np.float32)
    k = rng.standard_normal(shape).astype(np.float32)
    if kind == "sparse_ties":
        for _ in range(7):
            b, t, s, h, w = (rng.randint(m) for m in (bs, n, n, nh, nw))
            k[b, s, h, w] = q[b, t, h, w]
        k[bs - 1, 5, 3, 7] = -0.0
        q[bs - 1, 9, 3, 7] = 0.0  # +0 == -0 is a tie too
    elif kind == "padded":
        q[:, n * 3 // 5:] = 0
        k[:, n * 9 // 20:] = 0
    elif kind == "q_is_k":
        k = q.copy()
    else:
        q, k = np.round(q * 2) / 2, np.round(k * 2) / 2
    g = rng.standard_normal((bs, n, n, nh)).astype(np.float32)
    dq, dk = (x.cpu().numpy() for x in cabi.dense_bwd(_dev(g), _dev(q), _dev(k)))
    rq, rk = oracle.dense_bwd(g.astype(np.float64), q.astype(np.float64), k.astype(np.float64))
    assert_close(dq, rq, 1e-5, "dq " + kind)
    assert_close(dk, rk, 1e-5, "dk " + kind)
    # without scratch every tile takes the exact loop: same answer
    dq2, dk2 = (x.cpu().numpy() for x in cabi.dense_bwd(_dev(g), _dev(q), _dev(k), scratch=None))
    assert_close(dq2, rq, 1e-5, "dq exact " + kind)
    assert_close(dk2, rk, 1e-5, "dk exact " + kind)


def test_deterministic():
    cabi = _cabi()
    q, k, g = _rand((2, 96, 16, 64), np.float32, 11)
    a = [cabi.dense_bwd(_dev(g), _dev(q), _dev(k)) for _ in range(2)]
    assert torch.equal(a[0][0], a[1][0]) and torch.equal(a[0][1], a[1][1])
    f = [cabi.dense_fwd(_dev(q), _dev(k)) for _ in range(2)]
    assert torch.equal(f[0], f[1])


def test_host_buffer_entry_points():
    from oracle import oracle
    cabi = _cabi()
    q, k, g = _rand((2, 37, 5, 24), np.float32, 3)
    attn = cabi.dense_fwd_host(q, k)
    dq, dk = cabi.dense_bwd_host(g, q, k)
    q64, k64, g64 = q.astype(np.float64), k.astype(np.float64), g.astype(np.float64)
    assert_close(attn, oracle.dense_fwd(q64, k64), 1e-5, "host attn")
    rq, rk = oracle.dense_bwd(g64, q64, k64)
    assert_close(dq, rq, 1e-5, "host dq")
    assert_close(dk, rk, 1e-5, "host dk")
    # asynchronous forms: forward and an independent backward enqueued together, several times over (the arena
    # has to grow and to be reused), results valid after the sync and equal to the synchronous ones
    for rep in range(3):
        attn2 = np.empty_like(attn)
        dq2, dk2 = np.empty_like(dq), np.empty_like(dk)
        cabi.dense_fwd_host(q, k, out=attn2, wait=False)
        cabi.dense_bwd_host(g, q, k, out=(dq2, dk2), wait=False)
        cabi.host_sync()
        assert np.array_equal(attn2, attn) and np.array_equal(dq2, dq) and np.array_equal(dk2, dk)
    assert cabi.lib().l1attn_host_release() == 0


def test_fp64_long_context_variant_full():
    """The float64 long-context variant [2,512,8,128], checked in full against the oracle at 1e-12."""
    from oracle import oracle
    cabi = _cabi()
    rng = np.random.RandomState(3001)
    shape = (2, 512, 8, 128)
    q, k = rng.standard_normal(shape), rng.standard_normal(shape)
    g = rng.standard_normal((2, 512, 512, 8))
    attn = cabi.dense_fwd(_dev(q), _dev(k)).cpu().numpy()
    dq, dk = (x.cpu().numpy() for x in cabi.dense_bwd(_dev(g), _dev(q), _dev(k)))
    assert_close(attn, oracle.dense_fwd(q, k), 1e-12, "attn")
    rq, rk = oracle.dense_bwd(g, q, k)
    assert_close(dq, rq, 1e-12, "dq")
    assert_close(dk, rk, 1e-12, "dk")


@pytest.mark.parametrize("shape", [(16, 1024, 16, 64), (2, 4096, 8, 128)])
def test_full_size_properties(shape):
    """The fp32 benchmark shapes [16,1024,16,64] and [2,4096,8,128], too large for the oracle: size-independent properties.
      * swapping q and k transposes the score matrix exactly (|q-k| is symmetric);
      * sampled (b, s, t) entries and sampled gradient rows match a float64 numpy evaluation;
      * the backward is linear in d_attn."""
    cabi = _cabi()
    bs, n, h, w = shape
    gen = torch.Generator(device="cuda").manual_seed(2000)
    q = torch.randn(shape, generator=gen, device="cuda")
    k = torch.randn(shape, generator=gen, device="cuda")
    attn = cabi.dense_fwd(q, k)
    attn_sw = cabi.dense_fwd(k, q)
    assert torch.equal(attn, attn_sw.transpose(1, 2))
    del attn_sw
    scale = -1.0 / np.sqrt(w)
    rng = np.random.RandomState(7)
    qh, kh = q.double().cpu().numpy(), k.double().cpu().numpy()
    for _ in range(64):
        b, s, t = rng.randint(bs), rng.randint(n), rng.randint(n)
        ref = scale * np.abs(qh[b, t] - kh[b, s]).sum(-1)
        assert_close(attn[b, s, t].cpu().numpy(), ref, 1e-5, "sample attn")
    g1 = torch.randn(attn.shape, generator=gen, device="cuda")
    dq1, dk1 = cabi.dense_bwd(g1, q, k)
    for _ in range(8):
        b, t = rng.randint(bs), rng.randint(n)
        sg = np.sign(qh[b, t][None] - kh[b])  # [s, h, w]
        ref = scale * (sg * g1[b, :, t].double().cpu().numpy()[:, :, None]).sum(0)
        assert_close(dq1[b, t].cpu().numpy(), ref, 1e-5, "sample dq")
        s = rng.randint(n)
        sg = np.sign(qh[b] - kh[b, s][None])  # [t, h, w]
        ref = -scale * (sg * g1[b, s].double().cpu().numpy()[:, :, None]).sum(0)
        assert_close(dk1[b, s].cpu().numpy(), ref, 1e-5, "sample dk")
    g2 = torch.randn(attn.shape, generator=gen, device="cuda")
    dq2, dk2 = cabi.dense_bwd(g2, q, k)
    g1.add_(g2)
    del g2
    dq3, dk3 = cabi.dense_bwd(g1, q, k)
    assert_close((dq1 + dq2).cpu().numpy(), dq3.cpu().numpy(), 1e-5, "linearity dq")
    assert_close((dk1 + dk2).cpu().numpy(), dk3.cpu().numpy(), 1e-5, "linearity dk")


def _offset_by_one(t):
    """A contiguous copy of t whose storage starts one element (4 bytes) past a 16-byte boundary."""
    buf = torch.empty(t.numel() + 1, dtype=t.dtype, device=t.device)
    view = buf[1:].view(t.shape)
    view.copy_(t)
    assert view.is_contiguous() and view.data_ptr() % 16 == 4
    return view


def test_pointers_aligned_to_the_element_only():
    """The C ABI promises element alignment, not 16 bytes: tensors that start 4 bytes past a 16-byte
    boundary (a contiguous view with storage offset 1) must take the kernels without vector loads or
    tensor maps and give the aligned call's results -- dense forward/backward (with and without tie
    scratch), the fused consumer and the sparse operators."""
    import l1attn_fused_cuda
    cabi = _cabi()
    q, k, g = (torch.from_numpy(a).cuda() for a in _rand((2, 72, 8, 64), np.float32, 31))
    k[1, 7, 3, 5] = q[1, 9, 3, 5]  # one planted tie
    want_attn = cabi.dense_fwd(q, k)
    want = cabi.dense_bwd(g, q, k)
    qo, ko, go = _offset_by_one(q), _offset_by_one(k), _offset_by_one(g)
    out = _offset_by_one(torch.empty_like(want_attn))
    assert_close(cabi.dense_fwd(qo, ko, out=out).cpu().numpy(), want_attn.cpu().numpy(), 1e-6, "attn")
    for scratch in ("auto", None):
        outs = (_offset_by_one(torch.empty_like(q)), _offset_by_one(torch.empty_like(k)))
        got = cabi.dense_bwd(go, qo, ko, out=outs, scratch=scratch)
        for a, b in zip(got, want):
            assert_close(a.cpu().numpy(), b.cpu().numpy(), 1e-6, "gradients")
    # mixed: only q misaligned (the tie detector and the tensor-map path must both decline)
    got = cabi.dense_bwd(g, qo, k)
    for a, b in zip(got, want):
        assert_close(a.cpu().numpy(), b.cpu().numpy(), 1e-6, "gradients, q offset only")
    v = torch.randn(2, 72, 8, 64, device="cuda")
    want_vo = cabi.dense_softmax_v_fwd(0.3 * q, 0.3 * k, v)
    got_vo = cabi.dense_softmax_v_fwd(_offset_by_one(0.3 * q), _offset_by_one(0.3 * k), _offset_by_one(v),
                                      out=_offset_by_one(torch.empty_like(v)))
    assert_close(got_vo.cpu().numpy(), want_vo.cpu().numpy(), 1e-6, "fused vo")
    # sparse, through the C ABI with every float tensor offset
    from oracle import oracle
    rng = np.random.RandomState(4)
    co = np.stack([rng.randint(0, 72, 500), rng.randint(0, 72, 500)], 1)
    coo, dm, _ = oracle.expand_coo(co)
    ix = cabi.SparseIndex(torch.from_numpy(coo).cuda(), 72, dm)
    ix.check()
    qs, ks = 0.3 * q, 0.3 * k
    vo, attn = cabi.sparse_fwd(v, qs, ks, ix, True)
    grads = cabi.sparse_bwd(g[:, :, :64].contiguous().view(2, 72, 8, 64), v, qs, ks, ix, attn, True)
    dvo_o = _offset_by_one(g[:, :, :64].contiguous().view(2, 72, 8, 64))
    vo2, attn2 = cabi.sparse_fwd(_offset_by_one(v), _offset_by_one(qs), _offset_by_one(ks), ix, True,
                                 out=(_offset_by_one(torch.empty_like(vo)), _offset_by_one(torch.empty_like(attn))))
    assert_close(vo2.cpu().numpy(), vo.cpu().numpy(), 1e-6, "sparse vo")
    outs = (_offset_by_one(torch.empty_like(v)), None, _offset_by_one(torch.empty_like(q)), _offset_by_one(torch.empty_like(k)))
    grads2 = cabi.sparse_bwd(dvo_o, _offset_by_one(v), _offset_by_one(qs), _offset_by_one(ks), ix, attn2, True,
                             out=outs, scratch=_offset_by_one(torch.empty_like(attn)))
    for a, b in zip(grads2, grads):
        assert_close(a.cpu().numpy(), b.cpu().numpy(), 1e-6, "sparse gradients")
    torch.cuda.synchronize()
    assert cabi.lib().l1attn_device_status() == 0


def test_bounded_wait_gives_up_and_is_reported():
    """Every wait of the TMA kernels is bounded in time.  Here one warp waits (limit 3 ms) on a barrier that nothing
    completes: the wait gives up, the kernel returns, l1attn_device_status() reports the timeout exactly once, and
    the library keeps working.  Nothing faults and nothing hangs -- a wait that runs out is the whole test."""
    import time
    cabi = _cabi()
    lib = cabi.lib()
    torch.cuda.synchronize()
    assert lib.l1attn_device_status() == 0
    returned = torch.zeros(2, dtype=torch.int32, device="cuda")
    pinned = torch.zeros(16, dtype=torch.int32).pin_memory()
    t0 = time.time()
    assert lib.l1attn_test_wait_timeout(3000, returned.data_ptr(), None) == 0
    assert lib.l1attn_device_status_async(pinned.data_ptr(), None) == 0  # the no-sync way to learn of it
    torch.cuda.synchronize()
    assert time.time() - t0 < 30.0
    assert int(returned[0]) == 1, "the kernel must come back from the wait with `false`"
    assert int(pinned[0]) == 1
    # duration of one failed poll: the hot loops poll 2^18 times before they look at the clock, which must stay
    # in the range of a second
    ns_per_poll = 3e6 / max(1, int(returned[1]))
    print("failed mbarrier.try_wait poll: %.0f ns" % ns_per_poll)
    assert ns_per_poll < 20000
    assert lib.l1attn_device_status() == -7 and b"bounded wait" in lib.l1attn_strerror(-7)
    assert lib.l1attn_device_status() == 0  # cleared by the read
    assert lib.l1attn_test_wait_timeout(0, returned.data_ptr(), None) == -1  # limits outside 1 us .. 100 ms are refused
    q, k, g = (torch.from_numpy(a).cuda() for a in _rand((1, 64, 8, 64), np.float32, 2))
    a1 = cabi.dense_fwd(q, k)
    torch.cuda.synchronize()
    assert lib.l1attn_device_status() == 0 and torch.isfinite(a1).all()


def test_driver_raises_on_a_pending_timeout():
    """The pybind driver never synchronises; it polls the error word through pinned memory and raises at the next
    call after a kernel gave up a wait."""
    import l1attn_cuda_drv
    cabi = _cabi()
    lib = cabi.lib()
    q = torch.randn(1, 32, 8, 64, device="cuda")
    l1attn_cuda_drv.forward(q, q)
    torch.cuda.synchronize()
    l1attn_cuda_drv.forward(q, q)  # nothing pending: fine
    returned = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert lib.l1attn_test_wait_timeout(2000, returned.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    l1attn_cuda_drv.forward(q, q)  # enqueued behind the probe; copies the (now set) word to the pinned word
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        l1attn_cuda_drv.forward(q, q)
    assert lib.l1attn_device_status() == 0  # the raise cleared it
    out = l1attn_cuda_drv.forward(q, q)[0]
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
