"""The allocation-free sparse backward (l1attn_sparse_bwd_static).

Some callers cannot allocate device memory where they run the backward -- a plugin that only gets
device pointers from the runtime embedding it, or code in a region where cudaMalloc is forbidden or
would stall the device.  For them the library keeps the backward's d(logit) scratch in a fixed 32 MiB
device array of its own.  This file checks, through the C ABI, that the entry point gives what
l1attn_sparse_bwd gives with caller-provided scratch, on two calls in a row (the second on a
different graph and different tensors, so contents left in the shared array by the first call must
not matter), and that a problem too large for the array is refused before anything is launched.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import numpy as np
import pytest

from conftest import assert_close


def _problem(seed, bs, n, h, w, deg, bidi):
    import torch
    rng = np.random.RandomState(seed)
    rows = []
    for d in range(n):
        srcs = rng.choice(n, size=rng.randint(1, deg + 1), replace=False)
        rows += [[d, s] for s in srcs]
    co = np.array(rows, dtype=np.int64)
    co = co[rng.permutation(co.shape[0])]
    mk = lambda scale=1.0: torch.from_numpy((scale * rng.standard_normal((bs, n, h, w))).astype(np.float32)).cuda()
    return co, dict(q=mk(0.3), k=mk(0.3), v=mk(), vb=mk() if bidi else None, dvo=mk())


@pytest.mark.gpu
def test_static_scratch_backward_matches_regular_entry_point():
    import torch
    import l1attn_cabi as cabi

    lib = cabi.lib()
    assert lib.l1attn_sparse_bwd_static_capacity() == 32 << 20
    for seed, (bs, n, h, w, deg, bidi) in enumerate([(2, 96, 8, 64, 12, False), (3, 50, 4, 32, 7, True)]):
        co, t = _problem(100 + seed, bs, n, h, w, deg, bidi)
        coo_h, dm, _ = cabi.expand_coo_host(co)
        index = cabi.SparseIndex(torch.from_numpy(coo_h).cuda(), n, dm)
        index.check()
        _, attn = cabi.sparse_fwd(t["v"], t["q"], t["k"], index, True, vb=t["vb"])
        want = cabi.sparse_bwd(t["dvo"], t["v"], t["q"], t["k"], index, attn, True, vb=t["vb"])
        # outputs pre-allocated, so the call under test performs no allocation of any kind
        out = (torch.empty_like(t["v"]), torch.empty_like(t["v"]) if bidi else None,
               torch.empty_like(t["q"]), torch.empty_like(t["k"]))
        torch.cuda.synchronize()
        n_alloc = torch.cuda.memory_stats()["allocation.all.allocated"]  # cumulative count of torch allocations
        free_before, _ = torch.cuda.mem_get_info()                         # cudaMemGetInfo: sees the runtime's own allocations too
        got = cabi.sparse_bwd_static(t["dvo"], t["v"], t["q"], t["k"], index, attn, True, vb=t["vb"], out=out)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == n_alloc
        if seed > 0:  # (the very first call on a device may load the kernels' module image, which the driver places in device memory)
            assert free_after == free_before, "device memory in use changed across the call: %d -> %d" % (free_before, free_after)
        assert lib.l1attn_device_status() == 0
        # ... and against the CPU oracle, like the other sparse tests (fp32: 1e-5 norm-wise)
        from oracle import oracle
        f64 = lambda x: None if x is None else x.cpu().double().numpy()
        if bidi:
            ref = oracle.sparse_bidi_bwd(f64(t["dvo"]), f64(t["v"]), f64(t["vb"]), f64(t["q"]), f64(t["k"]), coo_h, f64(attn), dm, True)
        else:
            ref = oracle.sparse_bwd(f64(t["dvo"]), f64(t["v"]), f64(t["q"]), f64(t["k"]), coo_h, f64(attn), dm, True)
        for a, r in zip(got, ref):
            assert_close(a.cpu().numpy(), r, 1e-5, "static-scratch backward vs oracle")
        for a, b in zip(got, want):
            # same kernels, same order of operations: equal to the last bit, and so within the
            # 1e-5 fp32 tolerance of the other sparse tests
            assert_close(a.cpu().numpy(), b.cpu().numpy(), 1e-5, "static-scratch backward")
            assert torch.equal(a, b)


@pytest.mark.gpu
def test_static_scratch_backward_refuses_oversized_problem():
    import l1attn_cabi as cabi

    lib = cabi.lib()
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    # 16 x 8192 x 64 slots x 8 heads x 4 bytes = 256 MiB of scratch > 32 MiB: refused, nothing is launched
    assert lib.l1attn_sparse_bwd_scratch_bytes(16, 8192, 8, 64, 0) > lib.l1attn_sparse_bwd_static_capacity()
    rc = lib.l1attn_sparse_bwd_static(p, p, None, p, p, p, p, p, None, p, p, 16, 8192, 8, 64, 64, 10, 64, 1, 0, 0, None)
    assert rc == -8
    assert b"scratch" in lib.l1attn_strerror(rc)
