"""CPU-side checks of the C ABI: the library loads, exports every function that
include/l1attn_b200.h declares, the ctypes table covers the same set, and argument validation
answers before any CUDA call is made (so these run on a box without a GPU)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

import l1attn_cabi

HEADER = os.path.join(ROOT, "include", "l1attn_b200.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(l1attn_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_expected_surface():
    names = declared_functions()
    for must in ("l1attn_dense_fwd", "l1attn_dense_bwd", "l1attn_sparse_fwd", "l1attn_sparse_bwd",
                 "l1attn_sparse_build_index", "l1attn_expand_coo", "l1attn_dense_fwd_host"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = l1attn_cabi.lib()
    for name in declared_functions():
        assert hasattr(lib, name), "libl1attn_b200.so does not export %s" % name


def test_ctypes_table_matches_header():
    assert sorted(l1attn_cabi.SIGNATURES) == declared_functions()


def test_version_and_strerror():
    lib = l1attn_cabi.lib()
    assert lib.l1attn_version() >= 100
    assert lib.l1attn_strerror(0) == b"ok"
    for code in range(-6, 0):
        assert b"unknown l1attn" not in lib.l1attn_strerror(code)
    assert b"unknown l1attn" in lib.l1attn_strerror(-99)


def test_argument_validation_needs_no_gpu():
    lib = l1attn_cabi.lib()
    buf = (ctypes.c_double * 16)()
    p = ctypes.addressof(buf)
    # negative size, unknown dtype, NULL pointer, misaligned pointer
    assert lib.l1attn_dense_fwd(p, p, p, -1, 1, 1, 1, 0, None) == -1
    assert lib.l1attn_dense_fwd(p, p, p, 1, 1, 1, 1, 7, None) == -1
    assert lib.l1attn_dense_fwd(None, p, p, 1, 1, 1, 1, 0, None) == -1
    assert lib.l1attn_dense_fwd(p + 2, p, p, 1, 1, 1, 1, 0, None) == -6
    assert lib.l1attn_dense_bwd(p, p, p, p, None, None, 1, 1, 1, 1, 1, None) == -1
    assert lib.l1attn_dense_fwd(p, p, p, 1, 1, 1, 0, 0, None) == -1  # width must be >= 1
    assert lib.l1attn_sparse_fwd(p, None, p, p, p, p, p, 1, 1, 1, 0, 1, 1, 1, 1, 0, 0, None) == -1
    assert lib.l1attn_sparse_fwd(p, None, p, p, None, p, p, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0, None) == -1
    assert lib.l1attn_sparse_fwd(p, None, p, p, p, p, p, 1, 1, 1, 1, 1, 1, 1, 1, 1, 0, None) == -1  # bidi without vb
    assert lib.l1attn_sparse_build_index(None, 3, 4, 2, p, None, None) == -1
    assert lib.l1attn_sparse_build_index(p, 1, 1 << 20, 1 << 12, p, None, None) == -2  # slot table > 2^31
    assert lib.l1attn_expand_coo(None, 4, p, p, 0, 10, None, None) == -1
    # fused consumer: unknown mode, zero value width, NULL tensor, 16-bit dtypes (sparse forward only)
    assert lib.l1attn_dense_softmax_v_fwd(p, p, p, p, None, 1, 1, 1, 1, 1, 3, 0, None) == -1
    assert lib.l1attn_dense_softmax_v_fwd(p, p, p, p, None, 1, 1, 1, 1, 0, 0, 0, None) == -1
    assert lib.l1attn_dense_softmax_v_fwd(p, p, None, p, None, 1, 1, 1, 1, 1, 0, 0, None) == -1
    assert lib.l1attn_dense_softmax_v_fwd(p, p, p, p, None, 1, 1, 1, 1, 1, 0, 2, None) == -1
    assert lib.l1attn_dense_softmax_v_bwd_dx(p, p, p, p, p, None, p, p, 1, 1, 1, 1, 1, 0, None) == -1
    assert lib.l1attn_dense_fwd(p, p, p, 1, 1, 1, 1, 2, None) == -1  # float16 is not a dense dtype
    assert lib.l1attn_sparse_bwd(p, p, None, p, p, p, p, p, None, p, p, p, 1, 1, 1, 1, 1, 1, 1, 1, 0, 2, None) == -1
    # empty problems are fine and touch nothing
    assert lib.l1attn_dense_softmax_v_fwd(None, None, None, None, None, 0, 4, 2, 8, 8, 0, 0, None) == 0
    assert lib.l1attn_dense_fwd(None, None, None, 0, 5, 2, 8, 0, None) == 0
    assert lib.l1attn_dense_bwd(None, None, None, None, None, None, 3, 0, 2, 8, 1, None) == 0


def test_size_queries():
    lib = l1attn_cabi.lib()
    assert lib.l1attn_sparse_index_bytes(0, 0, 0) >= 16
    n = lib.l1attn_sparse_index_bytes(131072, 4096, 32)
    assert n >= 4 * (4096 * 32 + 4097 + 131072) and n % 16 == 0
    assert lib.l1attn_sparse_bwd_scratch_bytes(8, 4096, 8, 32, 0) == 8 * 4096 * 8 * 32 * 4
    assert lib.l1attn_sparse_bwd_scratch_bytes(8, 4096, 8, 32, 1) == 8 * 4096 * 8 * 32 * 8
    # tie flags (x per 4 rows, y per 16 rows, per pass and group) | tie header | 4096 tie entries | 8 shares of d_k
    assert lib.l1attn_dense_bwd_scratch_bytes(16, 1024, 16, 64, 0) == 2 * 64 * (256 + 64) + 256 + 4096 * 16 + 8 * 16 * 1024 * 16 * 64 * 4
    # long context, two batch items: 32 shares of d_k, and the source rows split in two -> two partial d_q
    n3 = 2 * 4096 * 8 * 128 * 4
    assert lib.l1attn_dense_bwd_scratch_bytes(2, 4096, 8, 128, 0) == 2 * 8 * (1024 + 256) + 256 + 4096 * 16 + 32 * n3 + 2 * n3
    assert lib.l1attn_dense_bwd_scratch_bytes(16, 1024, 16, 64, 1) == 16  # float64 needs none
    assert lib.l1attn_expand_coo_scratch_bytes(4096) == 0
    assert lib.l1attn_expand_coo_scratch_bytes(1 << 20) == (1 << 20) * 8


def test_no_cpu_fallback_in_product():
    """The shipped package must never import the oracle."""
    pkg = os.path.join(ROOT, "l1-attention_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "build.py", "%s mentions the oracle" % f
