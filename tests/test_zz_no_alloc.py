"""sage_gemm_noalloc — the GEMM entry point for callers that are not allowed to allocate device
memory (their HBM is owned by another runtime, or they cannot afford cudaMalloc's device-wide
synchronisation).  Its operand-split scratch is a fixed array inside the library instead of
allocator memory, so it must (a) give the same result as sage_gemm, call after call, although all
calls share that one array, (b) not touch the context's allocator, and (c) refuse problems whose
split does not fit.  This file sorts last so that a run stopping at the first failure has already
been through every other test.
"""
import ctypes

import numpy as np
import pytest

import sage_b200 as S

pytestmark = pytest.mark.gpu
L = ctypes.c_int64


def gemm(ctx, fn, ta, tb, m, n, k, a, b):
    A, B, C = ctx.tensor(a), ctx.tensor(b), ctx.empty((m, n))
    st = fn(ctx.h, ta, tb, L(m), L(n), L(k), A.buf, L(0), L(a.shape[1]), B.buf, L(0), L(b.shape[1]), C.buf, L(0), L(n))
    ctx._ck(st)
    out = C.numpy()
    for t in (A, B, C):
        t.release()
    return out


def test_noalloc_gemm_matches_regular_entry_point_twice_in_a_row():
    ctx = S.Context(0)
    rng = np.random.default_rng(77)
    try:
        # two different problems back to back: the second call finds the first call's split in the scratch
        cases = [(0, 0, 256, 192, 160), (1, 1, 200, 136, 72), (0, 1, 129, 257, 63), (0, 0, 256, 192, 160)]
        for ta, tb, m, n, k in cases:
            a = rng.uniform(-1, 1, (k, m) if ta else (m, k)).astype(np.float32)
            b = rng.uniform(-1, 1, (n, k) if tb else (k, n)).astype(np.float32)
            ref = gemm(ctx, S.lib.sage_gemm, ta, tb, m, n, k, a, b)
            before = ctx.mem_stats()
            A, B, C = ctx.tensor(a), ctx.tensor(b), ctx.empty((m, n))
            held = ctx.mem_stats()
            for _ in range(2):
                ctx._ck(S.lib.sage_gemm_noalloc(ctx.h, ta, tb, L(m), L(n), L(k), A.buf, L(0), L(a.shape[1]), B.buf, L(0), L(b.shape[1]),
                                                C.buf, L(0), L(n)))
                got = C.numpy()
                # same kernels, same split arithmetic: the results are identical, not merely close
                assert np.array_equal(got, ref)
            after = ctx.mem_stats()
            assert after["mem_used"] == held["mem_used"] and after["num_device_allocs"] == held["num_device_allocs"]
            for t in (A, B, C):
                t.release()
            assert ctx.mem_stats()["mem_used"] == before["mem_used"]
        assert ctx.status_word() == 0
    finally:
        ctx.close()


def test_noalloc_gemm_with_a_long_k_stays_off_the_allocator():
    """sage_gemm cuts a long K with few output tiles into slices whose partial products live in allocator
    memory.  The no-allocation entry point must not: one pass over K, nothing taken from the pool (which is
    empty here, so any request would reach cudaMalloc and show in num_device_allocs)."""
    ctx = S.Context(0)
    rng = np.random.default_rng(78)
    try:
        for ta, tb, m, n, k in [(0, 0, 576, 64, 6272), (0, 0, 128, 512, 4608), (0, 0, 512, 512, 2048), (0, 0, 64, 64, 8192)]:
            a = rng.uniform(-1, 1, (k, m) if ta else (m, k)).astype(np.float32)
            b = rng.uniform(-1, 1, (n, k) if tb else (k, n)).astype(np.float32)
            A, B, C = ctx.tensor(a), ctx.tensor(b), ctx.empty((m, n))
            ctx._ck(S.lib.sage_release_cached(ctx.h))  # leave nothing in the pool that a hidden request could be served from
            held = ctx.mem_stats()
            outs = []
            for _ in range(2):
                ctx._ck(S.lib.sage_gemm_noalloc(ctx.h, ta, tb, L(m), L(n), L(k), A.buf, L(0), L(a.shape[1]), B.buf, L(0), L(b.shape[1]),
                                                C.buf, L(0), L(n)))
                outs.append(C.numpy())
            after = ctx.mem_stats()
            for key in ("mem_total", "mem_used", "mem_peak", "num_device_allocs"):
                assert after[key] == held[key], (key, m, n, k)
            assert np.array_equal(outs[0], outs[1])
            for t in (A, B, C):
                t.release()
            # sage_gemm splits K for these shapes, so the sums differ in order: compare within the contraction tolerance
            ref = gemm(ctx, S.lib.sage_gemm, ta, tb, m, n, k, a, b)
            exact = a.astype(np.float64) @ b.astype(np.float64)
            scale = np.maximum(np.abs(exact), np.sqrt(np.mean(exact * exact)))
            assert np.max(np.abs(outs[0] - ref) / scale) <= 1e-4
            assert np.max(np.abs(outs[0] - exact) / scale) <= 1e-5
        assert ctx.status_word() == 0
    finally:
        ctx.close()


def test_noalloc_gemm_rejects_what_does_not_fit():
    ctx = S.Context(0)
    try:
        m = n = k = 2048  # split needs 2 * 2 * 4 MiB * 4 B = 64 MiB > 32 MiB
        A, B, C = ctx.empty((m, k)), ctx.empty((k, n)), ctx.empty((m, n))
        st = S.lib.sage_gemm_noalloc(ctx.h, 0, 0, L(m), L(n), L(k), A.buf, L(0), L(k), B.buf, L(0), L(n), C.buf, L(0), L(n))
        assert st == 1 and b"scratch" in S.lib.sage_last_error(ctx.h)
        st = S.lib.sage_gemm_noalloc(ctx.h, 0, 0, L(8), L(8), L(8), A.buf, L(0), L(8), B.buf, L(0), L(8), C.buf, L(0), L(8))
        assert st == 7  # too small for the tensor-core path: SAGE_ERR_UNSUPPORTED, use sage_gemm
        for t in (A, B, C):
            t.release()
    finally:
        ctx.close()
