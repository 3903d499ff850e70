"""GPU: the allocation-free Frobenius normalisation (anc_fro_normalize_static) against the
regular entry point (anc_fro_normalize), through the C ABI.

Some callers cannot enter the CUDA allocator when they call into this library: their device
memory belongs to a framework's caching pool, or the call sits in a step that must stay free
of the synchronisation cudaMalloc brings.  For them the library keeps the reduction scratch
in a fixed array inside its own device image.  Both entry points launch the same kernels in
the same order, so their outputs must agree bit for bit.  The check runs on two calls in a row
with different shapes, because the built-in scratch is shared and keeps the previous call's
contents.  The file name sorts last so that a `pytest -x` run has already executed every
other test when it gets here; the test also passes when run alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

from ancora_cutile_b200 import _lib as L

pytestmark = pytest.mark.gpu


def _bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _dev_copy(lib, ctx, host):
    p = C.c_void_p()
    L.check(lib.anc_malloc(ctx, host.nbytes, C.byref(p)))
    L.check(lib.anc_h2d(ctx, p, host.ctypes.data, host.nbytes, None, 1))
    return p


def _read(lib, ctx, dptr, shape, dtype):
    out = np.empty(shape, dtype)
    L.check(lib.anc_d2h(ctx, out.ctypes.data, dptr, out.nbytes, None, 1))
    return out


def test_static_scratch_matches_regular_entry_point_twice():
    lib = L.lib()
    ctx = C.c_void_p()
    L.check(lib.anc_ctx_create(0, None, C.byref(ctx)))     # only for the test's own buffers
    stream = C.c_void_p()
    L.check(lib.anc_ctx_stream(ctx, C.byref(stream)))
    rng = np.random.default_rng(11)
    try:
        # second call is smaller than the first: stale partial sums stay behind in the array
        for (E, M, N, scale) in [(5, 256, 384, 1e-3), (2, 128, 128, 7.0)]:
            X = _bf16_bits(rng.standard_normal((E * M, N)) * scale)
            eps = 1e-7
            dX0, dX1 = _dev_copy(lib, ctx, X), _dev_copy(lib, ctx, X)
            r0 = _dev_copy(lib, ctx, np.zeros(E, np.float32))
            r1 = _dev_copy(lib, ctx, np.full(E, -1.0, np.float32))
            L.check(lib.anc_fro_normalize(ctx, dX0, r0, E, M, N, eps, stream))
            L.check(lib.anc_fro_normalize_static(0, dX1, r1, E, M, N, eps, stream))
            L.check(lib.anc_ctx_sync(ctx, stream))
            a, b = _read(lib, ctx, dX0, X.shape, np.uint16), _read(lib, ctx, dX1, X.shape, np.uint16)
            ra, rb = _read(lib, ctx, r0, (E,), np.float32), _read(lib, ctx, r1, (E,), np.float32)
            assert np.array_equal(ra.view(np.uint32), rb.view(np.uint32))      # tolerance: exact
            assert np.array_equal(a, b)
            assert not np.array_equal(b, X)                                    # it did run
            for p in (dX0, dX1, r0, r1):
                L.check(lib.anc_free(ctx, p))
    finally:
        lib.anc_ctx_destroy(ctx)


def test_static_scratch_rejects_oversize_and_bad_shapes():
    lib = L.lib()
    dummy = C.c_void_p(256)        # never dereferenced: validation comes first
    # 65537 blocks of 16384 elements: one more than the built-in scratch holds
    rc = lib.anc_fro_normalize_static(0, dummy, dummy, 65537, 128, 128, 1e-7, None)
    assert rc == L.E_INVALID
    assert b"built-in scratch" in lib.anc_last_error()
    assert lib.anc_fro_normalize_static(0, dummy, dummy, 1, 100, 100, 1e-7, None) == L.E_INVALID
    assert lib.anc_fro_normalize_static(0, None, dummy, 1, 128, 128, 1e-7, None) == L.E_INVALID
