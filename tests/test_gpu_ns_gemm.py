"""GPU: the tcgen05 GEMM phases of the Newton-Schulz chain against float64 matmuls of the
same bf16 inputs.  Tolerance: the fp32-accumulated result rounded to bf16 may differ from
the float64 result rounded to bf16 by one bf16 ulp where the exact value sits near a rounding
boundary, so the check is |got - want| <= 2^-7 * |want| + tiny (one ulp), per element, as the
reference validates per 128x128 tile at rel 2e-2 (tests/kernels/_probe_ns_fused.py:36-44).
Symmetry of modes 0/1 (mirrored store), run-to-run and batch-composition bit equality are
exact (tests/kernels/_probe_ns_tri3.py:84-97; tests/training/test_batched_proj_muon.py:74)."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200 import kernels as K
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits

pytestmark = pytest.mark.gpu


def _close(got_bits, want64):
    got = bits_to_f32(got_bits).astype(np.float64)
    tol = np.abs(want64) * 2.0 ** -7 + 1e-30 + np.abs(want64).max() * 2.0 ** -20
    bad = np.abs(got - want64) > tol
    return int(bad.sum()), float(np.abs(got - want64).max() / (np.abs(want64).max() + 1e-30))


def _mk(rng, rows, cols, scale=1.0):
    return f32_to_bf16_bits((rng.standard_normal((rows, cols)) * scale).astype(np.float32))


@pytest.mark.parametrize("E,M,N", [(1, 128, 128), (1, 256, 512), (2, 384, 640), (3, 512, 1024)])
def test_gram_phase(ctx, E, M, N):
    rng = np.random.default_rng(0)
    P = _mk(rng, E * M, N)
    dP, dC = anc.DBuf(P, ctx), anc.DBuf(np.full((E * M, M), 0x7FC0, np.uint16), ctx)
    K.ns_gemm_phase(0, dP, None, dC, E, M, N, ctx=ctx)
    ctx.sync()
    assert ctx.status() == 0
    C = dC.to_numpy()
    for e in range(E):
        x = bits_to_f32(P[e * M:(e + 1) * M]).astype(np.float64)
        nbad, rel = _close(C[e * M:(e + 1) * M], x @ x.T)
        assert nbad == 0, (e, nbad, rel)
        assert np.array_equal(C[e * M:(e + 1) * M], C[e * M:(e + 1) * M].T)   # exact symmetry
    dP.free(); dC.free()


@pytest.mark.parametrize("E,M", [(1, 128), (2, 256), (2, 640)])
def test_poly_phase(ctx, E, M):
    rng = np.random.default_rng(1)
    S = []
    for e in range(E):
        a = (rng.standard_normal((M, M)) * 0.05).astype(np.float32)
        S.append(f32_to_bf16_bits(np.tril(a) + np.tril(a, -1).T))
    P = np.concatenate(S, 0)
    b, c = -6.8946, 2.9270
    dP, dC = anc.DBuf(P, ctx), anc.DBuf(np.full((E * M, M), 0x7FC0, np.uint16), ctx)
    K.ns_gemm_phase(1, dP, None, dC, E, M, M, b, c, ctx=ctx)
    ctx.sync()
    assert ctx.status() == 0
    C = dC.to_numpy()
    for e in range(E):
        a = bits_to_f32(P[e * M:(e + 1) * M]).astype(np.float64)
        want = np.float64(np.float32(b)) * a + np.float64(np.float32(c)) * (a @ a)
        nbad, rel = _close(C[e * M:(e + 1) * M], want)
        assert nbad == 0, (e, nbad, rel)
        assert np.array_equal(C[e * M:(e + 1) * M], C[e * M:(e + 1) * M].T)
    dP.free(); dC.free()


@pytest.mark.parametrize("E,M,N", [(1, 128, 128), (1, 128, 384), (2, 256, 768), (2, 384, 1024)])
def test_apply_phase(ctx, E, M, N):
    rng = np.random.default_rng(2)
    P = _mk(rng, E * M, M, 0.05)
    Q = _mk(rng, E * M, N)
    a = 4.0848
    dP, dQ = anc.DBuf(P, ctx), anc.DBuf(Q, ctx)
    dC = anc.DBuf(np.full((E * M, N), 0x7FC0, np.uint16), ctx)
    K.ns_gemm_phase(2, dP, dQ, dC, E, M, N, a, 1.0, ctx=ctx)
    ctx.sync()
    assert ctx.status() == 0
    C = dC.to_numpy()
    for e in range(E):
        p = bits_to_f32(P[e * M:(e + 1) * M]).astype(np.float64)
        q = bits_to_f32(Q[e * M:(e + 1) * M]).astype(np.float64)
        nbad, rel = _close(C[e * M:(e + 1) * M], np.float64(np.float32(a)) * q + p @ q)
        assert nbad == 0, (e, nbad, rel)
    for x in (dP, dQ, dC):
        x.free()


def test_bits_independent_of_batch_and_run(ctx):
    rng = np.random.default_rng(3)
    M, N, E = 256, 512, 5
    P = _mk(rng, E * M, N)
    outs = []
    for rep in range(2):
        dP, dC = anc.DBuf(P, ctx), anc.DBuf.zeros((E * M, M), np.uint16, ctx)
        K.ns_gemm_phase(0, dP, None, dC, E, M, N, ctx=ctx)
        ctx.sync()
        outs.append(dC.to_numpy())
        dP.free(); dC.free()
    assert np.array_equal(outs[0], outs[1])
    e = 3
    dP, dC = anc.DBuf(P[e * M:(e + 1) * M], ctx), anc.DBuf.zeros((M, M), np.uint16, ctx)
    K.ns_gemm_phase(0, dP, None, dC, 1, M, N, ctx=ctx)
    ctx.sync()
    assert np.array_equal(dC.to_numpy(), outs[0][e * M:(e + 1) * M])
    dP.free(); dC.free()
