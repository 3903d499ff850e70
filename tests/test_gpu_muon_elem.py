"""GPU: Muon's elementwise kernels against the oracle (bit-exact), the transposed forms
against the plain forms plus a transpose (bit-exact, as tests/kernels/_probe_ns_fused.py:93-120
asks of the reference's fused kernels), and the Frobenius normalisation."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200 import kernels as K
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import bf16 as obf, muon_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(128, 256), (256, 128), (192, 64)])
@pytest.mark.parametrize("grad_dtype", ["bf16", "f32"])
@pytest.mark.parametrize("nesterov", [True, False])
def test_momentum_bit_exact(ctx, shape, grad_dtype, nesterov):
    rng = np.random.default_rng(0)
    Kd, N = shape
    buf = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    g = (rng.standard_normal(shape) * 1e-3).astype(np.float32)
    g_used = obf.rne_f32(g) if grad_dtype == "bf16" else g
    nb, u = muon_ref.momentum(buf, g_used, 0.95)
    want_u = obf.rne_bits(u if nesterov else nb)
    for tr in (False, True):
        dbuf = anc.DBuf(buf, ctx)
        dg = anc.DBuf(f32_to_bf16_bits(g) if grad_dtype == "bf16" else g, ctx)
        du = anc.DBuf.zeros((N, Kd) if tr else (Kd, N), np.uint16, ctx)
        K.muon_momentum(dbuf, dg, du, Kd, N, 0.95, nesterov, tr, grad_dtype, ctx=ctx)
        ctx.sync()
        assert np.array_equal(dbuf.to_numpy(), nb)
        got = du.to_numpy()
        assert np.array_equal(got.T if tr else got, want_u)
        for b in (dbuf, dg, du):
            b.free()


@pytest.mark.parametrize("shape", [(128, 256), (256, 128)])
def test_update_bit_exact(ctx, shape):
    rng = np.random.default_rng(1)
    Kd, N = shape
    p = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    O = obf.rne_bits((rng.standard_normal(shape) * 0.05).astype(np.float32))
    lr_scale = np.float32(0.02 * muon_ref.shape_scale(Kd, N))
    pn, p16 = muon_ref.update(p, O, lr_scale)
    for tr in (False, True):
        dp, dp16 = anc.DBuf(p, ctx), anc.DBuf.zeros(shape, np.uint16, ctx)
        dO = anc.DBuf(np.ascontiguousarray(O.T) if tr else O, ctx)
        K.muon_update(dp, dp16, dO, Kd, N, lr_scale, tr, ctx=ctx)
        ctx.sync()
        assert np.array_equal(dp.to_numpy(), pn)
        assert np.array_equal(dp16.to_numpy(), p16)
        for b in (dp, dp16, dO):
            b.free()


def test_fro_normalize(ctx):
    rng = np.random.default_rng(2)
    E, M, N = 3, 128, 384
    X = obf.rne_bits((rng.standard_normal((E * M, N)) * np.array([1e-3, 1.0, 30.0]).repeat(M)[:, None]).astype(np.float32))
    dX, dr = anc.DBuf(X, ctx), anc.DBuf.zeros((E,), np.float32, ctx)
    K.fro_normalize(dX, dr, E, M, N, 1e-7, ctx=ctx)
    ctx.sync()
    r1, X1 = dr.to_numpy(), dX.to_numpy()
    for e in range(E):
        blk = bits_to_f32(X[e * M:(e + 1) * M])
        want = muon_ref.fro_recip(blk)
        assert abs(r1[e] - want) / want < 1e-5
        # the scale itself is exact given the device's reciprocal
        assert np.array_equal(X1[e * M:(e + 1) * M], obf.rne_bits(blk * r1[e]))
    # fixed-order reduction: a second run, and a run with a different batch around matrix 1,
    # give the same bits
    dX2, dr2 = anc.DBuf(X[M:2 * M], ctx), anc.DBuf.zeros((1,), np.float32, ctx)
    K.fro_normalize(dX2, dr2, 1, M, N, 1e-7, ctx=ctx)
    ctx.sync()
    assert dr2.to_numpy()[0] == r1[1]
    assert np.array_equal(dX2.to_numpy(), X1[M:2 * M])
    for b in (dX, dr, dX2, dr2):
        b.free()
