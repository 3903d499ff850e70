"""GPU: the whole Newton-Schulz chain against the fp32 host chain.

Tolerances are the reference's own (tests/kernels/_probe_polar_express_device.py:72-78):
cos > 0.999 and relative Frobenius error < 0.02 vs the fp32 chain on the same bf16-rounded
input, for Keller and Polar-Express coefficients; batched matrices each against their own
host result at cos > 0.99, rel < 0.05 (same file :86-105, the cross-matrix leak detector).
Bitwise run-to-run and batch-composition equality is this build's own gate."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200 import muon_ns
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import muon_ref

pytestmark = pytest.mark.gpu


def cos_rel(a, b):
    a, b = a.ravel().astype(np.float64), b.ravel().astype(np.float64)
    return (float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30)),
            float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30)))


def ortho_err(Y):
    M = Y.shape[0]
    return float(np.linalg.norm(Y @ Y.T - np.eye(M, dtype=Y.dtype)) / np.sqrt(M))


def dev_ns(ctx, Xbits, E, M, N, steps, schedule):
    Z = lambda *s: anc.DBuf.zeros(s, np.uint16, ctx)
    gX = anc.DBuf(Xbits, ctx)
    gA, gA2, gB, gBX = Z(E * M, M), Z(1, 8), Z(E * M, M), Z(E * M, N)
    grecip = anc.DBuf.zeros((E, 1), np.float32, ctx)
    if E == 1:
        muon_ns.newton_schulz_resident(gX, gA, gA2, gB, gBX, grecip, M, N, ctx.stream, steps=steps, schedule=schedule)
    else:
        muon_ns.newton_schulz_resident_e(gX, gA, gA2, gB, gBX, grecip, E, M, N, ctx.stream, steps=steps,
                                         schedule=schedule)
    ctx.sync()
    assert ctx.status() == 0
    out = gX.to_numpy()
    for g in (gX, gA, gA2, gB, gBX, grecip):
        g.free()
    return out


@pytest.mark.parametrize("M,N", [(512, 512), (512, 1024), (1024, 2048)])
def test_single_matrix_keller_and_pe(ctx, M, N):
    rng = np.random.default_rng(1)
    W = (rng.standard_normal((M, N)) @ np.diag(rng.uniform(0.1, 3.0, N))).astype(np.float32)
    Xb = f32_to_bf16_bits(W)
    Xin = bits_to_f32(Xb)
    d_k5 = bits_to_f32(dev_ns(ctx, Xb, 1, M, N, 5, None))
    d_pe5 = bits_to_f32(dev_ns(ctx, Xb, 1, M, N, 5, muon_ns.PE_SCHEDULE))
    h_k5 = muon_ref.ns_fp32(Xin, 5, None)
    h_pe5 = muon_ref.ns_fp32(Xin, 5, muon_ref.PE_SCHEDULE)
    c, r = cos_rel(d_k5, h_k5)
    assert c > 0.999 and r < 0.02, ("keller", c, r)
    c, r = cos_rel(d_pe5, h_pe5)
    assert c > 0.999 and r < 0.02, ("pe", c, r)
    assert ortho_err(d_pe5) < ortho_err(d_k5)


def test_config2_momentum_matrix(ctx):
    """3072x1024 bf16 momentum ~ N(0,1e-3): runs as (1024,3072) after the transpose."""
    rng = np.random.default_rng(0)
    U = f32_to_bf16_bits((rng.standard_normal((3072, 1024)) * 1e-3).astype(np.float32))
    Xb = np.ascontiguousarray(U.T)
    got = bits_to_f32(dev_ns(ctx, Xb, 1, 1024, 3072, 5, muon_ns.PE_SCHEDULE))
    want = muon_ref.ns_fp32(bits_to_f32(U), 5, muon_ref.PE_SCHEDULE).T
    c, r = cos_rel(got, want)
    assert c > 0.999 and r < 0.02, (c, r)


def test_default_schedule_toggle(ctx):
    rng = np.random.default_rng(5)
    Xb = f32_to_bf16_bits(rng.standard_normal((256, 256)).astype(np.float32))
    Z = lambda *s: anc.DBuf.zeros(s, np.uint16, ctx)

    def run(**kw):
        gX, gA, gB, gBX, gr = anc.DBuf(Xb, ctx), Z(256, 256), Z(256, 256), Z(256, 256), anc.DBuf.zeros((1, 1), np.float32, ctx)
        muon_ns.newton_schulz_resident(gX, gA, None, gB, gBX, gr, 256, 256, ctx.stream, **kw)
        ctx.sync()
        o = gX.to_numpy()
        for g in (gX, gA, gB, gBX, gr):
            g.free()
        return o
    keller = run(schedule=None)
    assert np.array_equal(run(), keller)                  # default is Keller
    prev = anc.set_polar_express(True)
    try:
        assert prev is None
        assert np.array_equal(run(), run(schedule=muon_ns.PE_SCHEDULE))
        assert not np.array_equal(run(), keller)
        assert np.array_equal(run(schedule=None), keller)  # explicit None still means Keller
    finally:
        anc.set_polar_express(False)


def test_batched_each_matrix_vs_own_host_result(ctx):
    rng = np.random.default_rng(2)
    E, M, N = 4, 256, 384
    Ws = [f32_to_bf16_bits((rng.standard_normal((M, N)) @ np.diag(rng.uniform(0.1, 3.0, N))).astype(np.float32))
          for _ in range(E)]
    packed = np.concatenate(Ws, 0)
    out = dev_ns(ctx, packed, E, M, N, 5, muon_ns.PE_SCHEDULE)
    for e in range(E):
        c, r = cos_rel(bits_to_f32(out[e * M:(e + 1) * M]), muon_ref.ns_fp32(bits_to_f32(Ws[e]), 5, muon_ref.PE_SCHEDULE))
        assert c > 0.99 and r < 0.05, (e, c, r)
    # bitwise: run-to-run, and each matrix alone equals its slice of the batch
    assert np.array_equal(dev_ns(ctx, packed, E, M, N, 5, muon_ns.PE_SCHEDULE), out)
    for e in (0, 3):
        assert np.array_equal(dev_ns(ctx, Ws[e], 1, M, N, 5, muon_ns.PE_SCHEDULE), out[e * M:(e + 1) * M])


def test_odd_step_count_lands_in_x(ctx):
    rng = np.random.default_rng(3)
    Xb = f32_to_bf16_bits(rng.standard_normal((128, 256)).astype(np.float32))
    for steps in (1, 3, 4):
        got = bits_to_f32(dev_ns(ctx, Xb, 1, 128, 256, steps, muon_ns.PE_SCHEDULE))
        c, r = cos_rel(got, muon_ref.ns_fp32(bits_to_f32(Xb), steps, muon_ref.PE_SCHEDULE))
        assert c > 0.999 and r < 0.02, (steps, c, r)


def test_group_1024x1024_pe5_and_batch_of_seven(ctx):
    """The (1024,1024) shape group (k/v projections): Polar-Express x5 against the fp32 chain at
    the reference's bar (tests/kernels/_probe_polar_express_device.py:72-78), and a batch of 7
    (one rank's share at 8 GPUs) bitwise equal to each matrix run alone."""
    rng = np.random.default_rng(7)
    E, M, N = 7, 1024, 1024
    Ws = [f32_to_bf16_bits((rng.standard_normal((M, N)) * 1e-3).astype(np.float32)) for _ in range(E)]
    out = dev_ns(ctx, np.concatenate(Ws, 0), E, M, N, 5, muon_ns.PE_SCHEDULE)
    for e in (0, 6):
        c, r = cos_rel(bits_to_f32(out[e * M:(e + 1) * M]), muon_ref.ns_fp32(bits_to_f32(Ws[e]), 5, muon_ref.PE_SCHEDULE))
        assert c > 0.999 and r < 0.02, (e, c, r)
    for e in (0, 3, 6):
        assert np.array_equal(dev_ns(ctx, Ws[e], 1, M, N, 5, muon_ns.PE_SCHEDULE), out[e * M:(e + 1) * M]), e


@pytest.mark.parametrize("E,M,N,steps", [(1, 256, 256, 1), (3, 256, 512, 2), (5, 512, 1024, 5), (7, 1024, 1024, 5),
                                         (16, 768, 1024, 5), (2, 1024, 3072, 4), (11, 1024, 3072, 5),
                                         (40, 256, 256, 3)])
def test_single_launch_chain_equals_one_launch_per_phase(ctx, monkeypatch, E, M, N, steps):
    """The persistent chain kernel (dynamic tile queue over all phases, per-matrix dependency
    counters) must give the bits of the phase-by-phase launches: same tiles, same K order."""
    rng = np.random.default_rng(E * 1000 + M + N + steps)
    Xb = f32_to_bf16_bits((rng.standard_normal((E * M, N)) * 1e-3).astype(np.float32))
    monkeypatch.setenv("ANCORA_NS_CHAIN", "0")
    per_phase = dev_ns(ctx, Xb, E, M, N, steps, muon_ns.PE_SCHEDULE)
    monkeypatch.delenv("ANCORA_NS_CHAIN")
    chain = dev_ns(ctx, Xb, E, M, N, steps, muon_ns.PE_SCHEDULE)
    assert np.array_equal(chain, per_phase)
    for _ in range(3):                              # dynamic scheduling must not show in the bits
        assert np.array_equal(dev_ns(ctx, Xb, E, M, N, steps, muon_ns.PE_SCHEDULE), chain)


def test_reserved_sms_do_not_change_the_bits(ctx):
    """Leaving SMs to other streams (what a rank does while NCCL's all-gather overlaps the chain)
    changes how many CTA pairs share the tile queue, not what a tile computes."""
    rng = np.random.default_rng(11)
    E, M, N = 9, 512, 1024
    Xb = f32_to_bf16_bits((rng.standard_normal((E * M, N)) * 1e-3).astype(np.float32))
    want = dev_ns(ctx, Xb, E, M, N, 5, muon_ns.PE_SCHEDULE)
    try:
        for n in (16, 100, 146):
            ctx.reserve_sms(n)
            assert np.array_equal(dev_ns(ctx, Xb, E, M, N, 5, muon_ns.PE_SCHEDULE), want), n
    finally:
        ctx.reserve_sms(0)
    with pytest.raises(anc.AncoraError):
        ctx.reserve_sms(10 ** 6)


def test_dependency_wait_runs_out_and_context_survives(ctx):
    """A tile whose dependency nobody completes: the bounded wait gives up, status bit 0x10 is
    set, the kernel drains and returns, and the context keeps working (no trap, no hang)."""
    import ctypes as C
    from ancora_cutile_b200 import _lib as L
    ctx.sync()
    assert ctx.status() == 0
    L.check(L.lib().anc_ns_chain_wait_selftest(ctx.handle, C.c_uint32(2000)))
    assert ctx.status() == 0x10
    assert ctx.status() == 0                                       # reading clears it
    rng = np.random.default_rng(9)
    Xb = f32_to_bf16_bits(rng.standard_normal((256, 256)).astype(np.float32))
    got = bits_to_f32(dev_ns(ctx, Xb, 1, 256, 256, 5, muon_ns.PE_SCHEDULE))     # ordinary work still runs
    c, r = cos_rel(got, muon_ref.ns_fp32(bits_to_f32(Xb), 5, muon_ref.PE_SCHEDULE))
    assert c > 0.999 and r < 0.02


def test_shape_errors(ctx):
    d = anc.DBuf.zeros((128, 128), np.uint16, ctx)
    r = anc.DBuf.zeros((1,), np.float32, ctx)
    with pytest.raises(AssertionError):
        muon_ns.newton_schulz_resident(d, d, d, d, d, r, 256, 128, ctx.stream)      # M > N
    with pytest.raises(AssertionError):
        muon_ns.newton_schulz_resident(d, d, d, d, d, r, 64, 128, ctx.stream)       # tile-misaligned
    d.free(); r.free()
