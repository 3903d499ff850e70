"""GPU: the fused gradient producer (accumulate + bf16 downcast in one sweep) against the
CPU oracle, bit for bit.  The reference has the two halves as separate kernels
(ancora/kernels/fused.py:242-249 `_acc_f32`; the stochastic-rounding bit rule of
fused.py:159-161); exact equality under this build's Philox stream is this build's own gate."""
import numpy as np
import pytest

import ancora_cutile_b200 as anc
from ancora_cutile_b200 import kernels
from ancora_cutile_b200.bf16 import bits_to_f32, f32_to_bf16_bits
from oracle import grad_ref

pytestmark = pytest.mark.gpu


def _inputs(rng, n):
    acc = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    src = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    return acc, src


@pytest.mark.parametrize("src_dtype", ["f32", "bf16"])
@pytest.mark.parametrize("rounding", ["rne", "sr"])
@pytest.mark.parametrize("n", [8 * 1024 * 33, 4099, 5])
def test_accumulate_and_downcast_match_oracle(ctx, src_dtype, rounding, n):
    rng = np.random.default_rng(n)
    acc, src = _inputs(rng, n)
    if n > 16:
        acc[3], src[7], acc[11] = np.inf, np.nan, -0.0
    src_h = f32_to_bf16_bits(src) if src_dtype == "bf16" else src
    d_acc, d_src = anc.DBuf(acc, ctx), anc.DBuf(src_h, ctx)
    d_g = anc.DBuf.zeros((n,), np.uint16, ctx)
    kernels.grad_accumulate(d_acc, d_src, d_g, n, src_dtype=src_dtype, elem_offset=64, scale=0.25,
                            rounding=rounding, seed=99, step=7, ctx=ctx)
    ctx.sync()
    want_acc, want_g = grad_ref.grad_accumulate(acc, src_h, scale=0.25, rounding=rounding, seed=99, step=7,
                                                elem_offset=64)
    got_acc, got_g = d_acc.to_numpy(), d_g.to_numpy()
    nan = np.isnan(want_acc)          # NaN payloads are not part of the contract, NaN-ness is
    assert np.array_equal(np.isnan(got_acc), nan)
    assert np.array_equal(got_acc.view(np.uint32)[~nan], want_acc.view(np.uint32)[~nan])
    assert np.array_equal(got_g, want_g)
    for b in (d_acc, d_src, d_g):
        b.free()


def test_unaligned_views_and_odd_offset_draw_the_same_bits(ctx):
    """A slice that starts at an odd element (scalar path) must give the bits the aligned whole
    gives at the same global positions; downcast-only leaves acc untouched; zero_after clears."""
    n, cut = 8 * 1024 + 13, 1001
    rng = np.random.default_rng(3)
    acc, src = _inputs(rng, n)
    d_acc, d_src = anc.DBuf(acc, ctx), anc.DBuf(src, ctx)
    d_g = anc.DBuf.zeros((n,), np.uint16, ctx)
    # whole arena in two calls split at an odd element; global offsets keep the stream continuous
    kernels.grad_accumulate(d_acc.slice_elems(0, cut), d_src.slice_elems(0, cut), d_g.slice_elems(0, cut), cut,
                            rounding="sr", seed=5, step=2, ctx=ctx)
    kernels.grad_accumulate(d_acc.slice_elems(cut, n - cut), d_src.slice_elems(cut, n - cut),
                            d_g.slice_elems(cut, n - cut), n - cut, elem_offset=cut, rounding="sr", seed=5,
                            step=2, ctx=ctx)
    ctx.sync()
    want_acc, want_g = grad_ref.grad_accumulate(acc, src, rounding="sr", seed=5, step=2)
    assert np.array_equal(d_acc.to_numpy(), want_acc)
    assert np.array_equal(d_g.to_numpy(), want_g)
    # downcast only (no contribution): acc unchanged, new bits from the new step
    kernels.grad_accumulate(d_acc, None, d_g, n, rounding="sr", seed=5, step=3, ctx=ctx)
    ctx.sync()
    _, want_g3 = grad_ref.grad_accumulate(want_acc, None, rounding="sr", seed=5, step=3)
    assert np.array_equal(d_acc.to_numpy(), want_acc)
    assert np.array_equal(d_g.to_numpy(), want_g3)
    assert not np.array_equal(want_g3, want_g)
    # accumulate only, then final downcast that clears the accumulator
    kernels.grad_accumulate(d_acc, d_src, None, n, ctx=ctx)
    kernels.grad_accumulate(d_acc, None, d_g, n, scale=0.5, zero_after=True, ctx=ctx)
    ctx.sync()
    acc2, _ = grad_ref.grad_accumulate(want_acc, src, want_g16=False)
    _, want_g4 = grad_ref.grad_accumulate(acc2, None, scale=0.5)
    assert np.array_equal(d_g.to_numpy(), want_g4)
    assert not d_acc.to_numpy().any()
    for b in (d_acc, d_src, d_g):
        b.free()


def test_rejects_bad_arguments(ctx):
    d = anc.DBuf.zeros((64,), np.float32, ctx)
    with pytest.raises(anc.AncoraError):
        kernels.grad_accumulate(d, None, None, 64, ctx=ctx)          # nothing to do
    with pytest.raises(anc.AncoraError):
        kernels.grad_accumulate(d, d.slice_elems(0, 8).ptr + 2, None, 8, ctx=ctx)   # misaligned f32
    d.free()


def test_sr_downcast_is_unbiased(ctx):
    """Mean of the stochastic downcast over many steps approaches the float32 value
    (the property tests/kernels/_probe_sr_ops.py checks for the reference's dither)."""
    n, steps = 4096, 256
    rng = np.random.default_rng(11)
    acc = (rng.standard_normal(n) * 1e-3).astype(np.float32)
    d_acc = anc.DBuf(acc, ctx)
    d_g = anc.DBuf.zeros((n,), np.uint16, ctx)
    tot = np.zeros(n, np.float64)
    for t in range(steps):
        kernels.grad_accumulate(d_acc, None, d_g, n, rounding="sr", seed=1, step=t, ctx=ctx)
        ctx.sync()
        tot += bits_to_f32(d_g.to_numpy()).astype(np.float64)
    ulp = np.abs(acc).astype(np.float64) * 2.0 ** -8
    # standard error of the mean of a two-point distribution of width <= 1 ulp(bf16)
    assert np.all(np.abs(tot / steps - acc) <= 6 * ulp / np.sqrt(steps) + 1e-12)
    d_acc.free(); d_g.free()


def test_engine_accumulates_micro_batches_and_steps_on_the_sum(ctx):
    """Three micro-batches folded into the float32 accumulators, one sweep that writes the bf16
    gradients of the step: bits equal the oracle's, and the step equals a step on those bits."""
    from ancora_cutile_b200 import shapes as S
    shp = S.qwen3_0_6b_shapes(n_layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=128, ffn=768, vocab=2048)
    params = S.synthetic_params(shp, seed=5)
    mu = [n for n, p in params.items() if anc.default_is_muon(n, p)]
    nd = tuple(n for n, s in shp.items() if len(s) == 1)
    kw = dict(adamw_kw=dict(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, wd=0.1), grad_dtype="bf16", rounding="sr",
              seed=7, schedule=anc.PE_SCHEDULE, ctx=ctx)
    micro = [S.synthetic_grads_bf16(shp, seed=60 + k) for k in range(3)]
    eng = anc.ResidentHybrid(params, mu, nd, **kw)
    eng.enable_grad_accumulation()
    for k, g in enumerate(micro):
        eng.upload_grads(g, ctx.stream)
        if k < 2:
            eng.accumulate_grads(ctx.stream)
        else:
            eng.finalize_grads(ctx.stream)             # scale 1/3, SR, seed 8, step 1
    ctx.sync()
    summed = {}
    for n in shp:
        acc = np.zeros(int(np.prod(shp[n])), np.float32)
        for g in micro:
            acc, _ = grad_ref.grad_accumulate(acc, g[n].reshape(-1), want_g16=False)
        off = eng.a_off[n] if n in eng.a_off else eng.a_padded + eng.m_off[n]
        _, bits = grad_ref.grad_accumulate(acc, None, scale=1.0 / 3.0, rounding="sr", seed=8, step=1, elem_offset=off)
        summed[n] = bits.reshape(shp[n])
        assert np.array_equal(eng.grad_view(n).to_numpy(), summed[n]), n
    assert not eng.acc_a.to_numpy().any() and not eng.acc_m.to_numpy().any()
    eng.step(ctx.stream)
    ctx.sync()
    got, _ = eng.download_weights_bits()
    got = {n: b.copy() for n, b in got.items()}
    eng.free()
    ref = anc.ResidentHybrid(params, mu, nd, **kw)
    ref.upload_grads(summed, ctx.stream)
    ref.step(ctx.stream)
    ctx.sync()
    want, _ = ref.download_weights_bits()
    for n in shp:
        assert np.array_equal(got[n], want[n]), n
    ref.free()
    assert ctx.status() == 0
