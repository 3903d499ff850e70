"""CPU: properties of the gradient-producer oracle and of the transposed MXFP8 oracle that do
not depend on any device (the oracle is the checker of the GPU tests, so it is checked first)."""
import numpy as np

from oracle import grad_ref, quant_ref
from oracle.bf16 import bits_f32, rne_bits


def test_accumulate_is_one_float32_add_and_scale_only_touches_the_output():
    rng = np.random.default_rng(0)
    acc = rng.standard_normal(1000).astype(np.float32)
    src = rng.standard_normal(1000).astype(np.float32)
    out, g = grad_ref.grad_accumulate(acc, src, scale=0.5)
    assert np.array_equal(out, acc + src)
    assert np.array_equal(g, rne_bits((acc + src) * np.float32(0.5)))
    out0, g0 = grad_ref.grad_accumulate(acc, src, zero_after=True)
    assert not out0.any() and np.array_equal(g0, rne_bits(acc + src))


def test_sr_keeps_representable_values_and_brackets_the_rest():
    rng = np.random.default_rng(1)
    x = rng.standard_normal(4096).astype(np.float32)
    exact = bits_f32(rne_bits(x)).astype(np.float32)
    _, g = grad_ref.grad_accumulate(exact, None, rounding="sr", seed=3, step=4)
    assert np.array_equal(bits_f32(g), exact)
    _, g = grad_ref.grad_accumulate(x, None, rounding="sr", seed=3, step=4)
    lo = (x.view(np.uint32) >> 16).astype(np.uint16)
    assert np.all((g == lo) | (g == lo + 1))
    # a split arena with global offsets draws the bits of the whole
    _, ga = grad_ref.grad_accumulate(x[:1001], None, rounding="sr", seed=3, step=4)
    _, gb = grad_ref.grad_accumulate(x[1001:], None, rounding="sr", seed=3, step=4, elem_offset=1001)
    assert np.array_equal(np.concatenate([ga, gb]), g)


def test_transposed_mxfp8_is_the_row_major_bytes_transposed_and_decodes_within_a_step():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((128, 64)) * np.exp(rng.uniform(-6, 1, (1, 64)))).astype(np.float32)
    w16 = rne_bits(w.reshape(-1)).reshape(w.shape)
    q, b = quant_ref.quant_mxfp8_w(w16)
    qt, bt = quant_ref.quant_mxfp8_w_cm(w16)
    assert qt.shape == (64, 128) and bt.shape == (64, 4)
    assert np.array_equal(qt.T, q) and np.array_equal(bt.T, b)
    back = quant_ref.dequant_mxfp8_w(q, b)
    ref = bits_f32(w16).astype(np.float64)
    amax = np.abs(ref).reshape(4, 32, 64).max(axis=1)
    # E4M3 keeps 3 mantissa bits: error at most 2^-4 of the block's power-of-two ceiling
    assert np.all(np.abs(back - ref).reshape(4, 32, 64) <= amax[:, None, :] * 2.0 ** -3)
