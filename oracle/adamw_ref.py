"""AdamW restated in numpy float32 (test infrastructure; never on the product path).

Follows the reference kernel's operation order, ancora/optim/adamw.py:34-37:

    mn  = beta1 * m + (1.0 - beta1) * g
    vn  = beta2 * v + (1.0 - beta2) * g * g          # ((1-beta2)*g)*g, left to right
    upd = (mn * ibc1) / (sqrt(vn * ibc2) + eps) + wd * p
    pn  = p - lr * upd

which is also the router's host form in ancora/kernels/moe.py:607-609.  Every
product and sum is a separate float32 operation (numpy never contracts to FMA).

The derived scalars are materialised ONCE, the same way for this oracle and for
the device kernel (``adamw_scalars``): beta/eps/lr/wd are the float32 casts of
the Python floats the reference passes as kernel scalars (adamw.py:95-97);
``1 - beta`` is the float32 subtraction the reference kernel performs in-kernel
(adamw.py:34-35: ``1.0 - beta1`` on a float32 scalar); the bias corrections are
computed in Python double and then cast (adamw.py:90-91,97).
"""
from collections import namedtuple
import numpy as np

from .bf16 import rne_bits, sr_bits, bits_f32
from .philox import dither16_range

Scalars = namedtuple("Scalars", "b1 omb1 b2 omb2 eps lr ibc1 ibc2")


def adamw_scalars(lr, b1, b2, eps, t):
    f = np.float32
    return Scalars(b1=f(b1), omb1=f(1.0) - f(b1), b2=f(b2), omb2=f(1.0) - f(b2),
                   eps=f(eps), lr=f(lr),
                   ibc1=f(1.0 / (1.0 - b1 ** t)), ibc2=f(1.0 / (1.0 - b2 ** t)))


def adamw_update(p, m, v, g, s, wd):
    """One AdamW step on float32 arrays; g is float32 (a bf16 grad is widened exactly
    before the call).  Returns (pn, mn, vn), all float32."""
    f = np.float32
    p = np.asarray(p, f); m = np.asarray(m, f); v = np.asarray(v, f); g = np.asarray(g, f)
    wd = f(wd)
    mn = s.b1 * m + s.omb1 * g
    vn = s.b2 * v + (s.omb2 * g) * g
    upd = (mn * s.ibc1) / (np.sqrt(vn * s.ibc2) + s.eps) + wd * p
    pn = p - s.lr * upd
    assert pn.dtype == f and mn.dtype == f and vn.dtype == f
    return pn, mn, vn


def adamw_step(p, m, v, g, s, wd, rounding="rne", seed=0, step=0, elem_offset=0):
    """Full step for one flat tensor: state update plus the bf16 parameter copy.

    rounding="rne": ancora/optim/adamw.py:41 (``astype(bfloat16)``).
    rounding="sr" : stochastic rounding with the Philox stream of oracle/philox.py;
                    ``elem_offset`` is the tensor's first index in the global arena.
    Returns (pn, mn, vn, p16_bits).
    """
    pn, mn, vn = adamw_update(p, m, v, g, s, wd)
    flat = pn.reshape(-1)
    if rounding == "rne":
        p16 = rne_bits(flat)
    elif rounding == "sr":
        p16 = sr_bits(flat, dither16_range(elem_offset, flat.size, seed, step))
    else:
        raise ValueError(rounding)
    return pn, mn, vn, p16.reshape(pn.shape)


def adamw_reference_test_form(p, m, v, g, lr, b1, b2, eps, wd, t):
    """The divide-by-bias-correction form the reference's own test compares with at
    rel 1e-5 (tests/optim/test_adamw.py:37-41; also model/resident_model.py:168-172)."""
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    mh = m / (1 - b1 ** t)
    vh = v / (1 - b2 ** t)
    p = p - lr * (mh / (np.sqrt(vh) + eps) + wd * p)
    return p, m, v
