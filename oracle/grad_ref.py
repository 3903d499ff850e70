"""Gradient producer restated in numpy (test infrastructure; never on the product path).

Accumulation follows ancora/kernels/fused.py:242-249 (`_acc_f32`: dst = src + dst, one float32
add per element); the stochastic downcast uses the bit rule of ancora/kernels/fused.py:159-161
(`_gemm_dx_sr`: (bits + dither16) >> 16) with this build's Philox stream (oracle/philox.py) in
place of the reference's coordinate hash: parity of the dither stream is unpinned by the
reference, the add and the bit rule are pinned by the formulas cited.
"""
import numpy as np

from .bf16 import bits_f32, rne_bits, sr_bits
from .philox import dither16_range


def grad_accumulate(acc, src=None, want_g16=True, scale=1.0, rounding="rne", seed=0, step=0,
                    elem_offset=0, zero_after=False):
    """Returns (acc_out, g16_bits or None).  ``src`` is float32 or bf16 bits (uint16)."""
    f = np.float32
    a = np.asarray(acc, f).reshape(-1)
    if src is not None:
        s = np.asarray(src).reshape(-1)
        s = bits_f32(s).astype(f) if s.dtype == np.uint16 else s.astype(f)
        a = (s + a).astype(f)
    g16 = None
    if want_g16:
        x = (a * f(scale)).astype(f)
        if rounding == "rne":
            g16 = rne_bits(x)
        elif rounding == "sr":
            g16 = sr_bits(x, dither16_range(elem_offset, x.size, seed, step))
        else:
            raise ValueError(rounding)
    out = np.zeros_like(a) if zero_after else a
    return out, g16
