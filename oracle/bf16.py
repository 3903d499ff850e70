"""bf16 <-> f32 bit helpers (test infrastructure).

``rne_bits`` follows ancora/optim/adamw.py:63-66 (``_bf16_bits``: add 0x7FFF plus
the lsb of the kept half, shift right 16), with one stated extension: a NaN maps
to the canonical quiet NaN 0x7FFF, which is what the hardware conversion the
device kernels use (``cvt.rn.bf16.f32``) produces; the reference's bit trick is
undefined there.  ``sr_bits`` follows the bit rule of
ancora/kernels/fused.py:159-161 (``(u32 + dither16) >> 16`` on the raw pattern).
"""
import numpy as np


def f32_bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def bits_f32(u16):
    return (np.asarray(u16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def rne_bits(x):
    """float32 array -> bf16 bit patterns (uint16), round to nearest even."""
    u = f32_bits(x).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)
    nan = np.isnan(np.asarray(x, dtype=np.float32))
    return np.where(nan, np.uint16(0x7FFF), r).astype(np.uint16)


def rne_f32(x):
    """Round to bf16 and return the value as float32 (ancora/optim/muon.py:83-85 ``_bf``)."""
    return bits_f32(rne_bits(x))


def sr_bits(x, dither):
    """Stochastic rounding: ``(bits + dither) >> 16`` with a 16-bit dither per element.

    Values exactly representable in bf16 map to themselves; the magnitude rounds
    away from zero with probability low16/65536; +-Inf pass through; NaN -> 0x7FFF.
    """
    u = f32_bits(x).astype(np.uint64)
    d = np.asarray(dither).astype(np.uint64) & np.uint64(0xFFFF)
    r = ((u + d) >> np.uint64(16)).astype(np.uint16)
    nan = np.isnan(np.asarray(x, dtype=np.float32))
    return np.where(nan, np.uint16(0x7FFF), r).astype(np.uint16)
