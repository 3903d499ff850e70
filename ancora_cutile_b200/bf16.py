"""Host-side bf16 bit helpers used to prepare inputs and decode outputs.

``f32_to_bf16_bits`` rounds to nearest even exactly as the reference's ``_bf16_bits``
(ancora/optim/adamw.py:63-66); ``bits_to_f32`` is its ``_bits_f32`` (adamw.py:66).
These only convert data on the host; no optimizer arithmetic happens here.
"""
import numpy as np


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)
    nan = np.isnan(np.asarray(x, dtype=np.float32))
    if nan.any():
        r = np.where(nan, np.uint16(0x7FFF), r).astype(np.uint16)
    return r


def bits_to_f32(u16):
    return (np.asarray(u16).astype(np.uint32) << np.uint32(16)).view(np.float32)
