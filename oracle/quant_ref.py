"""MXFP8 weight re-quantisation restated in numpy (test infrastructure).

Follows ancora/kernels/quant.py:56-68 (`_quant_mxfp8_w`): blocks of 32 along K (axis 0);
per block and column the E8M0 scale byte is ``max(exponent_bits(max|w|) - 7, 0)`` (floor
exponent), the scale ``2**(byte-127)`` and the stored value ``RNE_e4m3fn(w / scale)``.
The reference kernel only runs on a GPU, so the block formula (floor-exponent scale byte) is a
restatement by reading: parity of the scale rule is unpinned by reference outputs.  What the
reference's host helpers can pin is pinned by fixtures recorded from them
(tests/golden/e4m3.npz: `_e4m3_table`, `f32_to_e4m3`, `dequantize_rowblock`, quant.py:92-175):
the code table, the nearest-value rounding away from exact ties, the block dequantisation.  At
exact ties the kernels' conversion is round-to-nearest-even (followed here); the host helper
rounds ties to the smaller magnitude.
"""
import numpy as np

from .bf16 import bits_f32


def _e4m3_rne(x):
    """float32 -> E4M3fn byte, round to nearest even.  Uses ml_dtypes when present, else a
    table search over the 256 code points (ancora/kernels/quant.py `_e4m3_table`)."""
    try:
        import ml_dtypes
        return x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    except ImportError:                                       # pragma: no cover
        vals = e4m3_table()
        pos = np.where(np.isnan(vals), np.inf, vals)
        order = np.argsort(pos[:0x7F])
        grid = pos[:0x7F][order]
        a = np.abs(x.astype(np.float64))
        hi = np.clip(np.searchsorted(grid, a), 1, len(grid) - 1)
        lo = hi - 1
        dl, dh = a - grid[lo], grid[hi] - a
        pick = np.where((dl < dh) | ((dl == dh) & (order[lo] % 2 == 0)), order[lo], order[hi])
        return (pick | np.where(np.signbit(x), 0x80, 0)).astype(np.uint8)


def e4m3_table():
    v = np.zeros(256, np.float64)
    for b in range(256):
        s = -1.0 if (b & 0x80) else 1.0
        e, m = (b >> 3) & 0xF, b & 0x7
        if e == 0:
            val = (m / 8.0) * 2.0 ** -6
        elif e == 15 and m == 7:
            val = np.nan
        else:
            val = (1 + m / 8.0) * 2.0 ** (e - 7)
        v[b] = s * val
    return v


def quant_mxfp8_w(w16):
    """w16: (K,N) bf16 bits -> (fp8 (K,N) uint8, scale (K//32,N) uint8)."""
    w = bits_f32(w16).astype(np.float32)
    K, N = w.shape
    blk = w.reshape(K // 32, 32, N)
    amax = np.abs(blk).max(axis=1)
    ea = (amax.view(np.uint32) >> np.uint32(23)) & np.uint32(0xFF)
    byte = np.where(ea >= 7, ea - 7, 0).astype(np.uint8)
    sc = np.exp2(byte.astype(np.float32) - np.float32(127.0)).astype(np.float32)
    q = _e4m3_rne((blk / sc[:, None, :]).astype(np.float32)).reshape(K, N)
    return q, byte


def quant_mxfp8_w_cm(w16):
    """w16: (K,N) bf16 bits -> (fp8 (N,K) uint8, scale (N,K//32) uint8): the same bytes as
    `quant_mxfp8_w`, stored transposed (ancora/kernels/quant.py:79-90, `_quant_mxfp8_w_cm`)."""
    q, byte = quant_mxfp8_w(w16)
    return np.ascontiguousarray(q.T), np.ascontiguousarray(byte.T)


def dequant_mxfp8_w(q, byte):
    K, N = q.shape
    v = e4m3_table()[q].reshape(K // 32, 32, N)
    return (v * np.exp2(byte.astype(np.float64) - 127.0)[:, None, :]).reshape(K, N)
