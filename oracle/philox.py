"""Philox4x32-10 counter-based generator (Salmon et al., SC'11), vectorised numpy.

Test infrastructure: the checker for the device kernel's stochastic-rounding
dither.  The reference repository has no Philox (its only stochastic rounding,
ancora/kernels/fused.py:154-161, hashes tile coordinates), so this stream is
defined by this build and pinned by the published known-answer vectors in
``KNOWN_ANSWERS`` below.

Stream layout used by the optimizer (fixed by the spec, not by a launch shape):

    key     = (seed & 0xffffffff, seed >> 32)
    counter = (blk & 0xffffffff, blk >> 32, step & 0xffffffff, step >> 32)
    blk     = global_element_index // 8

One Philox call yields four 32-bit words = eight 16-bit dithers for the eight
consecutive elements ``8*blk .. 8*blk+7``: element ``j`` of the block takes word
``j // 2``, low half when ``j`` is even, high half when ``j`` is odd.
"""
import numpy as np

PHILOX_M0 = np.uint64(0xD2511F53)
PHILOX_M1 = np.uint64(0xCD9E8D57)
PHILOX_W0 = 0x9E3779B9
PHILOX_W1 = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)
_SH32 = np.uint64(32)

# (counter words, key words, expected output words)
KNOWN_ANSWERS = [
    ((0x00000000, 0x00000000, 0x00000000, 0x00000000), (0x00000000, 0x00000000),
     (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF), (0xFFFFFFFF, 0xFFFFFFFF),
     (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
     (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
]


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Ten Philox rounds on arrays (or scalars) of 32-bit counter words.

    Returns four uint32 arrays.  All inputs are broadcast against each other.
    """
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _MASK32 for c in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0 = int(k0) & 0xFFFFFFFF
    k1 = int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = PHILOX_M0 * c0                      # 32x32 -> 64, exact in uint64
        p1 = PHILOX_M1 * c2
        n0 = (p1 >> _SH32) ^ c1 ^ np.uint64(k0)
        n1 = p1 & _MASK32
        n2 = (p0 >> _SH32) ^ c3 ^ np.uint64(k1)
        n3 = p0 & _MASK32
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + PHILOX_W0) & 0xFFFFFFFF
        k1 = (k1 + PHILOX_W1) & 0xFFFFFFFF
    return tuple(c.astype(np.uint32) for c in (c0, c1, c2, c3))


def dither16(elem_index, seed, step):
    """16-bit dither for each global element index (uint64 array) under (seed, step)."""
    idx = np.asarray(elem_index, dtype=np.uint64)
    blk = idx >> np.uint64(3)
    lane = (idx & np.uint64(7)).astype(np.int64)
    # one Philox call per distinct block
    ublk, inv = np.unique(blk, return_inverse=True)
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    step = int(step) & 0xFFFFFFFFFFFFFFFF
    w = philox4x32_10(ublk & _MASK32, ublk >> _SH32,
                      np.uint64(step & 0xFFFFFFFF), np.uint64(step >> 32),
                      seed & 0xFFFFFFFF, seed >> 32)
    words = np.stack(w, axis=-1)                 # (nblk, 4) uint32
    word = words[inv.reshape(idx.shape), lane >> 1]
    return np.where(lane & 1, word >> np.uint32(16), word & np.uint32(0xFFFF)).astype(np.uint32)


def dither16_range(start, count, seed, step):
    """Dithers for the contiguous element range [start, start+count) without the
    ``np.unique`` pass (fast path for large arenas)."""
    start = int(start); count = int(count)
    b0 = start >> 3
    b1 = (start + count + 7) >> 3
    blk = np.arange(b0, b1, dtype=np.uint64)
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    step = int(step) & 0xFFFFFFFFFFFFFFFF
    w = philox4x32_10(blk & _MASK32, blk >> _SH32,
                      np.uint64(step & 0xFFFFFFFF), np.uint64(step >> 32),
                      seed & 0xFFFFFFFF, seed >> 32)
    words = np.stack(w, axis=-1).reshape(-1)     # word-major: blk*4 + word
    halves = np.empty(words.size * 2, dtype=np.uint32)
    halves[0::2] = words & np.uint32(0xFFFF)
    halves[1::2] = words >> np.uint32(16)
    off = start - (b0 << 3)
    return halves[off:off + count]
