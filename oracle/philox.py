"""Philox4x32-10 on the CPU.  TEST INFRASTRUCTURE ONLY.

The seeded draw is not part of the reference (it draws through torch's generator,
hydraserve/engine/sampling.py:144-150); the CUDA sampler draws from a counter-based Philox
stream instead.  This file restates the published generator (Salmon, Moraes, Dror, Shaw:
"Parallel random numbers: as easy as 1, 2, 3", SC'11; the Random123 library's philox4x32 with
10 rounds) so that a test can say which 32-bit words a (counter, key) pair gives and hold the
kernels' stream to it bit for bit.  Pinned by the generator's published known-answer vectors
(tests/test_oracle.py).  Only tests import it.
"""
from __future__ import annotations

M0, M1 = 0xD2511F53, 0xCD9E8D57  # round multipliers
W0, W1 = 0x9E3779B9, 0xBB67AE85  # key increments (golden ratio, sqrt(3) - 1)
_MASK = 0xFFFFFFFF


def philox4x32_10(counter, key):
    """(c0, c1, c2, c3), (k0, k1) -> four 32-bit words."""
    c0, c1, c2, c3 = (int(v) & _MASK for v in counter)
    k0, k1 = (int(v) & _MASK for v in key)
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0, k1 = (k0 + W0) & _MASK, (k1 + W1) & _MASK
    return c0, c1, c2, c3


def first_draw_words(stream_key: int):
    """The four words a row's first draw uses: counter 0, key = the low and high half of the
    row's 63-bit stream key (the reference's mixed seed, sampling.py:148)."""
    return philox4x32_10((0, 0, 0, 0), (stream_key & _MASK, (stream_key >> 32) & _MASK))
