"""Test infrastructure: CPU restatement of the counter-based generator behind
the device-side noise (csrc/noise.cu).  Philox4x32-10 as published by Salmon,
Moraes, Dror and Shaw, "Parallel random numbers: as easy as 1, 2, 3" (SC'11):
ten rounds of  (c0, c1, c2, c3) <- (hi(M1 c2) ^ c1 ^ k0, lo(M1 c2),
hi(M0 c0) ^ c3 ^ k1, lo(M0 c0)), the key bumped by the Weyl constants between
rounds.  The reference has no counterpart (it draws from per-thread
std::mt19937 streams); this file pins the device generator, nothing else."""
from __future__ import annotations

import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(counters, key):
    """counters: [N, 4] uint32, key: (k0, k1); returns [N, 4] uint32."""
    c = np.asarray(counters, np.uint64) & MASK
    c0, c1, c2, c3 = (c[:, j].copy() for j in range(4))
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        c0, c1, c2, c3 = ((p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0), p1 & MASK,
                          (p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1), p0 & MASK)
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def words(n, seed, stream, step, first=0):
    """The n 32-bit words of a draw: word i is lane (first + i) mod 4 of the
    block with counter ((first + i) / 4 low, high, stream, step), key = seed."""
    idx = np.arange(first, first + n, dtype=np.uint64)
    blocks, inverse = np.unique(idx // np.uint64(4), return_inverse=True)
    ctr = np.zeros((blocks.size, 4), np.uint64)
    ctr[:, 0] = blocks & MASK
    ctr[:, 1] = blocks >> np.uint64(32)
    ctr[:, 2] = stream
    ctr[:, 3] = step
    out = philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    return out[inverse, (idx % np.uint64(4)).astype(np.int64)]


def unit(x):
    """24 random bits -> [0, 1) in fp32."""
    return (x >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def uniform(n, lo, hi, seed, stream, step, first=0):
    width = np.float32(np.float32(hi) - np.float32(lo))
    return (unit(words(n, seed, stream, step, first)) * width + np.float32(lo)).astype(np.float32)


def bernoulli(n, p, seed, stream, step, first=0):
    return (unit(words(n, seed, stream, step, first)) < np.float32(p)).astype(np.uint8)
