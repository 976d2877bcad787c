"""NumPy restatement of the device noise generator (csrc/kernels/dp_step.cu): Philox4x32-10 + Box-Muller.

Element ``e`` of the global flat parameter vector uses counter ``(e // 4, step, stream_id)`` and key ``seed``;
lane ``e % 4`` selects one of the four normals. Used as the CPU oracle of the GPU noise and by the CPU paths.
"""
from __future__ import annotations

import numpy as np

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = np.uint32(0x9E3779B9), np.uint32(0xBB67AE85)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint32) for c in (c0, c1, c2, c3))
    k0 = np.uint32(k0)
    k1 = np.uint32(k1)
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = _M0 * c0.astype(np.uint64)
            p1 = _M1 * c2.astype(np.uint64)
            n0 = (p1 >> np.uint64(32)).astype(np.uint32) ^ c1 ^ k0
            n1 = p1.astype(np.uint32)
            n2 = (p0 >> np.uint64(32)).astype(np.uint32) ^ c3 ^ k1
            n3 = p0.astype(np.uint32)
            c0, c1, c2, c3 = n0, n1, n2, n3
            k0 = np.uint32(k0 + _W0)
            k1 = np.uint32(k1 + _W1)
    return c0, c1, c2, c3


def normal(n: int, seed: int, step: int, *, stream_id: int = 0, offset: int = 0) -> np.ndarray:
    """Standard normals for global elements ``offset .. offset+n-1`` as float32."""
    seed &= 2**64 - 1
    e = np.arange(offset, offset + n, dtype=np.uint64)
    q = e >> np.uint64(2)
    lane = (e & np.uint64(3)).astype(np.int64)
    uq, inv = np.unique(q, return_inverse=True)
    r = philox4x32_10((uq & np.uint64(0xFFFFFFFF)).astype(np.uint32), (uq >> np.uint64(32)).astype(np.uint32),
                      np.full(uq.shape, step & 0xFFFFFFFF, np.uint32), np.full(uq.shape, stream_id, np.uint32),
                      seed & 0xFFFFFFFF, seed >> 32)
    k = np.float32(2.3283064365386963e-10)
    u1 = (r[0].astype(np.float32) + np.float32(1.0)) * k
    u2 = r[1].astype(np.float32) * k
    u3 = (r[2].astype(np.float32) + np.float32(1.0)) * k
    u4 = r[3].astype(np.float32) * k
    ra = np.sqrt(np.float32(-2.0) * np.log(np.minimum(u1, np.float32(1.0))))
    rb = np.sqrt(np.float32(-2.0) * np.log(np.minimum(u3, np.float32(1.0))))
    two_pi = np.float32(2.0 * np.pi)
    z = np.stack([ra * np.cos(two_pi * u2), ra * np.sin(two_pi * u2), rb * np.cos(two_pi * u4), rb * np.sin(two_pi * u4)],
                 axis=1).astype(np.float32)
    return z[inv, lane]
