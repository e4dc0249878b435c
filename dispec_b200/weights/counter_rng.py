"""Counter-based normal numbers on the CPU: value = f(seed, tensor ordinal, element index).

The same function as the device kernel ``dsp_fill_normal`` (csrc/random_fill.cu), bit for bit:
Philox-4x32-10 with counter (index // 4 low word, high word, ordinal, 0) and key (seed low word,
high word); the four output words make two Box-Muller pairs whose logarithm, sine and cosine are
spelled out in float32 with single correctly rounded operations (numpy float32 arithmetic here,
``__fmul_rn`` and friends there), so any element of any tensor can be computed alone, in any
order, on either side.  The reference has no such generator (it draws test weights with the model
library's own initialiser under ``torch.manual_seed``, puneethgv/DiSpec tests/tiny_models.py:17-23).
"""
from __future__ import annotations

import numpy as np

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_F = np.float32


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Arrays of uint64 holding 32-bit words in, four such arrays out."""
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & _MASK, p1 >> np.uint64(32), p1 & _MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def _log(u):
    bits = u.view(np.uint32)
    e = (bits >> np.uint32(23)).astype(np.int32) - np.int32(127)
    m = ((bits & np.uint32(0x007FFFFF)) | np.uint32(0x3F800000)).view(np.float32)
    big = m > _F(1.41421354)
    m = np.where(big, m * _F(0.5), m)
    e = e + big.astype(np.int32)
    f = m - _F(1.0)
    s = f / (f + _F(2.0))
    z = s * s
    p = z * _F(0.222222224) + _F(0.285714298)
    p = z * p + _F(0.400000006)
    p = z * p + _F(0.666666687)
    p = z * p + _F(2.0)
    return e.astype(np.float32) * _F(0.693147182) + s * p


def _sincos(n):
    octant = n >> np.uint32(21)
    r = n & np.uint32(0x1FFFFF)
    r = np.where((octant & np.uint32(1)) == 1, np.uint32(0x200000) - r, r)
    a = (r.astype(np.float32) * _F(4.76837158e-07)) * _F(0.785398185)
    a2 = a * a
    ps = a2 * _F(2.75573188e-06) + _F(-1.98412701e-04)
    ps = a2 * ps + _F(8.33333377e-03)
    ps = a2 * ps + _F(-0.166666672)
    ps = a2 * ps + _F(1.0)
    s = a * ps
    pc = a2 * _F(-2.75573188e-07) + _F(2.48015876e-05)
    pc = a2 * pc + _F(-1.38888892e-03)
    pc = a2 * pc + _F(4.16666679e-02)
    pc = a2 * pc + _F(-0.5)
    c = a2 * pc + _F(1.0)
    swap = (((octant + np.uint32(1)) >> np.uint32(1)) & np.uint32(1)) == 1
    sv, cv = np.where(swap, c, s), np.where(swap, s, c)
    sn = np.where(octant >= 4, -sv, sv)
    cs = np.where((octant >= 2) & (octant <= 5), -cv, cv)
    return sn, cs


def _pair(w0, w1):
    k0 = (w0 >> np.uint64(9)).astype(np.uint32)
    k1 = (w1 >> np.uint64(9)).astype(np.uint32)
    u = (np.uint32(2) * k0 + np.uint32(1)).astype(np.float32) * _F(5.96046448e-08)
    radius = np.sqrt(_F(-2.0) * _log(u))
    sn, cs = _sincos(np.uint32(2) * k1 + np.uint32(1))
    return radius * cs, radius * sn


def standard_normal(seed: int, ordinal: int, n: int, start: int = 0) -> np.ndarray:
    """Elements ``start .. start + n - 1`` of tensor ``ordinal`` under ``seed`` (float32)."""
    if n <= 0:
        return np.zeros((0,), dtype=np.float32)
    first, last = start // 4, (start + n - 1) // 4
    out = np.empty(((last - first + 1) * 4,), dtype=np.float32)
    step = 1 << 20  # Philox blocks per pass: bounds the temporaries
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    with np.errstate(over="ignore"):
        for lo in range(first, last + 1, step):
            hi = min(lo + step, last + 1)
            b = np.arange(lo, hi, dtype=np.uint64)
            w = philox4x32_10(b & _MASK, b >> np.uint64(32), np.full_like(b, ordinal & 0xFFFFFFFF),
                              np.zeros_like(b), k0, k1)
            z0, z1 = _pair(w[0], w[1])
            z2, z3 = _pair(w[2], w[3])
            view = out[(lo - first) * 4:(hi - first) * 4].reshape(-1, 4)
            view[:, 0], view[:, 1], view[:, 2], view[:, 3] = z0, z1, z2, z3
    off = start - first * 4
    return out[off:off + n]


def normal(seed: int, ordinal: int, shape, std: float, mean: float = 0.0) -> np.ndarray:
    """``mean + std * z`` in float32 (one multiplication, one addition, each rounded once)."""
    n = int(np.prod(shape)) if len(shape) else 1
    z = standard_normal(seed, ordinal, n)
    return (_F(mean) + _F(std) * z).astype(np.float32).reshape(shape)
