"""A normal-number generator that gives the same bits on every machine.

The random-weights mode has to produce one tensor set from (seed, tensor name), whether
the numbers are made by numpy on a host or by the kernel in `csrc/kernels/random_init.cu`
on the GPU, so that a model measured on the device can be rebuilt anywhere and compared
with a plain implementation.  Library generators cannot promise that (host and device
generators differ, and `log` / `cos` of different maths libraries differ in the last bit),
so everything here is built from operations that IEEE 754 defines exactly: 64-bit integer
arithmetic, and double-precision add, multiply, divide and square root, each written as
a separate step so that no compiler fuses two of them.

    key      = mix(FNV-1a(name) xor mix(seed + G))                     per tensor
    a, b     = mix(key + 2 i G), mix(key + (2 i + 1) G)                per element i
    u1, u2   = ((a >> 11) + 1) / 2^53  in (0, 1],   (b >> 11) / 2^53  in [0, 1)
    z        = sqrt(-2 ln u1) * cos(2 pi u2)                           Box-Muller
    value    = float32(z * std)   or   float32(1 + z * std)

`ln` and `cos` are the series below (atanh series after splitting off the exponent;
Taylor series after reducing to a quarter turn), accurate to a few units of 1e-16.
The device kernel restates the same steps in the same order.  The reference has no
counterpart; its test fixture fills weights with a counter (tests/qwen3_fixture.h:48-54).
"""
from __future__ import annotations

import numpy as np

_MASK = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB
LN2 = 0.6931471805599453
HALF_PI = 1.5707963267948966
SQRT_HALF = 0.7071067811865476
LN_TERMS = 11          # s^1 .. s^21
_FACTORIALS = [1.0]
for _i in range(1, 18):
    _FACTORIALS.append(_FACTORIALS[-1] * _i)


def mix64(x: int) -> int:
    x &= _MASK
    x ^= x >> 30
    x = (x * _M1) & _MASK
    x ^= x >> 27
    x = (x * _M2) & _MASK
    x ^= x >> 31
    return x


def tensor_key(seed: int, name: str) -> int:
    h = 0xCBF29CE484222325
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _MASK
    return mix64(h ^ mix64((seed + GOLDEN) & _MASK))


def _mix64_array(x: np.ndarray) -> np.ndarray:
    x = x ^ (x >> np.uint64(30))
    x = x * np.uint64(_M1)
    x = x ^ (x >> np.uint64(27))
    x = x * np.uint64(_M2)
    return x ^ (x >> np.uint64(31))


def _ln(u: np.ndarray) -> np.ndarray:
    m, e = np.frexp(u)                       # u = m 2^e, m in [0.5, 1)
    low = m < SQRT_HALF
    m = np.where(low, m * 2.0, m)            # now in [sqrt(1/2), sqrt(2))
    e = np.where(low, e - 1, e).astype(np.float64)
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    poly = np.full_like(s, 1.0 / (2 * LN_TERMS - 1))
    for k in range(LN_TERMS - 2, -1, -1):
        poly = poly * s2 + (1.0 / (2 * k + 1))
    return e * LN2 + (2.0 * s) * poly


def _cos_turns(t: np.ndarray) -> np.ndarray:
    """cos(2 pi t) for t in [0, 1)."""
    a = t * 4.0
    j = np.floor(a + 0.5)
    theta = (a - j) * HALF_PI                # in [-pi/4, pi/4]
    t2 = theta * theta
    c = np.full_like(t, 1.0 / _FACTORIALS[16])
    for k in range(7, 0, -1):
        c = c * t2 + ((1.0 if k % 2 == 0 else -1.0) / _FACTORIALS[2 * k])
    c = c * t2 + 1.0
    s = np.full_like(t, 1.0 / _FACTORIALS[17])
    for k in range(7, 0, -1):
        s = s * t2 + ((1.0 if k % 2 == 0 else -1.0) / _FACTORIALS[2 * k + 1])
    s = (s * t2 + 1.0) * theta
    quarter = j.astype(np.int64) & 3
    return np.where(quarter == 0, c, np.where(quarter == 1, -s, np.where(quarter == 2, -c, s)))


def normal_float32(seed: int, name: str, count: int, std: float, one_plus: bool = False,
                   chunk: int = 1 << 20) -> np.ndarray:
    """`count` float32 numbers of tensor `name`: N(0, std^2), or 1 + N(0, std^2)."""
    key = np.uint64(tensor_key(seed, name))
    out = np.empty(count, dtype=np.float32)
    golden = np.uint64(GOLDEN)
    with np.errstate(over="ignore"):
        for first in range(0, count, chunk):
            i = np.arange(first, min(first + chunk, count), dtype=np.uint64)
            c = key + (i * np.uint64(2)) * golden
            a = _mix64_array(c)
            b = _mix64_array(c + golden)
            u1 = ((a >> np.uint64(11)) + np.uint64(1)).astype(np.float64) * 2.0 ** -53
            u2 = (b >> np.uint64(11)).astype(np.float64) * 2.0 ** -53
            z = np.sqrt(-2.0 * _ln(u1)) * _cos_turns(u2)
            v = z * float(std)
            if one_plus:
                v = v + 1.0
            out[first:first + len(i)] = v.astype(np.float32)
    return out
