"""The random-weights generator in plain numpy, operation for operation.

Element i of a tensor is a function of (key, i) alone (formulas: the header comment of
llm_b200/csrc/random_normal.h; the seeded fixture writer it stands in for is
scripts/make_tiny_moe.py:93-119 of MythEclipse/llm). Every step below is one correctly rounded
32-bit operation, as in the C++ and CUDA versions, so all three agree bit for bit.
Nothing in the llm_b200 package imports this file.
"""
import zlib

import numpy as np

F = np.float32


def tensor_key(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) & 0xFFFFFFFFFFFFFFFF


def mix(key: int, index: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = np.uint64(key) + (index.astype(np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return x


def log_unit(a: np.ndarray) -> np.ndarray:
    a = a.astype(np.uint32)
    shift = np.zeros_like(a)
    for _ in range(24):
        shift = shift + ((a << shift) < np.uint32(1 << 24)).astype(np.uint32)
    m = (a << shift).astype(F) * F(2.0 ** -24)
    e = -(shift.astype(F))
    s = (m + F(-1.0)) / (m + F(1.0))
    s2 = s * s
    p = np.full_like(s, F(1.0) / F(13.0))
    for d in (11.0, 9.0, 7.0, 5.0, 3.0):
        p = p * s2 + F(1.0) / F(d)
    p = p * s2 + F(1.0)
    ln_m = (F(2.0) * s) * p
    return e * F(0.693147182464599609375) + ln_m


def cos_sin(t: np.ndarray):
    t2 = t * t
    pc = np.full_like(t, F(-1.0) / F(87178291200.0))
    for c in (F(1.0) / F(479001600.0), F(-1.0) / F(3628800.0), F(1.0) / F(40320.0), F(-1.0) / F(720.0),
              F(1.0) / F(24.0), F(-0.5)):
        pc = pc * t2 + c
    cos = pc * t2 + F(1.0)
    ps = np.full_like(t, F(1.0) / F(6227020800.0))
    for c in (F(-1.0) / F(39916800.0), F(1.0) / F(362880.0), F(-1.0) / F(5040.0), F(1.0) / F(120.0),
              F(-1.0) / F(6.0), F(1.0)):
        ps = ps * t2 + c
    return cos, ps * t


def normal(key: int, n: int, mean: float, deviation: float) -> np.ndarray:
    """float32 [n]: mean + deviation * z(key, i)."""
    x = mix(key, np.arange(n, dtype=np.uint64))
    a = (x >> np.uint64(40)).astype(np.uint32) + np.uint32(1)
    quadrant = ((x >> np.uint64(38)) & np.uint64(3)).astype(np.int64)
    b = ((x >> np.uint64(16)) & np.uint64(0x3FFFFF)).astype(F)
    radius = np.sqrt(F(-2.0) * log_unit(a))
    t = ((b + F(0.5)) * F(2.0 ** -22)) * F(1.57079637050628662109375)
    c, s = cos_sin(t)
    direction = np.choose(quadrant, [c, -s, -c, s])
    z = radius * direction
    return (F(mean) + F(deviation) * z).astype(F)
