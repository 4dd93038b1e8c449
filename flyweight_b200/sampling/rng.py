"""The per-request random generator: xorshift64* with flyweight's constants
(native/src/v2_runtime.cpp:29307-29314; seeding at :32593-32596).  It runs on the host
-- one 64-bit update per sampled token -- and its uniform number is handed to the
sampling kernel, so a seeded request draws the same numbers whatever else is in the batch
and however often it was preempted."""
from __future__ import annotations

import time

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


class XorShift64Star:
    def __init__(self, seed=None, request_number: int = 0):
        if seed is None:
            seed = (time.monotonic_ns() ^ ((request_number * _GOLDEN) & _MASK)) & _MASK
        self.state = (int(seed) & _MASK) or _GOLDEN

    def uniform(self) -> float:
        value = self.state or _GOLDEN
        value ^= value >> 12
        value ^= (value << 25) & _MASK
        value ^= value >> 27
        self.state = value
        return (((value * 2685821657736338717) & _MASK) >> 11) * (1.0 / 9007199254740992.0)
