"""The generator the reference draws from: java.util.Random.

A 48-bit linear congruential generator; ``nextFloat()`` is its top 24 bits over
2^24. The reference makes one per request from the sampler's seed and takes one
float per sampled token (sampler/CompositeSampler.java:24, :387-395), so a
sequence's draws depend on its seed alone, never on what else is in the batch.
"""

_MULT = 0x5DEECE66D
_MASK = (1 << 48) - 1


class JavaRandom:
    def __init__(self, seed: int):
        self._state = (int(seed) ^ _MULT) & _MASK

    def _next(self, bits: int) -> int:
        self._state = (self._state * _MULT + 0xB) & _MASK
        return self._state >> (48 - bits)

    def next_float(self) -> float:
        return self._next(24) / float(1 << 24)
