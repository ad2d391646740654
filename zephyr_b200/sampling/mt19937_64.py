"""The 64-bit Mersenne Twister (MT19937-64 of Matsumoto and Nishimura), the generator the reference
gives every sequence (``std::mt19937_64``, src/engine/engine.cpp:350-351).  Written from the
published recurrence; the C++ standard fixes its 10000th output for the default seed 5489 at
9981545732273789042, which the tests check."""

from __future__ import annotations

_NN, _MM = 312, 156
_MATRIX_A = 0xB5026F5AA96619E9
_UPPER, _LOWER = 0xFFFFFFFF80000000, 0x7FFFFFFF
_MASK = 0xFFFFFFFFFFFFFFFF


class MT19937_64:
    def __init__(self, seed: int = 5489):
        seed &= _MASK
        state = [0] * _NN
        state[0] = seed
        for i in range(1, _NN):
            prev = state[i - 1]
            state[i] = (6364136223846793005 * (prev ^ (prev >> 62)) + i) & _MASK
        self._state = state
        self._index = _NN

    def _refill(self) -> None:
        s = self._state
        for i in range(_NN):
            x = (s[i] & _UPPER) | (s[(i + 1) % _NN] & _LOWER)
            s[i] = s[(i + _MM) % _NN] ^ (x >> 1) ^ (_MATRIX_A if x & 1 else 0)
        self._index = 0

    def next_u64(self) -> int:
        if self._index >= _NN:
            self._refill()
        x = self._state[self._index]
        self._index += 1
        x ^= (x >> 29) & 0x5555555555555555
        x ^= (x << 17) & 0x71D67FFFEDA60000
        x ^= (x << 37) & 0xFFF7EEE000000000
        x ^= x >> 43
        return x & _MASK

    def next_uniform(self) -> float:
        """A float32-exact uniform number in [0, 1): the top 24 bits times 2^-24
        (reference: src/sampler/sampler.cpp:331)."""
        return float(self.next_u64() >> 40) * (2.0 ** -24)
