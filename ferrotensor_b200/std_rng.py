"""The random stream of the reference's sampler, restated.

The reference draws `rng.gen::<f32>()` from `rand::rngs::StdRng::seed_from_u64(seed)`
(ferrotensor-loader/src/tokenizer.rs:509-584; Cargo.lock pins rand 0.8.6, rand_chacha 0.3.1,
rand_core 0.6.4).  None of those crates is in the reference tree, so this file restates their
published algorithms:

* `StdRng` of rand 0.8 is `ChaCha12Rng`: the ChaCha block function (D. J. Bernstein's ChaCha,
  the quarter round and state layout of RFC 7539 section 2.3) with 12 rounds, a 256-bit key (the
  seed, little-endian words), a 64-bit block counter in words 12-13 starting at 0 and a 64-bit
  stream id in words 14-15 equal to 0.  Output words are consumed in block order; rand_chacha
  computes four blocks per refill, which does not change the word order.
* `SeedableRng::seed_from_u64` (rand_core 0.6): the 32 seed bytes are eight outputs of a PCG32
  generator (multiplier 6364136223846793005, increment 11634580027462260723; the state
  advances BEFORE each output; output = rotate_right(((s >> 18) ^ s) >> 27, s >> 59)), each
  stored little-endian.
* `Standard` for f32 (rand 0.8 `distributions/float.rs`): the top 24 bits of one `next_u32`
  times 2^-24, a value in [0, 1).

Pinned: the block function against the ChaCha20 block test vector of RFC 7539 section 2.3.2
(`tests/test_generate.py`), which fixes the quarter round, the round structure and the state
layout; the 12-round count, the seed expansion and the float conversion are restated from the
crates' documentation and sources as remembered, with no vector of the reference to hold them
against: for the sampled path parity stays unpinned.
"""

from __future__ import annotations

from typing import List

_MASK = 0xFFFFFFFF
_CONSTANTS = (0x61707865, 0x3320646E, 0x79622D32, 0x6B206574)     # "expand 32-byte k"


def _rotl(x: int, n: int) -> int:
    return ((x << n) | (x >> (32 - n))) & _MASK


def _quarter(s: List[int], a: int, b: int, c: int, d: int) -> None:
    s[a] = (s[a] + s[b]) & _MASK; s[d] = _rotl(s[d] ^ s[a], 16)
    s[c] = (s[c] + s[d]) & _MASK; s[b] = _rotl(s[b] ^ s[c], 12)
    s[a] = (s[a] + s[b]) & _MASK; s[d] = _rotl(s[d] ^ s[a], 8)
    s[c] = (s[c] + s[d]) & _MASK; s[b] = _rotl(s[b] ^ s[c], 7)


def chacha_block(key_words: List[int], tail_words: List[int], rounds: int) -> List[int]:
    """One 16-word ChaCha block: state = constants | 8 key words | 4 tail words (words 12-15:
    counter and nonce, or counter low/high and stream id low/high); `rounds` is even."""
    init = list(_CONSTANTS) + [w & _MASK for w in key_words] + [w & _MASK for w in tail_words]
    assert len(init) == 16 and rounds % 2 == 0
    s = list(init)
    for _ in range(rounds // 2):
        _quarter(s, 0, 4, 8, 12); _quarter(s, 1, 5, 9, 13); _quarter(s, 2, 6, 10, 14); _quarter(s, 3, 7, 11, 15)
        _quarter(s, 0, 5, 10, 15); _quarter(s, 1, 6, 11, 12); _quarter(s, 2, 7, 8, 13); _quarter(s, 3, 4, 9, 14)
    return [(a + b) & _MASK for a, b in zip(s, init)]


def seed_from_u64(state: int) -> bytes:
    """The 32-byte seed `SeedableRng::seed_from_u64` makes of a u64."""
    m64 = (1 << 64) - 1
    out = bytearray()
    state &= m64
    for _ in range(8):
        state = (state * 6364136223846793005 + 11634580027462260723) & m64
        xorshifted = (((state >> 18) ^ state) >> 27) & _MASK
        rot = state >> 59
        x = ((xorshifted >> rot) | (xorshifted << ((32 - rot) & 31))) & _MASK
        out += x.to_bytes(4, "little")
    return bytes(out)


class StdRng:
    """`rand::rngs::StdRng` (ChaCha12) seeded like `StdRng::seed_from_u64`."""

    ROUNDS = 12

    def __init__(self, seed32: bytes):
        assert len(seed32) == 32
        self.key = [int.from_bytes(seed32[4 * i:4 * i + 4], "little") for i in range(8)]
        self.counter = 0
        self.buf: List[int] = []

    @classmethod
    def seed_from_u64(cls, seed: int) -> "StdRng":
        return cls(seed_from_u64(seed))

    def next_u32(self) -> int:
        if not self.buf:
            c = self.counter
            self.buf = chacha_block(self.key, [c & _MASK, (c >> 32) & _MASK, 0, 0], self.ROUNDS)
            self.counter = (c + 1) & ((1 << 64) - 1)
        return self.buf.pop(0)

    def gen_f32(self) -> float:
        """`rng.gen::<f32>()`: 24 random bits scaled to [0, 1) (exact in f32)."""
        return (self.next_u32() >> 8) * (1.0 / (1 << 24))
