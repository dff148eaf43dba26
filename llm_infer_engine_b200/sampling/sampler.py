"""Token choice: greedy and temperature sampling with a top-p cut, in the reference's meaning
(src/sampler.py:4-33): temperature <= 0 is argmax; otherwise softmax(logits / T), drop tokens
once the probability mass before them (in falling order) exceeds top_p, renormalise, draw.
The draw runs on the device in float32 (`kernels/ops.sample`); the uniform number behind each
draw depends only on (seed, sequence id, how many tokens that sequence has drawn), so a
request's tokens do not depend on what it is batched with.
"""
from __future__ import annotations

from dataclasses import dataclass

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0      # the reference's CLI default: greedy (main.py:95)
    top_p: float = 1.0            # main.py:96
    seed: int = 0

    def __post_init__(self):
        if self.top_p < 0.0 or self.top_p > 1.0:
            object.__setattr__(self, "top_p", max(0.0, min(1.0, float(self.top_p))))   # sampler.py:12

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0


def _mix64(z: int) -> int:
    z &= _MASK
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & _MASK
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return z


def uniform_for(seed: int, seq_id: int, counter: int) -> float:
    """The uniform number in [0, 1) that the device sampler uses for the `counter`-th draw of
    sequence `seq_id` under `seed` (24 bits, exact in float32). Host twin of the kernel's generator."""
    x = _mix64((seed & _MASK) + _GOLDEN * (seq_id + 1))
    x = _mix64(x + _GOLDEN * (counter + 1))
    return (x >> 40) / 16777216.0
