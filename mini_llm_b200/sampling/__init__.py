"""Sampling parameters.

The draw itself happens on the device (``csrc/sampling_kernels.cu``): greedy
for ``temperature <= 0`` as in the reference's command line
(scripts/complete.py:116-123), else Gumbel-max over the nucleus ``top_p``.  A
request's randomness is (seed, number of tokens it has sampled so far): the
same request yields the same tokens in any batch.
"""

from __future__ import annotations

from dataclasses import dataclass

_M64 = (1 << 64) - 1


@dataclass
class SamplingParams:
    temperature: float = 0.0      # <= 0: greedy
    top_p: float = 1.0            # >= 1: no nucleus cut
    seed: int = 0
    counter: int = 0              # how many tokens this request has sampled so far


def request_seed(seed: int, index: int) -> int:
    """The seed of request ``index`` of a call that was given one ``seed``."""
    z = (int(seed) * 0x9E3779B97F4A7C15 + int(index) + 1) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return (z ^ (z >> 31)) & 0x7FFFFFFFFFFFFFFF
