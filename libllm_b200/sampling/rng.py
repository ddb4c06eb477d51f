"""Counter-based random numbers for sampling.

``uniform(seed, sequence, step)`` is a pure function: the draw for the n-th token of a
request does not depend on which other requests share its batch or on the slot it got.
The reference seeds one generator per process from the clock
(src/lutil/random.cc:28-31) or leaves cuRAND's default seed
(src/flint/cuda/cuda_operators.cc:274-276), so its draws cannot be replayed."""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    """The finalizer of SplitMix64."""
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, sequence: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits, exactly representable in float32."""
    h = _mix(seed & _MASK)
    h = _mix(h ^ (sequence & _MASK))
    h = _mix(h ^ (step & _MASK))
    return (h >> 40) / float(1 << 24)
