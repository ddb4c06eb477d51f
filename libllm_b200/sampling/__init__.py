"""Counter-based random numbers for sampling (sampling/rng.h, in the host library)."""
from .. import _lib


def uniform(seed: int, sequence: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits, a pure function of its arguments."""
    m = (1 << 64) - 1
    return float(_lib.lib().llm_uniform(seed & m, sequence & m, step & m))


__all__ = ["uniform"]
