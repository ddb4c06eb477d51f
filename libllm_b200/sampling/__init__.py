from .rng import uniform

__all__ = ["uniform"]
