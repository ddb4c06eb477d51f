from .model import Model, resolve_dtype
from .step import Engine, GREEDY, SamplingParams, StepItem
from .generate import generate, plan_batches, should_stop

__all__ = ["Model", "resolve_dtype", "Engine", "GREEDY", "SamplingParams", "StepItem", "generate",
           "plan_batches", "should_stop"]
