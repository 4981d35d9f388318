"""Fedipel model family (model.py: configuration, weights, state; step.py: the step function)."""
from .model import Fedipel, FedipelArgs, fedipel_configs  # noqa: F401
