from .optimizer import BaseOptimizer, DefaultOptimizer, OptimizerRegistry  # noqa: F401
