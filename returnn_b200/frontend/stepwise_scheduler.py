"""
Step-wise schedulers.  Parity: returnn/frontend/stepwise_scheduler.py.
"""

from .piecewise_linear import PiecewiseLinearStepwiseScheduler

__all__ = ["PiecewiseLinearStepwiseScheduler"]
