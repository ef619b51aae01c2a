"""Metrics and evaluator classes for in-loop evaluation."""

from .evaluator import Evaluator
from .lm_evaluator import LMEvaluator
from .metrics import MeanMetric, Metric

__all__ = ["Evaluator", "LMEvaluator", "Metric", "MeanMetric"]
