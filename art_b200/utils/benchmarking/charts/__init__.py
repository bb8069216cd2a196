"""Benchmark charts (parity: reference ``src/art/utils/benchmarking/charts/__init__.py``)."""
from .percentage_comparison_bar_chart import percentage_comparison_bar_chart
from .series import first_last, progress_series
from .training_progress_chart import training_progress_chart

__all__ = ["training_progress_chart", "percentage_comparison_bar_chart", "progress_series", "first_last"]
