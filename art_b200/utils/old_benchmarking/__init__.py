"""First-generation benchmark helpers that work from ``history.jsonl`` and the per-step trajectory files
(parity: reference ``src/art/utils/old_benchmarking/``)."""
from .calculate_step_metrics import calculate_step_std_dev
from .generate_comparison_table import generate_comparison_table
from .generate_line_graphs import generate_line_graphs
from .load_benchmarked_models import load_benchmarked_models
from .types import BenchmarkedModel, BenchmarkedModelKey, BenchmarkedModelStep

__all__ = ["BenchmarkedModel", "BenchmarkedModelKey", "BenchmarkedModelStep", "calculate_step_std_dev",
           "generate_comparison_table", "generate_line_graphs", "load_benchmarked_models"]
