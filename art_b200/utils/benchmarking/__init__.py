from .filter_model_split import filter_rename_model_split
from .load_trajectories import load_trajectories, load_trajectory_rows
from .types import BenchmarkModelKey

__all__ = ["BenchmarkModelKey", "filter_rename_model_split", "load_trajectories", "load_trajectory_rows"]
