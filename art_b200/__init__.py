"""B200-native agent reinforcement trainer with the public surface of OpenPipe/ART.

Public API parity: reference ``src/art/__init__.py:13-37``.
"""
from . import dev
from .backend import Backend
from .batches import trajectory_group_batches
from .gather import gather_trajectories, gather_trajectory_groups
from .model import Model, TrainableModel
from .trajectories import Trajectory, TrajectoryGroup
from .types import Messages, MessagesAndChoices, Tools, TrainConfig
from .utils import retry

__version__ = "0.1.0"

__all__ = [
    "dev", "gather_trajectories", "gather_trajectory_groups", "trajectory_group_batches", "Backend",
    "Messages", "MessagesAndChoices", "Tools", "Model", "TrainableModel", "retry", "TrainConfig",
    "Trajectory", "TrajectoryGroup",
]
