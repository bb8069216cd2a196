"""Flatten a trajectory into plain chat messages (parity: reference
``src/art/utils/get_trajectory_messages.py``)."""
from ..trajectories import Trajectory
from ..types import Messages


def get_trajectory_messages(trajectory: Trajectory) -> Messages:
    return trajectory.messages()
