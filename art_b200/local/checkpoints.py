"""Checkpoint directory housekeeping (parity: reference ``src/art/local/checkpoints.py:7-23``)."""
import os
import shutil

from ..utils.get_model_step import get_step_from_dir


def delete_checkpoints(output_dir: str, excluding: list[int]) -> list[int]:
    """Remove every numeric step directory not listed in ``excluding``; return what was removed."""
    removed = []
    for name in sorted(os.listdir(output_dir)):
        path = os.path.join(output_dir, name)
        if name.isdigit() and os.path.isdir(path) and int(name) not in excluding:
            shutil.rmtree(path)
            removed.append(int(name))
    return removed


def get_last_checkpoint_dir(output_dir: str) -> str | None:
    path = os.path.join(output_dir, f"{get_step_from_dir(output_dir):04d}")
    return path if os.path.exists(path) else None
