"""Current step = largest numeric checkpoint directory (parity: reference
``src/art/utils/get_model_step.py:9-22``)."""
import os

from .output_dirs import get_model_dir


def get_step_from_dir(output_dir: str) -> int:
    os.makedirs(output_dir, exist_ok=True)
    steps = [int(d) for d in os.listdir(output_dir) if d.isdigit() and os.path.isdir(os.path.join(output_dir, d))]
    return max(steps, default=0)


def get_model_step(model, art_path: str) -> int:
    return get_step_from_dir(get_model_dir(model=model, art_path=art_path))
