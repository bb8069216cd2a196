"""On-disk layout helpers (parity: reference ``src/art/utils/output_dirs.py:7-41``).

``{art_path}/{project}/models/{name}/`` holds ``model.json``, one ``{step:04d}/`` PEFT
adapter directory per step, ``trajectories/{split}/{step:04d}.yaml``, ``tensors/``,
``logs/`` and ``history.jsonl``.
"""
import os

from .get_repo_root_path import get_repo_root_path


def get_default_art_path() -> str:
    return os.path.join(get_repo_root_path(), ".art")


def get_models_dir(project_name: str, art_path: str | None = None) -> str:
    return f"{art_path or get_default_art_path()}/{project_name}/models"


def get_output_dir_from_model_properties(project: str, name: str, art_path: str | None = None) -> str:
    return f"{get_models_dir(project, art_path)}/{name}"


def get_model_dir(model, art_path: str | None = None) -> str:
    return get_output_dir_from_model_properties(model.project, model.name, art_path)


def get_step_checkpoint_dir(model_output_dir: str, step: int) -> str:
    return f"{model_output_dir}/{step:04d}"


def get_trajectories_dir(model_output_dir: str) -> str:
    return f"{model_output_dir}/trajectories"


def get_trajectories_split_dir(model_output_dir: str, split: str) -> str:
    return f"{model_output_dir}/trajectories/{split}"
