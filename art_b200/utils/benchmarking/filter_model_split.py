"""Select the rows of one model/split (parity: reference ``filter_model_split.py``)."""
from .types import BenchmarkModelKey


def filter_rename_model_split(df, model: BenchmarkModelKey):
    out = df[(df["model"] == model.name) & (df["split"] == model.split)].copy()
    out["model"] = model.display_name
    return out
