"""Select the rows of the given model/split keys and show them under their display names
(parity: reference ``src/art/utils/benchmarking/filter_model_split.py:6-32``; pandas frame)."""
from .types import BenchmarkModelKey


def filter_rename_model_split(df, models):
    """``models``: one :class:`BenchmarkModelKey` or a list of them."""
    keys = [models] if isinstance(models, BenchmarkModelKey) else list(models)
    keep = None
    for k in keys:
        hit = (df["model"] == k.name) & (df["split"] == k.split)
        keep = hit if keep is None else (keep | hit)
    if keep is None:
        return df.iloc[0:0].copy()
    out = df[keep].copy()
    for k in keys:
        if k.name != k.display_name:
            out.loc[(out["model"] == k.name) & (out["split"] == k.split), "model"] = k.display_name
    return out
