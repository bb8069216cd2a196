"""Pack tokenised trajectories into fixed-length rows with prompt sharing (parity:
reference ``src/art/local/pack.py:13-205``).

Eight ``[num_rows, seq_len]`` tensors come out: ``tokens``, ``group_ids``, ``parent_ids``,
``input_pos`` (int64), ``assistant_mask`` (bool), ``logprobs``, ``advantages``, ``weights``
(float32).  A trajectory whose group prompt already sits in the current row contributes
only its completion; the attention mask derived from ``group_ids`` / ``parent_ids`` lets
that completion attend to the shared prompt and to itself but not to its siblings.
"""
from __future__ import annotations

import os
import random
from typing import TypedDict

import torch

from .tokenize import TokenizedResult

KEYS_DTYPES = {
    "tokens": torch.long, "group_ids": torch.long, "parent_ids": torch.long, "input_pos": torch.long,
    "assistant_mask": torch.bool, "logprobs": torch.float32, "advantages": torch.float32, "weights": torch.float32,
}
_PAD = {"tokens": None, "group_ids": -1, "parent_ids": -1, "input_pos": 0, "assistant_mask": 0,
        "logprobs": float("nan"), "advantages": 0.0, "weights": 0.0}


class PackedTensors(TypedDict):
    tokens: torch.Tensor
    group_ids: torch.Tensor
    parent_ids: torch.Tensor
    input_pos: torch.Tensor
    assistant_mask: torch.Tensor
    logprobs: torch.Tensor
    advantages: torch.Tensor
    weights: torch.Tensor


class DiskPackedTensors(TypedDict):
    dir: str
    num_sequences: int
    sequence_length: int


class _Row:
    __slots__ = tuple(KEYS_DTYPES)

    def __init__(self) -> None:
        for k in KEYS_DTYPES:
            setattr(self, k, [])

    def __len__(self) -> int:
        return len(self.tokens)

    def truncate(self, n: int) -> None:
        for k in KEYS_DTYPES:
            del getattr(self, k)[n:]


def packed_tensors_from_tokenized_results(tokenized_results: list[TokenizedResult], seq_len: int,
                                          pad_token_id: int = -100, truncate_long_results: bool = True,
                                          verbosity: int = 1, rng: random.Random | None = None) -> PackedTensors:
    rng = rng or random
    rows = [_Row()]
    for result in tokenized_results:
        if len(result.token_ids) > seq_len and not truncate_long_results:
            if verbosity > 1:
                print("Result is too long, skipping")
            continue
        tail = result.without_prompt()
        if sum(tail.assistant_mask) == 0:
            if verbosity > 1:
                print("Result has no unique completion tokens, skipping")
            continue
        row = rows[-1]
        shared = result.prompt_id in row.group_ids
        if len(row) + len(tail.token_ids if shared else result.token_ids) > seq_len:
            row = _Row()
            rows.append(row)
            shared = False
        piece = tail if shared else result
        n = len(piece.token_ids)
        completion_group = rng.randint(-(2 ** 63), 2 ** 63 - 1)
        row.tokens.extend(piece.token_ids)
        row.group_ids.extend([piece.prompt_id] * piece.prompt_length + [completion_group] * (n - piece.prompt_length))
        row.parent_ids.extend([piece.prompt_id] * n)
        row.input_pos.extend(piece.input_pos)
        row.assistant_mask.extend(piece.assistant_mask)
        row.logprobs.extend(piece.logprobs)
        row.advantages.extend([piece.advantage] * n)
        row.weights.extend([1.0 / (sum(piece.assistant_mask) + 1e-6)] * n)
        if truncate_long_results and len(row) > seq_len:
            if verbosity > 0:
                print(f"Packed row exceeds {seq_len} tokens; truncating {len(row) - seq_len} tokens")
            row.truncate(seq_len)
    order = list(range(len(rows)))
    rng.shuffle(order)
    rows = [rows[i] for i in order]

    def tensor(key: str) -> torch.Tensor:
        pad = pad_token_id if key == "tokens" else _PAD[key]
        data = [getattr(r, key) + [pad] * (seq_len - len(r)) for r in rows]
        return torch.tensor(data, dtype=KEYS_DTYPES[key]).reshape(len(rows), seq_len)

    mask = tensor("assistant_mask")
    weights = torch.where(mask, tensor("weights"), torch.zeros(()))
    if mask.any():
        weights[mask] /= weights[mask].mean()
    out = {k: tensor(k) for k in KEYS_DTYPES if k not in ("assistant_mask", "weights")}
    out["assistant_mask"] = mask
    out["weights"] = weights
    return out  # type: ignore[return-value]


def packed_tensors_from_dir(**kw) -> PackedTensors:
    """Open (creating if needed) the shared-mmap files ``{dir}/{key}.pt``."""
    os.makedirs(kw["dir"], exist_ok=True)
    n, s = kw["num_sequences"], kw["sequence_length"]
    return {k: torch.from_file(f"{kw['dir']}/{k}.pt", shared=True, size=n * s, dtype=dt).view(n, s)
            for k, dt in KEYS_DTYPES.items()}  # type: ignore[return-value]


def packed_tensors_to_dir(tensors: PackedTensors, dir: str) -> DiskPackedTensors:
    os.makedirs(dir, exist_ok=True)
    meta: DiskPackedTensors = {"dir": dir, "num_sequences": tensors["tokens"].shape[0],
                               "sequence_length": tensors["tokens"].shape[1]}
    for k, dst in packed_tensors_from_dir(**meta).items():
        dst.copy_(tensors[k])  # type: ignore[literal-required]
    return meta


class PackedDataset(torch.utils.data.Dataset):
    def __init__(self, **kw) -> None:
        self.tensors = packed_tensors_from_dir(**kw)

    def __len__(self) -> int:
        return self.tensors["tokens"].shape[0]

    def __getitem__(self, i: int) -> PackedTensors:
        return {k: v[i] for k, v in self.tensors.items()}  # type: ignore[return-value]


def plot_packed_tensors(packed_tensors: PackedTensors, path: str | None = None) -> None:
    """Eight heat-maps of the packed tensors (needs matplotlib; written to ``path`` if given)."""
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError as e:
        raise RuntimeError("plot_packed_tensors needs matplotlib, which is not installed") from e
    fig, axes = plt.subplots(4, 2, figsize=(15, 24))
    for ax, key in zip(axes.flat, KEYS_DTYPES):
        im = ax.imshow(packed_tensors[key].float().nan_to_num().numpy(), aspect="auto", cmap="viridis")  # type: ignore[literal-required]
        ax.set_title(key)
        ax.set_xlabel("Sequence Position")
        ax.set_ylabel("Batch")
        fig.colorbar(im, ax=ax)
    fig.tight_layout()
    if path:
        fig.savefig(path)
    else:
        plt.show()
