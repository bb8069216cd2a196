"""Deterministic epoch/batch iteration with resume
(parity: reference ``src/art/utils/iterate_dataset.py:9-80``)."""
from __future__ import annotations

import math
import random
from typing import Generator, Sequence, TypeVar

from tqdm.auto import tqdm

T = TypeVar("T")


def iterate_dataset(dataset: Sequence[T], groups_per_step: int = 1, num_epochs: int = 1,
                    initial_step: int = 0, use_tqdm: bool = True
                    ) -> Generator[tuple[list[T], int, int, int], None, None]:
    """Yield ``(batch, epoch, global_step, epoch_step)``.

    Each epoch visits the dataset in an order that depends only on the epoch number
    (a ``random.Random(epoch)`` shuffle), so a restarted run that passes the step it had
    reached as ``initial_step`` sees exactly the batches it has not consumed yet.
    """
    n = len(dataset)
    if n == 0:
        return
    per_epoch = math.ceil(n / groups_per_step)
    bar = tqdm(initial=initial_step, total=per_epoch * num_epochs, desc="Iterating dataset", unit="batch") if use_tqdm else None
    try:
        for epoch in range(num_epochs):
            order = list(range(n))
            random.Random(epoch).shuffle(order)
            for epoch_step in range(per_epoch):
                global_step = epoch * per_epoch + epoch_step
                if global_step < initial_step:
                    continue
                idx = order[epoch_step * groups_per_step:(epoch_step + 1) * groups_per_step]
                yield [dataset[i] for i in idx], epoch, global_step, epoch_step
                if bar is not None:
                    bar.update(1)
    finally:
        if bar is not None:
            bar.close()
