"""Records of the first-generation benchmark loader (parity: reference
``src/art/utils/old_benchmarking/types.py:3-44``)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class BenchmarkedModelKey:
    model: str
    split: str
    step_indices: list[int] | None = None     # None: every logged step; negative entries count from the last step

    def __str__(self) -> str:
        steps = ""
        if self.step_indices:
            steps = (f"{self.step_indices[0]}" if len(self.step_indices) == 1
                     else f"{self.step_indices[0]}-{self.step_indices[-1]}")
        return f"{self.model} {self.split} {steps}"


@dataclass
class BenchmarkedModelStep:
    index: int
    metrics: dict[str, float] = field(default_factory=dict)
    recorded_at: str | None = None

    def __str__(self) -> str:
        return f"{self.index} {self.metrics}"


@dataclass
class BenchmarkedModel:
    model_key: BenchmarkedModelKey
    steps: list[BenchmarkedModelStep] = field(default_factory=list)

    def __str__(self) -> str:
        return "\n".join([str(self.model_key)] + [str(s) for s in self.steps])
