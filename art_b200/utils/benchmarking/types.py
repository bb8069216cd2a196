"""Model/split selector used by the benchmark loaders (parity: reference
``src/art/utils/benchmarking/types.py``)."""


class BenchmarkModelKey:
    def __init__(self, name: str, display_name: str | None = None, split: str | None = "val"):
        self.name = name
        self.display_name = display_name or name
        self.split = split

    def __str__(self) -> str:
        return self.display_name

    def __repr__(self) -> str:
        return f"BenchmarkModelKey({self.name!r}, {self.display_name!r}, {self.split!r})"
