"""Rank layout of a job that combines several kinds of parallelism on one NVSwitch domain.

``ParallelLayout(world, tp=2, cp=1, pp=1)`` factors the ranks as ``dp x pp x cp x tp`` with tensor parallelism
innermost: the ranks of a TP group are consecutive (they exchange activations in every layer), then context
parallelism (K/V once per layer), then pipeline stages (one activation per micro-batch), and data parallelism
outermost (one gradient message per step).  Expert parallelism reuses ranks instead of multiplying them: an EP
group is ``ep`` consecutive ranks of the flattened ``dp x cp x tp`` ranks of one pipeline stage, as MoE layers
shard experts over ranks that are data-parallel for the dense layers.

``groups()`` lists the member ranks of every group of every axis; ``create_groups()`` creates them with
``torch.distributed.new_group`` -- every rank creates every group, in the same order, as the collective
libraries require -- and returns this rank's group per axis.

The reference is single-GPU (its only multi-GPU knob is the inference library's ``tensor_parallel_size``,
src/art/dev/engine.py); this is the bookkeeping a TP x CP x EP x DP trainer needs on top of it.
"""
from __future__ import annotations

from dataclasses import dataclass

AXES = ("dp", "pp", "cp", "tp")


@dataclass(frozen=True)
class ParallelLayout:
    world: int
    tp: int = 1
    cp: int = 1
    pp: int = 1
    ep: int = 1

    def __post_init__(self):
        inner = self.tp * self.cp * self.pp
        if min(self.tp, self.cp, self.pp, self.ep, self.world) < 1 or self.world % inner:
            raise ValueError(f"world={self.world} is not a multiple of tp*cp*pp={inner}")
        per_stage = self.world // self.pp
        if per_stage % self.ep:
            raise ValueError(f"ep={self.ep} does not divide the {per_stage} ranks of a pipeline stage")

    @property
    def dp(self) -> int:
        return self.world // (self.tp * self.cp * self.pp)

    def size(self, axis: str) -> int:
        return self.dp if axis == "dp" else getattr(self, axis)

    def coords(self, rank: int) -> dict[str, int]:
        """``rank == ((dp * PP + pp) * CP + cp) * TP + tp``."""
        if not 0 <= rank < self.world:
            raise ValueError(f"rank {rank} outside 0..{self.world - 1}")
        tp = rank % self.tp
        cp = rank // self.tp % self.cp
        pp = rank // (self.tp * self.cp) % self.pp
        return {"dp": rank // (self.tp * self.cp * self.pp), "pp": pp, "cp": cp, "tp": tp}

    def rank_of(self, dp: int = 0, pp: int = 0, cp: int = 0, tp: int = 0) -> int:
        return ((dp * self.pp + pp) * self.cp + cp) * self.tp + tp

    def group_ranks(self, axis: str, rank: int) -> list[int]:
        """Members of ``rank``'s group along ``axis`` (all other coordinates fixed), in axis order."""
        if axis == "ep":
            stage = self._stage_ranks(self.coords(rank)["pp"])
            i = stage.index(rank) // self.ep * self.ep
            return stage[i:i + self.ep]
        c = self.coords(rank)
        out = []
        for k in range(self.size(axis)):
            out.append(self.rank_of(**{**c, axis: k}))
        return out

    def _stage_ranks(self, pp: int) -> list[int]:
        return [r for r in range(self.world) if self.coords(r)["pp"] == pp]

    def groups(self) -> dict[str, list[list[int]]]:
        """Every group of every axis (axes of size 1 included, as singleton groups), each listed once."""
        out: dict[str, list[list[int]]] = {}
        for axis in AXES + ("ep",):
            seen, lst = set(), []
            for r in range(self.world):
                g = tuple(self.group_ranks(axis, r))
                if g not in seen:
                    seen.add(g)
                    lst.append(list(g))
            out[axis] = lst
        return out

    def data_shard(self, rank: int) -> tuple[int, int]:
        """(index, count) of the distinct data streams: ranks that differ only in tp / cp / pp see the same rows."""
        return self.coords(rank)["dp"], self.dp

    def create_groups(self, rank: int | None = None, backend: str | None = None) -> dict[str, object]:
        """Create every group (same order on every rank); returns ``{axis: this rank's group or None}``.

        Axes of size 1 get ``None`` (callers skip the collective)."""
        import torch.distributed as dist

        rank = dist.get_rank() if rank is None else rank
        mine: dict[str, object] = {}
        for axis, lst in self.groups().items():
            mine[axis] = None
            if len(lst[0]) == 1:
                continue
            for members in lst:
                g = dist.new_group(members, backend=backend)
                if rank in members:
                    mine[axis] = g
        return mine
