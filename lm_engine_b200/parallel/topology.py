"""Pure rank arithmetic of the parallel layout (no torch.distributed needed, so it is unit-testable in one process).

Global rank = mixed-radix number over the axes ``(pp, dp, tp)`` with ``tp`` fastest.  The data-parallel axis is viewed
in three ways that all flatten to the same ``dp`` index, as in the reference (lm_engine/parallel/manager.py:161-253):

* ``(ddp, fsdp)``   replication x sharding of parameters (HSDP),
* ``(batch, cp)``   distinct batches x context-parallel ranks that share one batch (``cp`` inner),
* ``(edp, ep)``     expert-data-parallel x expert-parallel (``ep`` inner, an extension of this engine).
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Topology:
    world_size: int
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ddp: int = 1
    fsdp: int = 1
    ep: int = 1

    def __post_init__(self) -> None:
        if self.tp * self.pp * self.ddp * self.fsdp != self.world_size:
            raise AssertionError(f"tp({self.tp}) x pp({self.pp}) x ddp({self.ddp}) x fsdp({self.fsdp}) != "
                                 f"world size {self.world_size}")
        if self.dp % self.cp:
            raise AssertionError("context parallel size must divide the data parallel size")
        if self.dp % self.ep:
            raise AssertionError("expert parallel size must divide the data parallel size")

    @staticmethod
    def build(world_size: int, tp: int = 1, pp: int = 1, cp: int = 1, ddp: int | None = None,
              fsdp: int | None = None, zero_stage: int = 3, ep: int = 1) -> "Topology":
        if world_size % (tp * pp * cp):
            raise AssertionError("world size is not divisible by tp x pp x cp")
        dp = world_size // (tp * pp)
        if zero_stage == 0:
            assert fsdp in (None, 1), "ZeRO stage 0 does not shard"
            ddp, fsdp = dp, 1
        elif ddp is None:
            assert fsdp is None
            ddp, fsdp = 1, dp
        else:
            assert fsdp is not None and ddp * fsdp == dp, "zero_topology does not match the data parallel size"
        return Topology(world_size, tp, pp, cp, ddp, fsdp, ep)

    # ------------------------------------------------------------------ sizes
    @property
    def dp(self) -> int:
        return self.ddp * self.fsdp

    @property
    def batch(self) -> int:
        """number of distinct micro-batches per step = data-loading world size"""
        return self.dp // self.cp

    # ------------------------------------------------------------------ coordinates
    def coords(self, rank: int) -> dict[str, int]:
        tp_r = rank % self.tp
        dp_r = (rank // self.tp) % self.dp
        pp_r = rank // (self.tp * self.dp)
        return {"tp": tp_r, "dp": dp_r, "pp": pp_r, "ddp": dp_r // self.fsdp, "fsdp": dp_r % self.fsdp,
                "batch": dp_r // self.cp, "cp": dp_r % self.cp, "edp": dp_r // self.ep, "ep": dp_r % self.ep}

    def rank_of(self, pp: int, dp: int, tp: int) -> int:
        return (pp * self.dp + dp) * self.tp + tp

    # ------------------------------------------------------------------ groups (lists of global ranks)
    def _dp_subgroup(self, rank: int, members: list[int]) -> list[int]:
        c = self.coords(rank)
        return [self.rank_of(c["pp"], d, c["tp"]) for d in members]

    def group(self, axis: str, rank: int) -> list[int]:
        c = self.coords(rank)
        if axis == "tp":
            return [self.rank_of(c["pp"], c["dp"], t) for t in range(self.tp)]
        if axis == "pp":
            return [self.rank_of(p, c["dp"], c["tp"]) for p in range(self.pp)]
        if axis == "dp":
            return self._dp_subgroup(rank, list(range(self.dp)))
        if axis == "fsdp":
            return self._dp_subgroup(rank, [c["ddp"] * self.fsdp + f for f in range(self.fsdp)])
        if axis == "ddp":
            return self._dp_subgroup(rank, [d * self.fsdp + c["fsdp"] for d in range(self.ddp)])
        if axis == "cp":
            return self._dp_subgroup(rank, [c["batch"] * self.cp + k for k in range(self.cp)])
        if axis == "batch":
            return self._dp_subgroup(rank, [b * self.cp + c["cp"] for b in range(self.batch)])
        if axis == "ep":
            return self._dp_subgroup(rank, [c["edp"] * self.ep + e for e in range(self.ep)])
        if axis == "edp":
            return self._dp_subgroup(rank, [d * self.ep + c["ep"] for d in range(self.dp // self.ep)])
        raise KeyError(axis)

    def all_groups(self, axis: str) -> list[list[int]]:
        seen, out = set(), []
        for r in range(self.world_size):
            g = tuple(self.group(axis, r))
            if g not in seen:
                seen.add(g)
                out.append(list(g))
        return out

    def pipeline_stage_ids(self, pp_rank: int, num_stages: int) -> list[int]:
        """Round-robin stage placement: rank r owns stages r, r + pp, r + 2 pp, ...
        (lm_engine/parallel/pipeline_parallel.py:11-21)."""
        assert num_stages % self.pp == 0
        return [pp_rank + i * self.pp for i in range(num_stages // self.pp)]
