"""Parallel runtime: topology / process groups, ZeRO/FSDP flat-buffer sharding, tensor / sequence / pipeline /
context / expert parallelism and the symmetric-memory fused collectives."""

from .manager import ProcessGroupManager, run_rank_n
from .topology import Topology
