"""Device mesh: process groups for every parallel dimension.

Rank order is tensor-parallel fastest, then context-parallel, data-parallel, pipeline-parallel
slowest (Megatron's ``tp-cp-dp-pp`` order, so a tensor-parallel group sits on adjacent GPUs of one
NVSwitch domain); expert-parallel groups are blocks of consecutive data-parallel ranks
(``ep`` divides ``dp``), as the reference's Megatron configs carve them
(small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:96-98;
llama2_sft/primus/conf/llama2_70b_lora_posttrain.yaml:18-23).  ``dp_replicate`` splits the
data-parallel dimension into replicate x shard for hybrid-sharded data parallel
(flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:48-49).

Every rank creates every group (``new_group`` is collective); a size-1 dimension gets a group of
the rank alone so callers need no special cases.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch.distributed as dist


@dataclass
class MeshSpec:
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    dp_replicate: int = 1

    def dp(self, world: int) -> int:
        denom = self.tp * self.pp * self.cp
        if world % denom:
            raise ValueError(f"world size {world} is not divisible by tp*pp*cp = {denom}")
        return world // denom


def coords(rank: int, spec: MeshSpec, world: int) -> dict:
    dp = spec.dp(world)
    t = rank % spec.tp
    c = (rank // spec.tp) % spec.cp
    d = (rank // (spec.tp * spec.cp)) % dp
    p = rank // (spec.tp * spec.cp * dp)
    return {"tp": t, "cp": c, "dp": d, "pp": p}


def group_ranks(spec: MeshSpec, world: int) -> dict[str, list[list[int]]]:
    """All groups of every dimension, as lists of global ranks (pure arithmetic, no communication)."""
    dp = spec.dp(world)
    if dp % spec.ep:
        raise ValueError(f"expert-parallel size {spec.ep} does not divide the data-parallel size {dp}")
    if dp % spec.dp_replicate:
        raise ValueError(f"dp_replicate {spec.dp_replicate} does not divide the data-parallel size {dp}")

    def rank_of(t, c, d, p):
        return ((p * dp + d) * spec.cp + c) * spec.tp + t

    out = {"tp": [], "cp": [], "dp": [], "pp": [], "ep": [], "edp": [], "dp_shard": [], "dp_replicate": [], "dp_cp": [], "edp_cp": []}
    for p in range(spec.pp):
        for d in range(dp):
            for c in range(spec.cp):
                out["tp"].append([rank_of(t, c, d, p) for t in range(spec.tp)])
            for t in range(spec.tp):
                out["cp"].append([rank_of(t, c, d, p) for c in range(spec.cp)])
        for c in range(spec.cp):
            for t in range(spec.tp):
                out["dp"].append([rank_of(t, c, d, p) for d in range(dp)])
                for e0 in range(0, dp, spec.ep):
                    out["ep"].append([rank_of(t, c, d, p) for d in range(e0, e0 + spec.ep)])
                # expert data parallel: the ranks that hold the same experts (same position in their ep block)
                for e in range(spec.ep):
                    out["edp"].append([rank_of(t, c, d, p) for d in range(e, dp, spec.ep)])
                shard = dp // spec.dp_replicate
                for r in range(spec.dp_replicate):
                    out["dp_shard"].append([rank_of(t, c, d, p) for d in range(r * shard, (r + 1) * shard)])
                for s in range(shard):
                    out["dp_replicate"].append([rank_of(t, c, r * shard + s, p) for r in range(spec.dp_replicate)])
    for d in range(dp):
        for c in range(spec.cp):
            for t in range(spec.tp):
                out["pp"].append([rank_of(t, c, d, p) for p in range(spec.pp)])
    # every rank that holds a replica of the same parameters: data x context (the gradient-reduction group)
    for p in range(spec.pp):
        for t in range(spec.tp):
            out["dp_cp"].append([rank_of(t, c, d, p) for d in range(dp) for c in range(spec.cp)])
            # ... and of the same experts: the same position in the expert-parallel blocks, every context chunk
            for e in range(spec.ep):
                out["edp_cp"].append([rank_of(t, c, d, p) for d in range(e, dp, spec.ep) for c in range(spec.cp)])
    return out


class Mesh:
    def __init__(self, spec: MeshSpec):
        if not dist.is_initialized():
            raise RuntimeError("initialise torch.distributed before building a mesh")
        self.spec = spec
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.coords = coords(self.rank, spec, self.world)
        self.groups: dict[str, dist.ProcessGroup] = {}
        self.ranks: dict[str, list[int]] = {}
        for dim, lists in group_ranks(spec, self.world).items():
            for ranks in lists:
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.groups[dim], self.ranks[dim] = g, ranks

    def group(self, dim: str) -> dist.ProcessGroup:
        return self.groups[dim]

    def size(self, dim: str) -> int:
        return len(self.ranks[dim])

    def index(self, dim: str) -> int:
        return self.ranks[dim].index(self.rank)

    def prev_next_stage(self) -> tuple[int | None, int | None]:
        """Global ranks of the previous / next pipeline stage (None at the ends)."""
        r, i = self.ranks["pp"], self.index("pp")
        return (r[i - 1] if i > 0 else None), (r[i + 1] if i + 1 < len(r) else None)
