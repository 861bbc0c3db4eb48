"""Which ranks of the job run which role.

The reference places every role (actor, reference, reward, critic, vision tower) on its own Ray
placement group when the roles are *disaggregated*, or packs them onto the actor's devices when
they are *co-located* (``mindspeed_rl/workers/scheduler/launcher.py:80-123``,
``config_cls/rl_config.py:132-136``: ``actor_resource`` / ``reference_resource`` /
``reward_resource`` / ``critic_resource`` / ``vit_resource``).  Here a job is one ``torchrun``
world, so a placement is a contiguous range of global ranks per role:

* co-located (``use_integrated_worker``, or a role without a resource entry): the role shares the
  actor's ranks and the roles time-share each GPU;
* disaggregated: the actor takes ranks ``[0, A)``, then reference, reward, critic and vision
  tower follow in that order, each with the ``num_gpus`` of its resource entry.  Ranges never
  straddle more nodes than they must: a role that fits on one node is not split over two.

A rank outside a role's range skips that role's stages, so stages of roles on disjoint ranks
run concurrently (reference forward on its GPUs while the actor computes old log-probs on its
own); the experience store orders the data dependencies between them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

ROLES = ("actor", "reference", "reward", "critic", "vit")


def _gpus(resource) -> int:
    if not resource:
        return 0
    return int(resource.get("num_gpus", resource.get("num_npus", 0)) or 0)


@dataclass
class Placement:
    world_size: int
    ranks: Dict[str, List[int]] = field(default_factory=dict)

    def of(self, role: str) -> List[int]:
        return self.ranks.get(role, self.ranks["actor"])

    def offset(self, role: str) -> int:
        return self.of(role)[0]

    def contains(self, role: str, rank: int) -> bool:
        return rank in self.of(role)

    def colocated(self, a: str, b: str) -> bool:
        return self.of(a) == self.of(b)

    def disjoint_roles(self) -> bool:
        """True when at least two roles live on different ranks (stages can overlap)."""
        sets = {tuple(v) for v in self.ranks.values()}
        return len(sets) > 1


def plan_placement(world_size: int, rl_config, gpus_per_node: Optional[int] = None,
                   roles=ROLES) -> Placement:
    """Rank ranges of the roles of one job (see the module docstring)."""
    actor = _gpus(getattr(rl_config, "actor_resource", None)) or world_size
    if actor > world_size:
        raise ValueError(f"actor_resource asks for {actor} GPUs but the job has {world_size}")
    plan = Placement(world_size, {"actor": list(range(actor))})
    if getattr(rl_config, "use_integrated_worker", False):
        return plan                                   # every role on the actor's ranks
    cursor = actor
    node = gpus_per_node or world_size
    for role in roles[1:]:
        n = _gpus(getattr(rl_config, f"{role}_resource", None))
        if role == "vit" and getattr(rl_config, "colocate_actor_and_vit", False):
            n = 0
        if n == 0:
            continue                                  # no entry: shares the actor's ranks
        if n <= node and cursor // node != (cursor + n - 1) // node:
            cursor = (cursor // node + 1) * node      # keep a role that fits on one node on one node
        if cursor + n > world_size:
            raise ValueError(f"{role}_resource asks for {n} GPUs starting at rank {cursor}, but the job has "
                             f"{world_size} ranks (actor uses {actor})")
        plan.ranks[role] = list(range(cursor, cursor + n))
        cursor += n
    return plan
