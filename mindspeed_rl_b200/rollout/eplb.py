"""Expert-parallel load balancer (EPLB): decide which experts get redundant replicas and where
every physical expert slot lives, from per-layer token statistics.

Three-stage hierarchical policy (the published DeepSeek EPLB scheme, which the reference ships in
``mindspeed_rl/workers/eplb/eplb.py:6-173``): (1) pack expert *groups* onto nodes so node loads
are even, (2) inside each node give the hottest experts extra replicas until all physical slots
are used, (3) pack the physical experts of a node onto its GPUs evenly.  When groups cannot be
split across nodes evenly the policy degenerates to one global group / one node.

``rebalance_experts(weight, num_replicas, num_groups, num_nodes, num_gpus)`` returns
``(phy2log [L, R], log2phy [L, E, max_rep] (-1 padded), logcnt [L, E])``.
"""
from __future__ import annotations

from typing import List, Tuple

import torch


def balanced_packing(weight: torch.Tensor, num_packs: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Longest-processing-time packing of ``n`` items into ``num_packs`` packs of equal item count.

    ``weight [X, n]`` -> ``(pack_index [X, n], rank_in_pack [X, n])``.
    """
    rows, n = weight.shape
    if n % num_packs:
        raise ValueError("the number of items must be divisible by the number of packs")
    cap = n // num_packs
    if cap == 1:
        return (torch.arange(n, dtype=torch.int64).expand(rows, n).clone(),
                torch.zeros(rows, n, dtype=torch.int64))
    w = weight.float().cpu()
    pack_index = torch.empty(rows, n, dtype=torch.int64)
    rank_in_pack = torch.empty(rows, n, dtype=torch.int64)
    for r in range(rows):
        load = [0.0] * num_packs
        fill = [0] * num_packs
        for item in torch.argsort(w[r], descending=True).tolist():
            best = min((p for p in range(num_packs) if fill[p] < cap), key=lambda p: load[p])
            pack_index[r, item] = best
            rank_in_pack[r, item] = fill[best]
            load[best] += float(w[r, item])
            fill[best] += 1
    return pack_index, rank_in_pack


def replicate_experts(weight: torch.Tensor, num_phy: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Give out ``num_phy - num_log`` extra replicas, always to the expert with the largest load
    per replica. Returns ``(phy2log [X, num_phy], rank [X, num_phy], logcnt [X, num_log])``."""
    rows, num_log = weight.shape
    if num_phy < num_log:
        raise ValueError("fewer physical slots than logical experts")
    w = weight.float()
    phy2log = torch.arange(num_phy, dtype=torch.int64).repeat(rows, 1)
    rank = torch.zeros(rows, num_phy, dtype=torch.int64)
    logcnt = torch.ones(rows, num_log, dtype=torch.int64)
    row_ids = torch.arange(rows)
    for slot in range(num_log, num_phy):
        hottest = (w / logcnt).argmax(dim=-1)
        phy2log[:, slot] = hottest
        rank[:, slot] = logcnt[row_ids, hottest]
        logcnt[row_ids, hottest] += 1
    return phy2log, rank, logcnt


def _inverse(perm: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(perm)
    inv.scatter_(1, perm, torch.arange(perm.size(1), dtype=torch.int64).expand_as(perm))
    return inv


def rebalance_experts_hierarchical(weight: torch.Tensor, num_physical_experts: int, num_groups: int,
                                   num_nodes: int, num_gpus: int):
    layers, num_log = weight.shape
    for a, b, what in ((num_log, num_groups, "experts / groups"), (num_groups, num_nodes, "groups / nodes"),
                       (num_gpus, num_nodes, "gpus / nodes"), (num_physical_experts, num_gpus, "slots / gpus")):
        if a % b:
            raise ValueError(f"{what}: {a} is not divisible by {b}")
    group_size = num_log // num_groups
    groups_per_node = num_groups // num_nodes
    slots_per_gpu = num_physical_experts // num_gpus
    # 1) groups -> nodes; "mlog" = logical experts renumbered so that a node's experts are contiguous
    group_load = weight.unflatten(-1, (num_groups, group_size)).sum(-1)
    g_pack, g_rank = balanced_packing(group_load, num_nodes)
    log2mlog = (((g_pack * groups_per_node + g_rank) * group_size).unsqueeze(-1)
                + torch.arange(group_size, dtype=torch.int64)).flatten(-2)
    mlog2log = _inverse(log2mlog)
    # 2) replicas inside every node
    node_load = weight.gather(-1, mlog2log).view(-1, num_log // num_nodes)
    phy2mlog, phyrank, mlogcnt = replicate_experts(node_load, num_physical_experts // num_nodes)
    # 3) physical experts of a node -> its GPUs
    phy_load = (node_load / mlogcnt).gather(-1, phy2mlog)
    p_pack, p_rank = balanced_packing(phy_load, num_gpus // num_nodes)
    phy2pphy = p_pack * slots_per_gpu + p_rank
    pphy2phy = _inverse(phy2pphy)
    pphy2mlog = phy2mlog.gather(-1, pphy2phy)
    node_base = torch.arange(0, num_log, num_log // num_nodes, dtype=torch.int64).view(1, -1, 1)
    pphy2mlog = (pphy2mlog.view(layers, num_nodes, -1) + node_base).flatten(-2)
    pphy2log = mlog2log.gather(-1, pphy2mlog)
    pphyrank = phyrank.gather(-1, pphy2phy).view(layers, -1)
    logcnt = mlogcnt.view(layers, -1).gather(-1, log2mlog)
    return pphy2log, pphyrank, logcnt


def rebalance_experts(weight: torch.Tensor, num_replicas: int, num_groups: int, num_nodes: int,
                      num_gpus: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    layers, num_log = weight.shape
    w = weight.float().cpu()
    if num_groups % num_nodes == 0:
        phy2log, phyrank, logcnt = rebalance_experts_hierarchical(w, num_replicas, num_groups, num_nodes, num_gpus)
    else:
        phy2log, phyrank, logcnt = rebalance_experts_hierarchical(w, num_replicas, 1, 1, num_gpus)
    max_rep = int(logcnt.max())
    log2phy = torch.full((layers, num_log, max_rep), -1, dtype=torch.int64)
    log2phy.view(layers, -1).scatter_(-1, phy2log * max_rep + phyrank,
                                      torch.arange(num_replicas, dtype=torch.int64).expand(layers, -1))
    return phy2log, log2phy, logcnt


def expert_map_from_counts(counts: torch.Tensor, num_gpus: int, num_redundancy_per_gpu: int = 1,
                           num_groups: int = 1, num_nodes: int = 1) -> dict:
    """Token statistics ``[L, E]`` -> the ``expert_map.json`` structure the rollout engine loads:
    per layer, per device, the list of logical expert ids hosted there (duplicates within a
    device are replaced by the device's least-replicated neighbour so a GPU never holds the same
    expert twice)."""
    layers, num_log = counts.shape
    num_phy = num_log + num_redundancy_per_gpu * num_gpus
    phy2log, _, _ = rebalance_experts(counts, num_phy, num_groups, num_nodes, num_gpus)
    per_gpu = num_phy // num_gpus
    if per_gpu > num_log:
        raise ValueError(f"{per_gpu} expert slots per device but only {num_log} experts: a device would have to "
                         f"host the same expert twice; lower num_redundancy_per_gpu or use more devices")
    layer_list = []
    for l in range(layers):
        devices = []
        for g in range(num_gpus):
            ids = phy2log[l, g * per_gpu:(g + 1) * per_gpu].tolist()
            seen, fixed = set(), []
            for e in ids:
                if e in seen:                      # de-duplicate inside a device
                    e = next(x for x in range(num_log) if x not in seen and x not in ids)
                seen.add(e)
                fixed.append(e)
            devices.append({"device_id": g, "device_expert": fixed})
        layer_list.append({"layer_id": l, "device_count": num_gpus, "device_list": devices})
    return {"moe_layer_count": layers, "layer_list": layer_list}
