"""ZeRO-1: optimizer-state ownership and parameter redistribution — drop-in for ``ramtorch.zero1``.

``create_zero_param_groups`` returns the same ``rank -> [group, ...]`` dict as the reference
(ramtorch/zero1.py:5-64): every rank gets every group, parameter k of a group goes to rank
``k % world_size`` (restarting at rank 0 for each group), all other keys of the group are copied,
and the lists hold references to the caller's parameters.  ``broadcast_zero_params`` leaves every
rank holding the owners' values, like the reference (zero1.py:67-91), but does it with ONE in-place
NCCL all-gather per (device, dtype) over a flat, owner-ordered parameter buffer instead of one
broadcast per tensor.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ._shard_plan import ShardPlan, plan_for

PARAM_IDS_KEY = "rt_param_ids"


class ZeroParamGroups(dict):
    """The ``rank -> groups`` dict, able to carry its flat shard plan (``.plan``)."""

    plan = None


def create_zero_param_groups(param_groups, world_size):
    """Assign whole parameters to ranks, round-robin inside each group.

    Args:
        param_groups: list of group dicts in the PyTorch format, e.g.
            ``[{'params': norm_params, 'weight_decay': 0.0}, {'params': other_params}]``.
        world_size: number of ranks.

    Returns:
        dict ``rank -> list of group dicts`` (all ranks and all groups present, possibly with an
        empty ``params`` list); pass ``result[rank]`` to ``AdamW``.  A dict of the same shape built
        by hand with another assignment works everywhere this one does.

    Each returned group also carries ``rt_param_ids``: the position of its parameters in the
    global order (group by group, as given).  ``AdamW`` keys its stochastic-rounding stream by
    these ids, so a parameter sees the same random bits whatever the world size.
    """
    rank_param_groups = ZeroParamGroups((rank, []) for rank in range(world_size))
    next_id = 0
    for group_idx, group in enumerate(param_groups):
        config = {k: v for k, v in group.items() if k != "params"}
        for rank in range(world_size):
            rank_param_groups[rank].append({"params": [], **config, PARAM_IDS_KEY: []})
        for k, param in enumerate(group["params"]):
            target = rank_param_groups[k % world_size][group_idx]
            target["params"].append(param)
            target[PARAM_IDS_KEY].append(next_id)
            next_id += 1
    return rank_param_groups


def broadcast_zero_params(rank_param_groups, async_op=True):
    """Give every rank the owners' parameter values (call after ``optimizer.step()``).

    Parameters flagged ``is_ramtorch`` live in CPU storage shared by all workers and are skipped, as
    in the reference (zero1.py:81).  Returns ``None``; when it returns the collectives have been
    waited for (device work is ordered on the current stream)."""
    plan = plan_for(rank_param_groups)
    if not (dist.is_available() and dist.is_initialized()):
        if plan.world_size == 1:
            return
        raise RuntimeError("broadcast_zero_params needs an initialised torch.distributed process group")
    plan.verify_across_ranks()
    plan.flatten_params()
    if plan.world_size == 1:
        return
    rank = dist.get_rank()
    works = []
    with torch.no_grad():
        for bucket in plan.buckets.values():
            mine = bucket.rank_segment(bucket.flat, rank)
            works.append(dist.all_gather_into_tensor(bucket.flat, mine, async_op=async_op))
        for param, owner in plan.loose:
            works.append(dist.broadcast(param.data, src=owner, async_op=async_op))
        for work in works:
            if work is not None:
                work.wait()
