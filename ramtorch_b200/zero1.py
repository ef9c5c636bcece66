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

from ._native import trace as _trace
from ._shard_plan import ALIGN_BYTES, PARAM_IDS_KEY, ShardPlan, plan_for


class ZeroParamGroups(dict):
    """The ``rank -> groups`` dict, able to carry its flat shard plan (``.plan``)."""

    plan = None


def create_zero_param_groups(param_groups, world_size, *, balance="count"):
    """Assign whole parameters to ranks.

    Args:
        param_groups: list of group dicts in the PyTorch format, e.g.
            ``[{'params': norm_params, 'weight_decay': 0.0}, {'params': other_params}]``.
        world_size: number of ranks.
        balance: ``"count"`` (default) is the reference's assignment (zero1.py:56-62): parameter k
            of a group goes to rank ``k % world_size``.  ``"bytes"`` (an addition; the reference's
            docstring allows any hand-built dict of this shape, zero1.py:31-32) gives each
            parameter, largest first, to the rank that owns the fewest bytes so far over all
            groups -- ties go to the lowest rank, so every rank computes the same map.  Lists that
            mix 250 MiB matrices with 8 KiB vectors then end up with nearly equal flat segments:
            the round-robin by count leaves the largest segment 12 % above the mean for a
            Llama-shaped list on 8 ranks, which every rank pays for in the all-gather.

    Returns:
        dict ``rank -> list of group dicts`` (all ranks and all groups present, possibly with an
        empty ``params`` list); pass ``result[rank]`` to ``AdamW``.  A dict of the same shape built
        by hand with another assignment works everywhere this one does.

    Each returned group also carries ``rt_param_ids``: the position of its parameters in the
    global order (group by group, as given).  ``AdamW`` keys its stochastic-rounding stream by
    these ids, so a parameter sees the same random bits whatever the world size.
    """
    if balance not in ("count", "bytes"):
        raise ValueError("balance must be 'count' or 'bytes'")
    rank_param_groups = ZeroParamGroups((rank, []) for rank in range(world_size))
    owner_of = _owners_by_bytes(param_groups, world_size) if balance == "bytes" else None
    next_id = 0
    for group_idx, group in enumerate(param_groups):
        config = {k: v for k, v in group.items() if k != "params"}
        for rank in range(world_size):
            rank_param_groups[rank].append({"params": [], **config, PARAM_IDS_KEY: []})
        for k, param in enumerate(group["params"]):
            owner = k % world_size if owner_of is None else owner_of[next_id]
            target = rank_param_groups[owner][group_idx]
            target["params"].append(param)
            target[PARAM_IDS_KEY].append(next_id)     # global position: the same whatever the owner
            next_id += 1
    return rank_param_groups


def _owners_by_bytes(param_groups, world_size):
    """Greedy longest-first assignment: global parameter position -> owner rank.  Sizes are padded
    to the flat buffer's alignment, which is what a segment actually holds."""
    sizes = []
    for group in param_groups:
        for param in group["params"]:
            nbytes = param.numel() * param.element_size()
            sizes.append((nbytes + ALIGN_BYTES - 1) // ALIGN_BYTES * ALIGN_BYTES)
    load = [0] * world_size
    owner_of = [0] * len(sizes)
    for pos in sorted(range(len(sizes)), key=lambda i: (-sizes[i], i)):
        rank = min(range(world_size), key=lambda r: (load[r], r))
        owner_of[pos] = rank
        load[rank] += sizes[pos]
    return owner_of


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
    with _trace("rt.zero1.redistribute"), torch.no_grad():
        barrier_needed = False
        for bucket in plan.buckets.values():
            if _owners_pushed(plan, bucket, rank):
                barrier_needed = True          # values already sit in every rank's buffer
            else:
                mine = bucket.rank_segment(bucket.flat, rank)
                works.append(dist.all_gather_into_tensor(bucket.flat, mine, async_op=async_op))
            bucket.pushed = False
        for param, owner in plan.loose:
            works.append(dist.broadcast(param.data, src=owner, async_op=async_op))
        if barrier_needed and not works:
            # nothing else orders this rank's reads after the other ranks' kernels: a one-element
            # all-reduce on the same stream does (it completes only after every rank's launch has)
            works.append(dist.all_reduce(_token(plan), async_op=async_op))
        for work in works:
            if work is not None:
                work.wait()


_CHECKED_CALLS = 3


def _token(plan: ShardPlan) -> torch.Tensor:
    tok = getattr(plan, "_token", None)
    if tok is None:
        device = next(b.device for b in plan.buckets.values() if b.peer_ptrs is not None)
        tok = plan._token = torch.zeros(1, dtype=torch.int32, device=device)
    return tok


def _owners_pushed(plan: ShardPlan, bucket, rank: int) -> bool:
    """Whether this bucket's owners already stored their updated parameters into every rank's
    buffer (the fused path of ``AdamW.step``), so the all-gather can be skipped.

    All ranks must take the same branch.  During the first few calls the ranks agree through a
    tiny all-reduce (a rank that owns nothing in the bucket, or whose optimizer pushed, votes yes);
    after that the agreed mode is kept.  The very first call always gathers, which also makes
    ranks that started from different initial values consistent."""
    if bucket.peer_ptrs is None:
        return False
    if bucket.mode == "gather":
        return False
    owns = any(o == rank for o in bucket.owner)
    vote = bucket.pushed or not owns
    if bucket.mode == "push":
        if not vote:
            raise RuntimeError("ZeRO-1 fused redistribution was agreed on, but this rank's optimizer did not "
                               "store its updated parameters into the peers' buffers this step; use "
                               "ramtorch_b200.AdamW for every rank or set RT_ZERO_FUSED_PUSH=0")
        return True
    first = bucket.checks == 0
    bucket.checks += 1
    flag = torch.tensor([1 if vote else 0], dtype=torch.int32, device=bucket.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    agreed = bool(flag.item())
    if bucket.checks >= _CHECKED_CALLS:
        bucket.mode = "push" if agreed else "gather"
    return agreed and not first
