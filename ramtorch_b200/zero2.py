"""ZeRO-2: gradients reduced to their owners — drop-in for ``ramtorch.zero2``.

The reference registers, on every parameter of every rank's groups, a hook that issues
``dist.reduce(grad, dst=owner, SUM)`` per tensor per backward (ramtorch/zero2.py:27-57).  The
contract a training loop relies on is: after ``backward``, the owner's gradient of each parameter
it owns is the SUM over ranks.  Here that is delivered by ONE in-place NCCL ``reduce_scatter``
per (device, dtype) over a flat gradient buffer laid out like the ZeRO-1 parameter buffer:
``p.grad`` of every parameter is a view into it, autograd accumulates in place, and the
reduce-scatter is launched by the hook of the last gradient to arrive.

CPU-resident ``is_ramtorch`` parameters keep the reference's hook-dict protocol under the name
``_ramtorch_zero_2_hooks`` (zero2.py:67-72) with its synchronous per-tensor reduce, because their
gradients are produced and consumed tensor by tensor inside ``Linear``'s backward.
"""
from __future__ import annotations

import os
import weakref

import torch
import torch.distributed as dist

from ._native import trace as _trace
from ._shard_plan import Bucket, ShardPlan, plan_for
from .helpers import ZERO2_HOOK_NAME, register_ramtorch_hook

_ACTIVE_PLANS = weakref.WeakSet()


def _reduce_bucket(plan: ShardPlan, bucket: Bucket, rank: int) -> None:
    """Sum the flat gradient buffer across ranks into each owner's segment, then clear the
    segments this rank does not own so that a later micro-batch accumulates onto zeros there
    (which keeps gradient accumulation equal to the reference's reduce-every-backward)."""
    bucket.ready = 0
    written, bucket.grads_written = bucket.grads_written, False
    if plan.world_size == 1 or not dist.is_initialized():
        return
    if bucket.gpeer_ptrs is not None:
        # fused reduction: the optimizer kernel will read every rank's copy itself; all that is
        # needed here is that no rank starts reading before every rank has finished writing
        if written:
            dist.all_reduce(_barrier_token(bucket))
        return
    with _trace("rt.zero2.reduce_scatter"):
        mine = bucket.rank_segment(bucket.gflat, rank)
        work = dist.reduce_scatter_tensor(mine, bucket.gflat, op=dist.ReduceOp.SUM, async_op=True)
        work.wait()   # orders the current stream after the collective; the host does not block on NCCL
        lo, hi = rank * bucket.segment, (rank + 1) * bucket.segment
        bucket.gflat[:lo].zero_()
        bucket.gflat[hi:].zero_()


def _barrier_token(bucket: Bucket) -> torch.Tensor:
    tok = getattr(bucket, "_token", None)
    if tok is None:
        tok = bucket._token = torch.zeros(1, dtype=torch.int32, device=bucket.device)
    return tok


def finish_grad_sync() -> None:
    """Reduce any bucket that received only part of its gradients in the last backward (unused
    parameters).  ``AdamW.step`` calls this first; every rank must call it the same number of
    times, as with any collective."""
    for plan in list(_ACTIVE_PLANS):
        for bucket in plan.buckets.values():
            if bucket.gflat is not None and (bucket.ready > 0 or
                                             (bucket.gpeer_ptrs is not None and bucket.grads_written)):
                _reduce_bucket(plan, bucket, plan.current_rank)


def reduce_gradients_now(rank_param_groups) -> None:
    """Reduce-scatter every flat gradient buffer of this dict right away, whether or not all
    gradients have arrived (for loops that produce gradients outside autograd).  Collective:
    every rank must call it."""
    plan = plan_for(rank_param_groups)
    if plan.current_rank is None:
        raise RuntimeError("call setup_grad_sharding_hooks first")
    for bucket in plan.buckets.values():
        if bucket.gflat is not None:
            bucket.grads_written = True
            _reduce_bucket(plan, bucket, plan.current_rank)


def setup_grad_sharding_hooks(rank_param_groups, current_rank):
    """Register the gradient-reduction hooks for every parameter of every rank's groups.

    Args:
        rank_param_groups: dict from ``create_zero_param_groups`` (or hand-built, same shape).
        current_rank: this process's rank.

    Returns:
        list with one handle per parameter, ordered by (owner, group, parameter) like the
        reference: a ``RemovableHandle`` for ordinary parameters, the integer hook id for
        ``is_ramtorch`` parameters.
    """
    plan = plan_for(rank_param_groups)
    plan.current_rank = current_rank
    plan.verify_across_ranks()
    plan.flatten_params()
    # RT_ZERO2_FUSED_PULL=1: no reduce-scatter at all -- the owners' optimizer kernel sums the ranks'
    # gradient copies over NVLink while it updates (fp32 accumulation in rank order).  The owner's
    # p.grad then stays the LOCAL gradient; code that inspects reduced gradients between backward
    # and step (gradient clipping by global norm, logging) needs the default mode.
    plan.attach_grad_buffers(fused_pull=os.environ.get("RT_ZERO2_FUSED_PULL", "0") == "1")
    _ACTIVE_PLANS.add(plan)

    def make_flat_hook(bucket: Bucket, index: int):
        view = bucket.grad_views[index]

        def hook(param):
            grad = param.grad
            if grad is not view:
                # zero_grad(set_to_none=True) dropped the view and autograd installed a fresh
                # tensor: fold it back into the flat buffer
                if grad is not None and grad.data_ptr() != view.data_ptr():
                    view.copy_(grad)
                param.grad = view
            bucket.ready += 1
            bucket.grads_written = True
            if bucket.ready >= bucket.expected:
                if bucket.gpeer_ptrs is not None:
                    bucket.ready = 0          # fused reduction: the barrier waits for optimizer.step()
                else:
                    _reduce_bucket(plan, bucket, current_rank)

        return hook

    def make_tensor_hook(param):
        owner = plan.owner_of[id(param)]

        def hook(grad):
            dist.reduce(grad, dst=owner, op=dist.ReduceOp.SUM, async_op=False)
            return grad if current_rank == owner else None

        return hook

    index_in_bucket = {}
    for bucket in plan.buckets.values():
        for k, p in enumerate(bucket.params):
            index_in_bucket[id(p)] = (bucket, k)

    handles, registered = [], {}
    for owner in range(plan.world_size):
        for group in rank_param_groups[owner]:
            for param in group["params"]:
                if id(param) in registered:          # a tensor listed twice gets one hook
                    handles.append(registered[id(param)])
                    continue
                if getattr(param, "is_ramtorch", False):
                    handle = register_ramtorch_hook(param, make_tensor_hook(param), ZERO2_HOOK_NAME)
                elif id(param) in index_in_bucket:
                    bucket, k = index_in_bucket[id(param)]
                    handle = param.register_post_accumulate_grad_hook(make_flat_hook(bucket, k))
                else:
                    handle = param.register_hook(make_tensor_hook(param))
                registered[id(param)] = handle
                handles.append(handle)
    return handles
