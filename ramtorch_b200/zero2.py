"""ZeRO-2: gradients reduced to their owners — drop-in for ``ramtorch.zero2``.

The reference registers, on every parameter of every rank's groups, a hook that issues
``dist.reduce(grad, dst=owner, SUM)`` per tensor per backward (ramtorch/zero2.py:27-57).  The
contract a training loop relies on is: after ``backward``, the owner's gradient of each parameter
it owns is the SUM over ranks.  Here that is delivered by in-place NCCL ``reduce_scatter``s over a
flat gradient buffer per (device, dtype): ``p.grad`` of every parameter is a view into it and
autograd accumulates in place.  The buffer is cut into pieces of about 512 MiB in the order in
which backward completes them; the hook of the last gradient of a piece launches that piece's
reduce-scatter at once, so the reduction overlaps the rest of backward (as the reference's
per-tensor reduce does) while still moving a few large messages instead of one per tensor.

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


def _launch_piece(plan: ShardPlan, bucket: Bucket, sub, rank: int) -> None:
    """Start the reduce-scatter of one complete piece of the flat gradient buffer.  NCCL runs it on
    its own stream, ordered after what the current stream has written so far, so the rest of
    backward overlaps it; nothing waits here."""
    sub.ready = 0
    region = bucket.gflat[sub.start:sub.start + sub.part * plan.world_size]
    mine = region[rank * sub.part:(rank + 1) * sub.part]
    with _trace("rt.zero2.reduce_scatter"):
        sub.work = dist.reduce_scatter_tensor(mine, region, op=dist.ReduceOp.SUM, async_op=True)
    # The parts this rank does not own are cleared again, so that a later micro-batch accumulates
    # onto zeros there (which keeps gradient accumulation equal to the reference's
    # reduce-every-backward).  That pass runs on a side stream behind the collective, off the
    # critical path; only _finish_pieces makes anyone wait for it.
    if bucket.side is None:
        bucket.side = torch.cuda.Stream(bucket.device) if bucket.device.type == "cuda" else False
    if bucket.side:
        with torch.cuda.stream(bucket.side):
            sub.work.wait()
            _clear_others(region, sub.part, rank)
            sub.zeroed = torch.cuda.Event()
            sub.zeroed.record()
            region.record_stream(bucket.side)
    else:                                   # CPU tensors (gloo): no streams, the collective has to finish first
        sub.work.wait()
        sub.work = None
        _clear_others(region, sub.part, rank)


def _clear_others(region: torch.Tensor, part: int, rank: int) -> None:
    region[:rank * part].zero_()
    region[(rank + 1) * part:].zero_()


def _finish_pieces(bucket: Bucket) -> None:
    """Order the current stream after every reduce-scatter (and clearing pass) started so far."""
    for sub in bucket.subs:
        if sub.work is not None:
            sub.work.wait()       # stream-level wait; the host does not block on NCCL
            sub.work = None
        if sub.zeroed is not None:
            torch.cuda.current_stream(bucket.device).wait_event(sub.zeroed)
            sub.zeroed = None


def _reduce_bucket(plan: ShardPlan, bucket: Bucket, rank: int, only_started: bool = False) -> None:
    """Sum the flat gradient buffer across ranks into each owner's parts: every piece that has not
    been reduced since its gradients arrived is reduced now, then the current stream is ordered
    after all of them.  ``only_started``: reduce only pieces that received at least one gradient."""
    bucket.ready = 0
    written, bucket.grads_written = bucket.grads_written, False
    if plan.world_size == 1 or not dist.is_initialized():
        for sub in bucket.subs:
            sub.ready = 0
        return
    if bucket.gpeer_ptrs is not None:
        # fused reduction: the optimizer kernel will read every rank's copy itself; all that is
        # needed here is that no rank starts reading before every rank has finished writing
        for sub in bucket.subs:
            sub.ready = 0
        if written:
            dist.all_reduce(_barrier_token(bucket))
        return
    for sub in bucket.subs:
        if sub.work is None and (sub.ready > 0 or not only_started):
            _launch_piece(plan, bucket, sub, rank)
    _finish_pieces(bucket)


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
            if bucket.gflat is None:
                continue
            pending = any(sub.work is not None or sub.zeroed is not None for sub in bucket.subs)
            if bucket.ready > 0 or (bucket.gpeer_ptrs is not None and bucket.grads_written):
                # a partial backward (unused parameters): every rank reduces every piece, so that the
                # collectives stay matched whatever each rank's autograd graph touched
                _reduce_bucket(plan, bucket, plan.current_rank)
            elif pending:
                _finish_pieces(bucket)


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
        sub = bucket.subs[bucket.sub_of[index]]

        def hook(param):
            grad = param.grad
            if grad is not view:
                # zero_grad(set_to_none=True) dropped the view and autograd installed a fresh
                # tensor: fold it back into the flat buffer
                if grad is not None and grad.data_ptr() != view.data_ptr():
                    view.copy_(grad)
                param.grad = view
            bucket.ready += 1
            sub.ready += 1
            bucket.grads_written = True
            fused = bucket.gpeer_ptrs is not None
            distributed = plan.world_size > 1 and dist.is_initialized()
            if not fused and distributed and sub.ready >= sub.expected and sub.work is None:
                _launch_piece(plan, bucket, sub, current_rank)     # overlaps the rest of backward
            if bucket.ready >= bucket.expected:
                bucket.ready = 0
                if fused or not distributed:
                    for piece in bucket.subs:
                        piece.ready = 0   # fused reduction: the barrier waits for optimizer.step()
                else:
                    # backward is over for this bucket: launch what a repeated parameter may have
                    # left behind and order the current stream after all pieces
                    _reduce_bucket(plan, bucket, current_rank, only_started=True)

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
