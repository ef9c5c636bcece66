"""Flat layout shared by ZeRO-1 (parameter all-gather) and ZeRO-2 (gradient reduce-scatter).

The reference moves one tensor per collective: a ``dist.broadcast`` per parameter after the step
(ramtorch/zero1.py:78-91) and a ``dist.reduce`` per gradient during backward
(ramtorch/zero2.py:27-57).  Here the parameters of every (device, dtype) are packed, grouped by
owner rank, into one flat buffer

    [ rank 0's tensors | pad ][ rank 1's tensors | pad ] ... [ rank W-1's tensors | pad ]

with equal-length segments, and each parameter's ``.data`` becomes a view into it.  One in-place
``all_gather_into_tensor`` then redistributes all updated parameters, and one in-place
``reduce_scatter_tensor`` over an identically laid out gradient buffer delivers every owner the
sum of its gradients.  Ownership stays at whole-tensor granularity, exactly as the dict returned
by ``create_zero_param_groups`` says, so ``optimizer.state[p]`` and ``state_dict()`` keep the
reference's shape.
"""
from __future__ import annotations

import hashlib
import os
import warnings
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

ALIGN_BYTES = 256
PARAM_IDS_KEY = "rt_param_ids"


def grad_bucket_bytes() -> int:
    """Target size of one gradient sub-bucket (bytes of flat buffer, all ranks' parts together):
    512 MiB unless RT_ZERO2_BUCKET_MB says otherwise.  Small enough that the first reduce-scatter
    starts early in backward; large enough that NCCL runs near link speed (measured on two GPUs,
    4 GiB in all: one call 4.5 ms, four calls of 1 GiB 4.9 ms, sixteen of 256 MiB 5.5 ms)."""
    return max(256, int(float(os.environ.get("RT_ZERO2_BUCKET_MB", "512")) * (1 << 20)))


class SubBucket:
    """A contiguous piece of a bucket's flat gradient buffer, [rank 0's part | ... | rank W-1's part]
    with equal parts, holding the gradients of a run of parameters that become ready at about the
    same time in backward.  Reduced with one in-place reduce-scatter as soon as it is complete."""

    __slots__ = ("start", "part", "expected", "ready", "work", "zeroed")

    def __init__(self, start, part):
        self.start, self.part = start, part       # element offset in gflat, elements per rank
        self.expected = 0                         # parameters of this piece that take part in backward
        self.ready = 0                            # gradients that arrived since the last reduction
        self.work = None                          # pending reduce-scatter
        self.zeroed = None                        # event: the other ranks' parts have been cleared again

# The fused paths use plain peer loads and stores only; keep PyTorch's symmetric memory from also
# binding the buffers to an NVLink multicast object (nothing here uses multimem, and a rank that
# dies while bound to one can disturb its peers' links).  Respect an explicit user setting.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class Bucket:
    """All flattened parameters of one (device, dtype)."""

    def __init__(self, device, dtype, world_size):
        self.device, self.dtype, self.world_size = device, dtype, world_size
        self.params: List[torch.Tensor] = []
        self.owner: List[int] = []
        self.offset: List[int] = []          # element offset of each parameter inside `flat`
        self.segment = 0                     # elements per rank segment
        self.flat: Optional[torch.Tensor] = None
        self.gflat: Optional[torch.Tensor] = None
        self.grad_views: List[Optional[torch.Tensor]] = []
        self.order: List[int] = []           # registration position of each parameter (backward runs it in reverse)
        self.subs: List[SubBucket] = []      # pieces of gflat, in the order backward completes them
        self.sub_of: List[int] = []          # parameter -> index into subs
        self.goffset: List[int] = []         # element offset of each parameter's gradient inside gflat
        self.ready = 0                       # gradients accumulated since the last reduction
        self.expected = 0                    # parameters that take part in backward
        self.side = None                     # stream that clears reduced pieces off the critical path
        # fused redistribution: `flat` is peer-mapped and the optimizer kernel stores updated
        # parameters straight into every peer's copy
        self.peer_ptrs: Optional[List[int]] = None   # base address of every rank's flat buffer
        self.rank = -1                       # this process's rank among the peers
        self.symm = None                     # keeps the peer mapping alive
        self.pushed = False                  # set by the optimizer after a pushing launch
        self.mode = None                     # None (undecided) | "push" | "gather"
        self.checks = 0
        # fused gradient reduction: `gflat` is peer-mapped and the optimizer kernel sums the
        # ranks' copies itself instead of a reduce-scatter pass
        self.gpeer_ptrs: Optional[List[int]] = None
        self.gsymm = None
        self.grads_written = False           # a backward wrote gradients since the last barrier

    def rank_segment(self, buf: torch.Tensor, rank: int) -> torch.Tensor:
        return buf[rank * self.segment:(rank + 1) * self.segment]


class ShardPlan:
    def __init__(self, rank_param_groups: Dict[int, list]):
        self.world_size = len(rank_param_groups)
        if sorted(rank_param_groups) != list(range(self.world_size)):
            raise ValueError("rank_param_groups must have one entry per rank 0..world_size-1")
        self.buckets: Dict[tuple, Bucket] = {}
        self.loose: List[tuple] = []         # (param, owner): redistributed one tensor at a time
        self.ramtorch: List[tuple] = []      # CPU-shared parameters: nothing to redistribute
        self.owner_of: Dict[int, int] = {}       # id(param) -> owner rank
        self.bucket_of: Dict[int, tuple] = {}    # id(param) -> bucket key
        self.current_rank: Optional[int] = None
        self.flattened = False
        self.verified = False
        seen = set()
        per_owner: Dict[tuple, Dict[int, list]] = {}
        order_of: Dict[int, tuple] = {}      # id(param) -> position in the caller's registration order
        # same iteration order as the reference (zero1.py:78-80, zero2.py:18-21): it is what keeps
        # the collectives matched across ranks
        for owner in range(self.world_size):
            for gi, group in enumerate(rank_param_groups[owner]):
                ids = group.get(PARAM_IDS_KEY)
                for k, p in enumerate(group["params"]):
                    # create_zero_param_groups records each parameter's global position; a hand-built
                    # dict falls back to "round-robin inside the group", the reference's assignment
                    order_of.setdefault(id(p), (0, int(ids[k])) if ids is not None and len(ids) == len(group["params"])
                                        else (1, gi, k * self.world_size + owner))
                    self.owner_of[id(p)] = owner
                    if id(p) in seen:
                        continue
                    seen.add(id(p))
                    if getattr(p, "is_ramtorch", False):
                        self.ramtorch.append((p, owner))
                    elif not p.data.is_contiguous():
                        self.loose.append((p, owner))
                    else:
                        key = (p.device, p.dtype)
                        per_owner.setdefault(key, {}).setdefault(owner, []).append(p)
        for key, owners in per_owner.items():
            b = Bucket(key[0], key[1], self.world_size)
            align = max(1, ALIGN_BYTES // torch.empty((), dtype=key[1]).element_size())
            rel, longest = {}, 0
            for owner in range(self.world_size):
                cur = 0
                for p in owners.get(owner, []):
                    rel[id(p)] = cur
                    cur += (p.numel() + align - 1) // align * align
                longest = max(longest, cur)
            b.segment = max(longest, align)
            for owner in range(self.world_size):
                for p in owners.get(owner, []):
                    b.params.append(p)
                    b.owner.append(owner)
                    b.offset.append(owner * b.segment + rel[id(p)])
                    b.order.append(order_of[id(p)])
                    self.bucket_of[id(p)] = key
            self.buckets[key] = b

    # ------------------------------------------------------------------ layout identity
    def fingerprint(self) -> str:
        h = hashlib.sha256()
        h.update(f"{self.world_size}/{grad_bucket_bytes()}".encode())
        for key in sorted(self.buckets, key=str):
            b = self.buckets[key]
            h.update(f"|{key[0].type}:{key[1]}:{b.segment}".encode())
            for p, o, off in zip(b.params, b.owner, b.offset):
                h.update(f";{tuple(p.shape)}@{o}+{off}".encode())
        for p, o in self.loose:
            h.update(f"|loose{tuple(p.shape)}{p.dtype}@{o}".encode())
        return h.hexdigest()

    def verify_across_ranks(self) -> None:
        """Every rank must have built the same layout, or the flat collectives would silently mix
        tensors.  Compared once, on the host, before any data-path collective."""
        if self.verified or not (dist.is_available() and dist.is_initialized()):
            return
        if dist.get_world_size() != self.world_size:
            raise ValueError(f"rank_param_groups describes {self.world_size} ranks but the process group "
                             f"has {dist.get_world_size()}")
        mine = self.fingerprint()
        everyone = [None] * self.world_size
        dist.all_gather_object(everyone, mine)
        if any(f != mine for f in everyone):
            bad = [r for r, f in enumerate(everyone) if f != everyone[0]]
            raise RuntimeError(f"ZeRO shard plans differ between ranks (ranks {bad} disagree with rank 0): "
                               "parameter order, shapes or dtypes are not identical everywhere")
        self.verified = True

    # ------------------------------------------------------------------ flattening
    def _peer_bucket(self) -> Optional[Bucket]:
        """The one bucket of this plan that gets peer-mapped buffers: the largest in bytes.  An
        optimizer launch carries one shared parameter region and one shared gradient region, so a
        model with parameters of several dtypes keeps its smaller buckets on the NCCL collectives."""
        if not self.buckets:
            return None
        return max(self.buckets.values(),
                   key=lambda b: b.segment * torch.empty((), dtype=b.dtype).element_size())

    def _allocate_flat(self, b: Bucket) -> torch.Tensor:
        """The flat parameter buffer of a bucket.  On NCCL ranks with CUDA parameters it is
        allocated as peer-mapped ("symmetric") memory so that the optimizer kernel can store the
        owners' new values directly into every rank's copy; anything else gets plain memory and
        the all-gather path.  Set RT_ZERO_FUSED_PUSH=0 to force the all-gather path."""
        n = b.segment * self.world_size
        want = (b is self._peer_bucket() and b.device.type == "cuda" and self.world_size > 1 and self.world_size - 1 <= 15 and
                dist.is_available() and dist.is_initialized() and dist.get_backend() == "nccl" and
                dist.get_world_size() == self.world_size and os.environ.get("RT_ZERO_FUSED_PUSH", "1") != "0")
        if want:
            try:
                import torch.distributed._symmetric_memory as symm
                flat = symm.empty(n, dtype=b.dtype, device=b.device)
                handle = symm.rendezvous(flat, dist.group.WORLD)
                b.peer_ptrs = [int(q) for q in handle.buffer_ptrs]
                b.rank = int(handle.rank)
                b.symm = handle
                flat.zero_()
                _PUSH_BUCKETS.setdefault(b.device.index, []).append(b)
                return flat
            except Exception as e:  # pragma: no cover - depends on driver / topology
                warnings.warn(f"peer-mapped parameter buffer unavailable ({e!r}); using NCCL all-gather")
                b.peer_ptrs = None
        return torch.zeros(n, dtype=b.dtype, device=b.device)

    def flatten_params(self) -> None:
        """Move every bucket's parameters into its flat buffer and re-point ``p.data`` at the views."""
        if self.flattened:
            return
        with torch.no_grad():
            for b in self.buckets.values():
                b.flat = self._allocate_flat(b)
                for p, off in zip(b.params, b.offset):
                    view = b.flat[off:off + p.numel()].view(p.shape)
                    view.copy_(p.data)
                    p.data = view
        self.flattened = True

    def _layout_grad_pieces(self, b: Bucket) -> int:
        """Cut the bucket's gradients into sub-buckets.  Parameters are taken in reverse registration
        order (the order in which backward finishes them); inside a piece each rank's tensors are
        packed into that rank's part, and all parts of a piece are as long as its longest.  A piece
        is closed once it holds the target number of bytes AND its parts are balanced (padding
        below 1/8 of the piece): a piece closed right after one huge tensor would consist
        mostly of the other ranks' empty parts, which the reduce-scatter would still move.  A
        lopsided last piece is merged into the one before it, and an ownership that never
        balances ends up as one piece, i.e. one collective at the end of backward.  Returns the
        length of the flat gradient buffer in elements."""
        esize = torch.empty((), dtype=b.dtype).element_size()
        align = max(1, ALIGN_BYTES // esize)
        target = max(align * self.world_size, grad_bucket_bytes() // esize)
        by_backward = sorted(range(len(b.params)), key=lambda k: b.order[k], reverse=True)
        b.subs, b.sub_of, b.goffset = [], [0] * len(b.params), [0] * len(b.params)
        pieces, fill, members = [], [0] * self.world_size, []
        for k in by_backward:
            members.append((k, fill[b.owner[k]]))
            fill[b.owner[k]] += (b.params[k].numel() + align - 1) // align * align
            span, useful = max(fill) * self.world_size, sum(fill)
            if useful >= target and (span - useful) * 8 < span:
                pieces.append((members, list(fill)))
                fill, members = [0] * self.world_size, []
        if members:
            if pieces and (max(fill) * self.world_size - sum(fill)) * 4 > max(fill) * self.world_size:
                # the tail is more than a quarter padding: append it to the previous piece
                prev_members, prev_fill = pieces.pop()
                members = prev_members + [(k, rel + prev_fill[b.owner[k]]) for k, rel in members]
                fill = [a + c for a, c in zip(prev_fill, fill)]
            pieces.append((members, list(fill)))
        start = 0
        for members, fills in pieces:
            part = max(max(fills), align)
            sub = SubBucket(start, part)
            for k, rel in members:
                b.sub_of[k] = len(b.subs)
                b.goffset[k] = start + b.owner[k] * part + rel
            b.subs.append(sub)
            start += part * self.world_size
        return max(start, align)

    def attach_grad_buffers(self, fused_pull: bool = False) -> None:
        """Allocate the flat gradient buffers and make every ``p.grad`` a view so that autograd
        accumulates straight into them.  With ``fused_pull`` (and a peer-mapped parameter buffer)
        the gradient buffer is peer-mapped too, for the optimizer kernel to read every rank's copy."""
        for b in self.buckets.values():
            if b.gflat is not None:
                continue
            n = self._layout_grad_pieces(b)
            if fused_pull and b.peer_ptrs is not None:
                import torch.distributed._symmetric_memory as symm
                b.gflat = symm.empty(n, dtype=b.dtype, device=b.device)
                handle = symm.rendezvous(b.gflat, dist.group.WORLD)
                b.gpeer_ptrs = [int(q) for q in handle.buffer_ptrs]
                b.gsymm = handle
                b.gflat.zero_()
                _PULL_BUCKETS.setdefault(b.device.index, []).append(b)
            else:
                b.gflat = torch.zeros(n, dtype=b.dtype, device=b.device)
            b.grad_views = []
            b.expected = 0
            for k, p in enumerate(b.params):
                if p.requires_grad:
                    off = b.goffset[k]
                    view = b.gflat[off:off + p.numel()].view(p.shape)
                    b.grad_views.append(view)
                    p.grad = view
                    b.expected += 1
                    b.subs[b.sub_of[k]].expected += 1
                else:
                    b.grad_views.append(None)


_PLANS: Dict[int, tuple] = {}
_PUSH_BUCKETS: Dict[int, List[Bucket]] = {}   # cuda device index -> buckets with peer-mapped buffers
_PULL_BUCKETS: Dict[int, List[Bucket]] = {}   # cuda device index -> buckets with peer-mapped gradients


def release_plan(rank_param_groups) -> None:
    """Forget the flat buffers of a ``rank -> groups`` dict: its peer-mapped buckets leave the
    registries the optimizer consults, so their memory is returned once the parameters that view
    them are gone.  For programs that build several sharded parameter sets one after another; the
    dict must not be used with ``broadcast_zero_params`` / the ZeRO-2 hooks afterwards."""
    plan = getattr(rank_param_groups, "plan", None)
    if plan is None:
        hit = _PLANS.pop(id(rank_param_groups), None)
        plan = hit[1] if hit is not None else None
    if plan is None:
        return
    for b in plan.buckets.values():
        for registry in (_PUSH_BUCKETS, _PULL_BUCKETS):
            for index in list(registry):
                registry[index] = [x for x in registry[index] if x is not b]
                if not registry[index]:
                    del registry[index]
        b.symm = b.gsymm = None
        b.peer_ptrs = b.gpeer_ptrs = None
        b.flat = b.gflat = None
        b.grad_views = []
    try:
        rank_param_groups.plan = None
    except AttributeError:
        pass


def pull_bucket_for(device_index: int, grad_ptrs) -> Optional[Bucket]:
    """The peer-mapped gradient bucket on ``device_index`` that holds most of the given addresses."""
    best, best_hits = None, 0
    for b in _PULL_BUCKETS.get(device_index, []):
        lo = b.gflat.data_ptr()
        hi = lo + b.gflat.numel() * b.gflat.element_size()
        hits = sum(1 for q in grad_ptrs if q is not None and lo <= q < hi)
        if hits > best_hits:
            best, best_hits = b, hits
    return best


def all_push_buckets() -> List[Bucket]:
    return [b for bs in _PUSH_BUCKETS.values() for b in bs]


def push_bucket_for(device_index: int, data_ptrs) -> Optional[Bucket]:
    """The peer-mapped bucket on ``device_index`` that holds most of the given parameter addresses."""
    best, best_hits = None, 0
    for b in _PUSH_BUCKETS.get(device_index, []):
        lo = b.flat.data_ptr()
        hi = lo + b.flat.numel() * b.flat.element_size()
        hits = sum(1 for q in data_ptrs if lo <= q < hi)
        if hits > best_hits:
            best, best_hits = b, hits
    return best


def plan_for(rank_param_groups) -> ShardPlan:
    """The plan attached to a ``rank -> groups`` dict (built on first use).  Hand-built dicts work
    too: the plan is cached by object identity and the dict is kept alive with it."""
    plan = getattr(rank_param_groups, "plan", None)
    if plan is not None:
        return plan
    hit = _PLANS.get(id(rank_param_groups))
    if hit is not None and hit[0] is rank_param_groups:
        return hit[1]
    plan = ShardPlan(rank_param_groups)
    try:
        rank_param_groups.plan = plan
    except AttributeError:
        _PLANS[id(rank_param_groups)] = (rank_param_groups, plan)
    return plan
