"""AdamW with bf16 stochastic rounding — drop-in for ``ramtorch.stochastic_optimizers.adamw``.

Same constructor, same ``state[p]`` keys (``step``, ``ema``, ``ema_squared``), same update rule as
the reference (ramtorch/stochastic_optimizers/adamw.py:33-234), but ``step()`` hands the whole
parameter list to ``librt_b200.so``:

* tensors whose parameter, gradient and moments all sit in HBM go through ONE fused
  multi-tensor kernel launch per dtype combination (the reference issues ~25 ATen launches and
  up to three generator constructions per tensor, adamw.py:160-222);
* tensors with any of them in CPU RAM go through the chunked copy-in / update / copy-out
  pipeline on side streams (the reference serialises ``.to(device)`` → math → ``.copy_`` on one
  stream, adamw.py:160-170, :204-222).

Differences from the reference that a user can observe, all deliberate:

* random bits come from a counter-based Philox stream keyed by ``(seed, step, tensor id, element
  index)`` instead of ``torch.Generator(seed=step+42/69/420)`` (adamw.py:206-218), so results do
  not depend on device, launch geometry, chunking or world size;
* there is no CPU path: without a CUDA device ``step()`` raises;
* one stream synchronisation at the end of ``step()`` replaces the device-wide synchronisations
  every ``chunk_size`` parameters (adamw.py:227-232); ``chunk_size`` is accepted and ignored.
"""
from __future__ import annotations

import ctypes
import operator
import warnings
from collections import defaultdict
from itertools import chain

import numpy as np

import torch
import torch.optim.optimizer as _torch_opt
from torch.optim import Optimizer

from .. import _native as N
from .. import _shard_plan as SP
from ..functional import sr_round_bf16_

import contextlib

from .. import zero2 as _zero2

import os

try:      # host-side helper: walks long parameter lists in C++ (built by ramtorch_b200.csrc.build)
    from .. import _fastscan as _FS
    if os.environ.get("RT_NO_FASTSCAN") == "1":
        _FS = None
except ImportError:  # pragma: no cover - the helper is optional; the Python passes below do the same
    _FS = None

_NULL_CTX = contextlib.nullcontext()
_GET_EMA, _GET_EMA_SQ, _GET_STEP = (operator.itemgetter(k) for k in ("ema", "ema_squared", "step"))
_PARAM_IDS_KEY = "rt_param_ids"
DEVICE_GRAD_ATTR = "rt_device_grad"


def _grad_of(p):
    """The gradient ``step`` consumes.  PyTorch refuses a CUDA ``.grad`` on a CPU parameter, so a
    producer that keeps the gradient of a CPU-resident parameter in HBM (instead of copying it to
    host memory only for ``step`` to copy it back, ramtorch/modules/linear.py:416-427 ->
    adamw.py:167) hands it over as ``p.rt_device_grad``; it takes precedence over ``p.grad`` for
    CPU parameters and is ignored for CUDA parameters."""
    if not p.is_cuda:
        g = getattr(p, DEVICE_GRAD_ATTR, None)
        if g is not None:
            return g
    return p.grad


def copy_stochastic_(target: torch.Tensor, source: torch.Tensor, seed=0):
    """bf16 stochastic rounding of an fp32 CUDA tensor into ``target`` (adamw.py:6-30).

    ``out = (bits(source) + r16) & 0xFFFF0000`` with ``r16`` uniform on [0, 65536).  The draws
    come from Philox keyed by ``seed`` and the element index."""
    with torch.no_grad():
        src = source.detach()
        if src.dtype != torch.float32:
            raise ValueError("source must be float32")
        src = src.contiguous()
        if target.is_contiguous():
            sr_round_bf16_(target.detach(), src, seed=int(seed))
        else:
            tmp = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
            sr_round_bf16_(tmp, src, seed=int(seed))
            target.copy_(tmp)


class _TrackedState(defaultdict):
    """``Optimizer.state`` that counts structural changes (an entry added, replaced or removed), so
    that the repeat-step fast path can tell in O(1) that the per-parameter state dicts it cached
    are still the ones in use."""

    epoch = 0

    def _bump(self):
        self.epoch += 1

    def __setitem__(self, key, value):
        self.epoch += 1
        super().__setitem__(key, value)

    def __delitem__(self, key):
        self.epoch += 1
        super().__delitem__(key)

    def pop(self, *a):
        self.epoch += 1
        return super().pop(*a)

    def popitem(self):
        self.epoch += 1
        return super().popitem()

    def clear(self):
        self.epoch += 1
        super().clear()

    def update(self, *a, **k):
        self.epoch += 1
        super().update(*a, **k)

    def setdefault(self, key, default=None):
        self.epoch += 1
        return super().setdefault(key, default)

    def __reduce__(self):   # pickles like the defaultdict it stands in for
        return (defaultdict, (dict,), None, None, iter(self.items()))


def _fast_dispatch_ok() -> bool:
    """Whether this torch build exposes what ``AdamW.step`` reads to decide that the stock
    ``Optimizer.step`` wrapper (profiler range + hook dispatch) has nothing to do.  If any name is
    missing, every step goes through the stock wrapper."""
    return (hasattr(_torch_opt, "_global_optimizer_pre_hooks") and
            hasattr(_torch_opt, "_global_optimizer_post_hooks") and
            hasattr(torch.autograd.profiler, "_is_profiler_enabled") and
            hasattr(Optimizer, "profile_hook_step") and hasattr(Optimizer, "_patch_step_function"))


_FAST_DISPATCH = _fast_dispatch_ok()


class _DevicePlan:
    """A live ``rt_plan`` handle plus the signature it was built from."""

    def __init__(self, device_index: int, signature, descs):
        self.signature = signature
        self.handle = ctypes.c_void_p()
        arr = (N.TensorDesc * len(descs))(*descs)
        N.check(N.lib().rt_plan_create(ctypes.byref(self.handle), arr, len(descs), device_index),
                "rt_plan_create")
        self.launches = N.lib().rt_plan_launches(self.handle)
        self.grad_ptrs = (N.c_void_p * len(descs))()
        # ZeRO-1: when the parameters live in a peer-mapped flat buffer, let the kernel store the
        # updated values into every peer's copy as well
        self.push_bucket = SP.push_bucket_for(device_index, [d.p for d in descs])
        if self.push_bucket is not None:
            b = self.push_bucket
            # peers in ring order starting with the right neighbour: at any moment the ranks' stores head
            # for different GPUs instead of all starting with rank 0
            world = len(b.peer_ptrs)
            peers = [b.peer_ptrs[(b.rank + k) % world] for k in range(1, world)]
            push = N.Push()
            push.local_base = b.flat.data_ptr()
            push.bytes = b.flat.numel() * b.flat.element_size()
            push.n_peers = len(peers)
            for k, q in enumerate(peers):
                push.peer_base[k] = q
            N.check(N.lib().rt_plan_set_push(self.handle, ctypes.byref(push)), "rt_plan_set_push")
        # ZeRO-2: when the gradients live in a peer-mapped flat buffer, let the kernel sum the
        # ranks' copies itself
        self.pull_bucket = SP.pull_bucket_for(device_index, [d.g for d in descs])
        if self.pull_bucket is not None:
            b = self.pull_bucket
            pull = N.Pull()
            pull.local_base = b.gflat.data_ptr()
            pull.bytes = b.gflat.numel() * b.gflat.element_size()
            pull.n_ranks = len(b.gpeer_ptrs)
            pull.self_rank = b.rank
            for k, q in enumerate(b.gpeer_ptrs):
                pull.base[k] = q
            N.check(N.lib().rt_plan_set_pull(self.handle, ctypes.byref(pull)), "rt_plan_set_pull")

    def close(self):
        if self.handle:
            N.lib().rt_plan_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


class AdamW(Optimizer):
    r"""
    Arguments (identical to the reference, adamw.py:57-69):
        params: iterable of parameters or dicts defining parameter groups.
        lr: learning rate (default 1e-3).
        betas: coefficients of the running averages (default (0.9, 0.999)).
        eps: added to the denominator (default 1e-8).
        weight_decay: decoupled weight decay, scaled by the bias-corrected step size as in the
            reference (default 1e-2).
        centralization: gradient centralization factor (default 0).
        chunk_size: accepted for compatibility; the fused path needs no periodic sync.
        dtype: dtype of ``ema`` / ``ema_squared`` (default bf16).
        storage_device: where the moments live; the string ``"cpu"`` means pinned host memory.

    Keyword-only additions:
        seed: Philox key of the stochastic-rounding stream (default 0).
        offload_chunk_elems: elements per streamed chunk for host-resident tensors.
        offload_ring_depth: staging slots of the streaming pipeline (2..8).
        sync: wait for the step to finish before returning, as the reference does (default True).
        reference_order: form the denominator and the quotient in the reference's own operation
            order (``sqrt(v)/bc + eps`` and ``p + (a*m)/den``: two IEEE divisions per element)
            instead of the default ``fma(sqrt(v), 1/bc, eps)`` and ``fma(a*m, 1/den, p)``.  Both
            are reproducible bit for bit by the CPU checker; the moments are identical either
            way and the parameters agree within 1e-6 (default False).
        register_host_memory: pin, in place (``cudaHostRegister``), host-resident parameters and
            moments whose storage is shared memory and not page-locked -- parameter storage shared
            between worker processes through ``mp.spawn`` pickling arrives like that in the worker
            -- so that their copies overlap with the update instead of falling back to pageable
            transfers.  The registration lasts until ``release_host_memory()`` or until the
            optimizer is collected; gradients are never registered (they are usually re-allocated
            by every backward).  Default True.
        shared_draws: one Philox block per eight elements serves parameter and both moments
            (lanes rotated by two per stream) instead of three independent blocks.  Every rounding
            still sees a uniform 16-bit draw, the three roundings of any one element stay mutually
            independent, and the result is bit-identical to the checker run with the same flag;
            what is shared is the draw of p[i], ema[i-2] and ema_squared[i-4] inside a group of
            eight.  Default True (it only matters for bf16 moments, where it is the difference
            between 0.70 and 0.90 of the HBM roofline); pass False for three independent blocks.
    """

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2,
                 centralization=0, chunk_size=64, dtype=torch.bfloat16, storage_device="cpu",
                 *, seed=0, offload_chunk_elems=1 << 24, offload_ring_depth=3, sync=True,
                 reference_order=False, shared_draws=True, register_host_memory=True):
        if dtype not in N.DTYPE_CODE:
            raise ValueError(f"unsupported state dtype {dtype}: bf16, fp32 or fp16")
        if offload_chunk_elems <= 0 or offload_chunk_elems % 8:
            raise ValueError("offload_chunk_elems must be a positive multiple of 8")
        if not 2 <= offload_ring_depth <= 8:
            raise ValueError("offload_ring_depth must be in 2..8")
        self._next_tensor_id = 0
        self._tensor_ids = {}
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                        centralization=centralization)
        super().__init__(params, defaults)
        self._track_state()

        self.chunk_size = chunk_size
        self.optim_state_dtype = dtype
        self.optim_state_device = storage_device
        self.seed = int(seed)
        self.offload_chunk_elems = int(offload_chunk_elems)
        self.offload_ring_depth = int(offload_ring_depth)
        self.sync = bool(sync)
        self.reference_order = bool(reference_order)
        self.shared_draws = bool(shared_draws)
        self.register_host_memory = bool(register_host_memory)
        self._registered = {}   # storage address -> bytes pinned in place by this optimizer
        self._plans = {}      # cuda device index -> _DevicePlan
        self._staging = {}    # cuda device index -> uint8 tensor
        self._row_scratch = {}  # cuda device index -> fp32 row means for centralization
        self._keepalive = []
        self._warned_pageable = False
        self._push_marks = []  # peer-mapped buckets the last validated step fully redistributed
        self._fast = None     # cache that lets an unchanged, fully resident step skip re-validation
        self._cuda_checked = False
        self.last_step_info = {}

        # eager state, as adamw.py:84-104; "cpu" (the string) means pinned, and the pinned
        # moments of all parameters share two allocations instead of two per tensor
        fresh = [p for g in self.param_groups for p in g["params"] if not self.state[p]]
        self._allocate_states(fresh)

    # ------------------------------------------------------------------ bookkeeping
    def _track_state(self):
        if not isinstance(self.state, _TrackedState):
            tracked = _TrackedState(dict)
            tracked.update(self.state)
            self.state = tracked
        self.state._bump()

    def __setstate__(self, state):
        # load_state_dict() and unpickling replace self.state and the group dicts wholesale: whatever
        # the repeat-step fast path and the device plans remembered is stale from here on
        super().__setstate__(state)
        self._track_state()
        self._fast = None
        for plan in getattr(self, "_plans", {}).values():
            plan.close()
        self._plans = {}

    def add_param_group(self, param_group):
        super().add_param_group(param_group)
        group = self.param_groups[-1]
        ids = group.get(_PARAM_IDS_KEY)
        if ids is not None and len(ids) != len(group["params"]):
            raise ValueError(f"{_PARAM_IDS_KEY} must list one id per parameter of the group")
        for k, p in enumerate(group["params"]):
            if ids is not None:
                self._tensor_ids[p] = int(ids[k])
            else:
                self._tensor_ids[p] = self._next_tensor_id
                self._next_tensor_id += 1

    def _allocate_states(self, params):
        """``step = 0`` and zero moments of ``dtype`` on ``storage_device`` (adamw.py:85-104)."""
        if not params:
            return
        dtype, dev = self.optim_state_dtype, self.optim_state_device
        if isinstance(dev, str) and dev == "cpu":
            esize = torch.empty((), dtype=dtype).element_size()
            offs, total = [], 0
            for p in params:
                offs.append(total)
                total += (p.numel() * esize + 255) // 256 * 256
            pools = [torch.zeros(max(total, 256), dtype=torch.uint8, pin_memory=True) for _ in range(2)]
            for p, off in zip(params, offs):
                nbytes = p.numel() * esize
                st = self.state[p]
                st["step"] = 0
                st["ema"], st["ema_squared"] = (
                    pool[off:off + nbytes].view(dtype).view(p.shape) for pool in pools)
        else:
            for p in params:
                st = self.state[p]
                st["step"] = 0
                st["ema"] = torch.zeros(p.shape, dtype=dtype, device=dev)
                st["ema_squared"] = torch.zeros(p.shape, dtype=dtype, device=dev)

    def zero_grad(self, set_to_none: bool = True) -> None:
        """``Optimizer.zero_grad`` plus the device-side gradients of CPU parameters
        (``p.rt_device_grad``, see ``helpers.accumulate_device_grad``): dropped, or zeroed in place
        with ``set_to_none=False``, exactly like ``p.grad``."""
        super().zero_grad(set_to_none=set_to_none)
        for group in self.param_groups:
            for p in group["params"]:
                g = p.__dict__.get(DEVICE_GRAD_ATTR)
                if g is not None:
                    if set_to_none:
                        setattr(p, DEVICE_GRAD_ATTR, None)
                    else:
                        g.zero_()

    def _pin_in_place(self, lib, t: torch.Tensor) -> bool:
        """Page-lock the storage of a host tensor where it lies (``rt_host_register``); True when the
        storage is pinned afterwards."""
        # Only storages in shared memory qualify: they are mappings of their own (page-aligned, no
        # neighbours), and they are the case that needs it.  Page-locking a few bytes in the middle
        # of the malloc heap would also lock whatever shares their pages, and a later copy from a
        # buffer that straddles locked and unlocked pages is refused by the CUDA runtime.
        if not self.register_host_memory or not t.is_shared():
            return False
        storage = t.untyped_storage()
        ptr, nbytes = storage.data_ptr(), storage.nbytes()
        if ptr in self._registered:
            return True
        if nbytes == 0 or lib.rt_host_register(ptr, nbytes) != 0:
            return False
        self._registered[ptr] = nbytes
        return True

    def __del__(self):   # the pages must not stay locked once nobody streams them any more
        try:
            self.release_host_memory()
        except Exception:  # pragma: no cover - interpreter shutdown
            pass

    def release_host_memory(self) -> None:
        """Undo the in-place pinning done by ``register_host_memory`` (after a device synchronise:
        no copy may still be using the pages)."""
        if not getattr(self, "_registered", None):
            return
        torch.cuda.synchronize()
        lib = N.lib()
        for ptr in list(self._registered):
            lib.rt_host_unregister(ptr)
            del self._registered[ptr]

    def _staging_for(self, index: int, nbytes: int) -> torch.Tensor:
        buf = self._staging.get(index)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", index))
            self._staging[index] = buf
        return buf

    # ------------------------------------------------------------------ the step
    if _FAST_DISPATCH:
        def _patch_step_function(self) -> None:
            # torch wraps every Optimizer.step in a profiler range plus hook dispatch (~35 us per
            # call, as much as the fused kernel needs for 16M elements).  step() below keeps the
            # same behaviour -- pre/post hooks run, the range is opened while a profiler is
            # recording -- but skips the machinery when there is nothing to run or record.
            self._zero_grad_profile_name = f"Optimizer.zero_grad#{self.__class__.__name__}.zero_grad"

        def step(self, closure=None):
            if (self._optimizer_step_pre_hooks or self._optimizer_step_post_hooks or
                    _torch_opt._global_optimizer_pre_hooks or _torch_opt._global_optimizer_post_hooks or
                    torch.autograd.profiler._is_profiler_enabled):
                return _HOOKED_STEP(self, closure)
            return self._step(closure)
    else:  # pragma: no cover - a torch build without the names inspected above
        def step(self, closure=None):
            # the base class wraps this method with its own profiler range and hook dispatch
            return self._step(closure)

    def _step(self, closure=None):
        loss = None
        if closure is not None:
            loss = closure()
        if not self._cuda_checked:
            if not torch.cuda.is_available():
                raise RuntimeError("ramtorch_b200.AdamW needs a CUDA device: there is no CPU fallback")
            self._cuda_checked = True
        lib = N.lib()
        self._keepalive.clear()
        if _zero2._ACTIVE_PLANS:
            _zero2.finish_grad_sync()   # ZeRO-2: reduce buckets a partial backward left behind
        if self._fast is not None and self._step_fast(lib):
            return loss
        self._fast = None

        resident = {}   # device index -> list of (p, grad, ema, ema_sq, tensor_id, hyper_index)
        streamed = []   # (device index, p, grad, ema, ema_sq, tensor_id, hyper_index)
        hyper_rows, hyper_index = [], {}
        centered = {}   # device index -> {position in resident[index]: number of rows}
        centered_streamed = {}   # position in streamed: number of rows
        skipped_empty = False
        late = []
        stepped = []    # state dicts whose counter advances with this step
        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                grad = _grad_of(p)
                if grad is None:
                    continue
                if grad.is_sparse:
                    raise RuntimeError("AdamW does not support sparse gradients")
                if not self.state[p]:
                    late.append(p)
        self._allocate_states(late)  # lazy state for parameters added late (adamw.py:125-148)

        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                grad = _grad_of(p)
                if grad is None:
                    continue
                state = self.state[p]
                t = state["step"] + 1     # written back once every tensor of the step has been validated
                stepped.append(state)
                key = (gi, t)
                hi = hyper_index.get(key)
                if hi is None:
                    hi = hyper_index[key] = len(hyper_rows)
                    hyper_rows.append(N.make_hyper(group["lr"], group["betas"], group["eps"],
                                                   group["weight_decay"], t,
                                                   group["centralization"], self.reference_order, self.shared_draws))
                ema, ema_sq = state["ema"], state["ema_squared"]
                pd = p.data
                if pd.numel() == 0:
                    skipped_empty = True      # nothing to update; the step counter still advances
                    continue
                if not pd.is_contiguous():
                    raise ValueError("parameters must be contiguous for the in-place fused update")
                if not grad.is_contiguous():
                    grad = grad.contiguous()
                    self._keepalive.append(grad)
                if not (ema.is_contiguous() and ema_sq.is_contiguous()):
                    raise ValueError("optimizer state tensors must be contiguous")
                if ema.dtype != ema_sq.dtype:
                    raise ValueError("ema and ema_squared must share a dtype")
                for t, name in ((pd, "parameter"), (grad, "gradient"), (ema, "state")):
                    if t.dtype not in N.DTYPE_CODE:
                        raise ValueError(f"unsupported {name} dtype {t.dtype}: bf16, fp32 or fp16")
                if not (grad.numel() == ema.numel() == ema_sq.numel() == pd.numel()):
                    raise ValueError("parameter, gradient and state sizes differ")
                cuda_devs = {t.device.index for t in (pd, grad, ema, ema_sq) if t.is_cuda}
                if len(cuda_devs) > 1:
                    raise ValueError("parameter, gradient and state sit on different CUDA devices")
                # compute device: the parameter's, or the current one for CPU parameters
                # (adamw.py:152-157)
                index = cuda_devs.pop() if cuda_devs else torch.cuda.current_device()
                entry = (pd, grad, ema, ema_sq, self._tensor_ids[p], hi)
                if pd.is_cuda and grad.is_cuda and ema.is_cuda and ema_sq.is_cuda:
                    resident.setdefault(index, []).append(entry)
                    if group["centralization"] != 0:
                        # rows = size of dim 0; tensors with fewer than two dimensions are one row
                        # (the reference's mean over an empty dim tuple reduces everything)
                        rows = pd.shape[0] if pd.dim() >= 2 else 1
                        centered.setdefault(index, {})[len(resident[index]) - 1] = rows
                else:
                    if group["centralization"] != 0:
                        centered_streamed[len(streamed)] = pd.shape[0] if pd.dim() >= 2 else 1
                    if grad.is_cuda and SP.pull_bucket_for(index, [grad.data_ptr()]) is not None:
                        raise RuntimeError("ZeRO-2 fused gradient reduction (RT_ZERO2_FUSED_PULL=1) needs the moments in "
                                           "HBM (storage_device on the GPU): the streamed path does not sum the ranks' "
                                           "gradients")
                    streamed.append((index,) + entry)

        if len(hyper_rows) > 1024:
            raise ValueError("more than 1024 distinct (group, step) pairs in one step")
        for state in stepped:     # nothing above raised: the step happens (adamw.py:177)
            state["step"] += 1
        hyper_arr = (N.Hyper * max(len(hyper_rows), 1))(*hyper_rows)
        seed = self.seed & (2 ** 64 - 1)
        used = set()
        launches = 0

        for index, entries in resident.items():
            used.add(index)
            with N.trace("rt.step.resident"), torch.cuda.device(index):
                stream = N.stream_ptr(index)
                row_info = self._row_means(lib, index, entries, centered.get(index, {}), stream)
                plan = self._plan_for(index, entries, row_info)
                for k, e in enumerate(entries):
                    plan.grad_ptrs[k] = e[1].data_ptr()
                N.check(lib.rt_plan_set_grads(plan.handle, plan.grad_ptrs, stream), "rt_plan_set_grads")
                N.check(lib.rt_adamw_sr_multi(plan.handle, hyper_arr, len(hyper_rows), seed, stream),
                        "rt_adamw_sr_multi")
                launches += plan.launches

        # one staging ring per device, sized for the largest streamed tensor of this step, so that
        # all of them share its geometry and follow each other through the pipeline
        jobs, ring_bytes = [], {}
        for pos, (index, pd, grad, ema, ema_sq, tid, hi) in enumerate(streamed):
            row_mean = None
            rows = centered_streamed.get(pos)
            if rows is not None:
                # Gradient centralization (adamw.py:179-184) needs the row means before the first
                # chunk is updated: one pass over g alone.  A host-resident gradient is brought to the
                # device whole for that pass and the step then reads it there, so it crosses the
                # link once, as it would without centralization.
                with torch.cuda.device(index):
                    if not grad.is_cuda:
                        grad = grad.to(torch.device("cuda", index), non_blocking=True)
                        self._keepalive.append(grad)
                    row_len = grad.numel() // rows
                    means = torch.empty(rows, dtype=torch.float32, device=grad.device)
                    self._keepalive.append(means)
                    N.check(lib.rt_row_means(grad.data_ptr(), N.DTYPE_CODE[grad.dtype], rows, row_len,
                                             means.data_ptr(), N.stream_ptr(index)), "rt_row_means")
                    row_mean = (means.data_ptr(), row_len if rows > 1 else 0)
            tensors = (pd, grad, ema, ema_sq)
            host = [not t.is_cuda for t in tensors]
            for t, h, what in zip(tensors, host, ("parameter", "gradient", "moment", "moment")):
                if h and not t.is_pinned() and not (what != "gradient" and self._pin_in_place(lib, t)):
                    if not self._warned_pageable:
                        warnings.warn(f"a host-resident {what} is not pinned: its copies fall back to "
                                      "pageable transfers and do not overlap; pin it for full speed")
                        self._warned_pageable = True
            codes = (N.DTYPE_CODE[pd.dtype], N.DTYPE_CODE[grad.dtype], N.DTYPE_CODE[ema.dtype])
            chunk = min(self.offload_chunk_elems, (pd.numel() + 7) // 8 * 8)
            need = lib.rt_offload_staging_bytes(chunk, self.offload_ring_depth, *codes, *map(int, host))
            if need < 0:
                N.check(int(need), "rt_offload_staging_bytes")
            ring_bytes[index] = max(ring_bytes.get(index, 256 * self.offload_ring_depth), int(need))
            jobs.append((index, pd, grad, ema, ema_sq, tid, hi, codes, chunk, row_mean))
        for index, pd, grad, ema, ema_sq, tid, hi, codes, chunk, row_mean in jobs:
            used.add(index)
            with N.trace("rt.step.streamed"), torch.cuda.device(index):
                staging = self._staging_for(index, ring_bytes[index])
                cfg = N.OffloadCfg(chunk, self.offload_ring_depth, 1, staging.data_ptr(), staging.numel())
                if row_mean is not None:
                    cfg.row_mean, cfg.row_len = row_mean
                N.check(lib.rt_adamw_sr_offload(pd.data_ptr(), grad.data_ptr(), ema.data_ptr(),
                                                ema_sq.data_ptr(), pd.numel(), *codes,
                                                ctypes.byref(hyper_arr[hi]), seed, tid,
                                                ctypes.byref(cfg), N.stream_ptr(index)),
                        "rt_adamw_sr_offload")
            launches += (pd.numel() + chunk - 1) // chunk
        for index in {e[0] for e in streamed}:
            # one join per device after the last tensor, so consecutive tensors overlap in the pipeline
            with torch.cuda.device(index):
                N.check(lib.rt_offload_join(N.stream_ptr(index)), "rt_offload_join")

        self._mark_pushed(resident, streamed)
        self.last_step_info = dict(launches=launches, resident=sum(map(len, resident.values())),
                                   streamed=len(streamed))
        if len(resident) == 1 and not streamed and not self._keepalive and not centered and not skipped_empty:
            self._remember_fast(next(iter(resident)), hyper_index)
        if self.sync:
            # results are visible to the host when step() returns (adamw.py:232)
            for index in used:
                torch.cuda.current_stream(index).synchronize()
            self._keepalive.clear()
        return loss

    def _mark_pushed(self, resident, streamed):
        """ZeRO-1 fused redistribution bookkeeping: a peer-mapped parameter bucket counts as
        redistributed by this step unless this step changed a parameter inside it WITHOUT the
        kernel's peer stores (a streamed tensor, or a tensor outside the plan's shared region)."""
        self._push_marks = []
        buckets = SP.all_push_buckets()
        if not buckets:
            return
        plain = [e[1].data_ptr() for e in streamed]          # (index, pd, ...) -> pd
        for index, entries in resident.items():
            pushing = self._plans[index].push_bucket
            for pd, *_ in entries:
                q = pd.data_ptr()
                if pushing is None or not (pushing.flat.data_ptr() <= q <
                                           pushing.flat.data_ptr() + pushing.flat.numel() * pushing.flat.element_size()):
                    plain.append(q)
        for b in buckets:
            lo = b.flat.data_ptr()
            hi = lo + b.flat.numel() * b.flat.element_size()
            if not any(lo <= q < hi for q in plain):
                b.pushed = True
                self._push_marks.append(b)

    # ------------------------------------------------------------------ repeat-step fast path
    def _remember_fast(self, index, hyper_index):
        """After a fully validated step whose tensors all sit on one CUDA device, keep what the
        next step needs to recognise that nothing but the gradients (and the step counters)
        changed: with tens of thousands of small tensors the per-tensor Python work of a full
        validation costs several times the GPU time of the update itself."""
        all_params = list(chain.from_iterable(g["params"] for g in self.param_groups))
        with_grad = [p for p in all_params if p.grad is not None]
        states = [self.state[p] for p in with_grad]
        classes = sorted(hyper_index.items(), key=lambda kv: kv[1])   # ((group, step), row) by row
        self._fast = dict(
            index=index, all_ids=list(map(id, all_params)), params=with_grad,
            has_grad=[p.grad is not None for p in all_params], states=states,
            emas=[st["ema"] for st in states], ema_sqs=[st["ema_squared"] for st in states],
            p_ptrs=list(map(torch.Tensor.data_ptr, with_grad)),
            g_dtypes=[p.grad.dtype for p in with_grad],
            classes=[key for key, _ in classes], n_groups=len(self.param_groups),
            zero_buffers=self._zero_buffer_count(index),
            state_epoch=self.state.epoch, steps=[st["step"] for st in states])
        if _FS is not None:
            f, n = self._fast, len(all_params)
            f["ids_t"] = torch.empty(n, dtype=torch.int64)
            _FS.param_ids(all_params, f["ids_t"])
            f["scan_t"] = torch.empty(n, 3, dtype=torch.int64)
            _FS.scan_params(all_params, f["ids_t"], f["scan_t"])
            scan = f["scan_t"].numpy()
            f["scan"] = scan
            f["mask"] = scan[:, 1] != 0
            f["all_grads"] = bool(f["mask"].all())
            f["p_col"] = scan[:, 0].copy()        # data pointer of every parameter
            f["props_col"] = scan[:, 2].copy()    # gradient properties (0: no gradient)
            f["props_np"] = scan[f["mask"], 2]
            f["ema_ids_t"] = torch.tensor(list(map(id, f["emas"])), dtype=torch.int64)
            f["ema_sq_ids_t"] = torch.tensor(list(map(id, f["ema_sqs"])), dtype=torch.int64)
            f["steps_t"] = torch.tensor(f["steps"], dtype=torch.int64)
            f["gptrs_np"] = np.empty(int(f["mask"].sum()), dtype=np.uint64)
            # what a gradient must look like: dense, contiguous, of a known dtype, on this device
            ok = ((f["props_np"] >> 8) & 3) == 1
            if not bool(ok.all()) or not bool((((f["props_np"] >> 16) & 0xFFFF) == index + 1).all()):
                self._fast = None

    @staticmethod
    def _zero_buffer_count(index):
        return len(SP._PUSH_BUCKETS.get(index, ())), len(SP._PULL_BUCKETS.get(index, ()))

    def _step_fast(self, lib) -> bool:
        f = self._fast
        groups = self.param_groups
        if len(groups) != f["n_groups"] or f["zero_buffers"] != self._zero_buffer_count(f["index"]):
            return False
        if getattr(self.state, "epoch", None) != f["state_epoch"]:
            return False    # a state dict was added, replaced or removed since the cache was armed
        all_params = list(chain.from_iterable(g["params"] for g in groups))
        if _FS is not None and "scan" in f:
            return self._step_fast_scanned(lib, f, groups, all_params)
        if list(map(id, all_params)) != f["all_ids"]:
            return False
        grads_all = [p.grad for p in all_params]
        if [g is not None for g in grads_all] != f["has_grad"]:
            return False
        params, states = f["params"], f["states"]
        grads = [g for g in grads_all if g is not None]
        if list(map(torch.Tensor.data_ptr, params)) != f["p_ptrs"]:
            return False
        if [g.dtype for g in grads] != f["g_dtypes"] or not all(map(torch.Tensor.is_contiguous, grads)):
            return False
        if any(g.is_sparse for g in grads):
            return False
        if not (all(map(operator.is_, map(_GET_EMA, states), f["emas"])) and
                all(map(operator.is_, map(_GET_EMA_SQ, states), f["ema_sqs"]))):
            return False
        steps = list(map(_GET_STEP, states))
        if steps != f["steps"]:
            return False    # a counter was edited in place: rebuild the hyper-parameter classes
        plan = self._plans.get(f["index"])
        if plan is None or len(plan.grad_ptrs) != len(params):
            return False
        for g in groups:
            if g["centralization"] != 0:
                return False
        # nothing structural changed: launch, then advance the counters
        rows = []
        for gi, step in f["classes"]:
            g = groups[gi]
            rows.append(N.make_hyper(g["lr"], g["betas"], g["eps"], g["weight_decay"], step + 1,
                                     g["centralization"], self.reference_order, self.shared_draws))
        hyper_arr = (N.Hyper * len(rows))(*rows)
        gptrs = np.fromiter(map(torch.Tensor.data_ptr, grads), dtype=np.uint64, count=len(grads))
        index = f["index"]
        with (_NULL_CTX if torch.cuda.current_device() == index else torch.cuda.device(index)):
            stream = N.stream_ptr(index)
            N.check(lib.rt_plan_set_grads(plan.handle, gptrs.ctypes.data_as(ctypes.POINTER(N.c_void_p)), stream),
                    "rt_plan_set_grads")
            N.check(lib.rt_adamw_sr_multi(plan.handle, hyper_arr, len(rows), self.seed & (2 ** 64 - 1), stream),
                    "rt_adamw_sr_multi")
        f["classes"] = [(gi, step + 1) for gi, step in f["classes"]]
        f["steps"] = steps = [t + 1 for t in steps]
        for st, t in zip(states, steps):
            st["step"] = t
        for bucket in self._push_marks:
            bucket.pushed = True
        self.last_step_info = dict(launches=plan.launches, resident=len(params), streamed=0, fast=True)
        if self.sync:
            torch.cuda.current_stream(index).synchronize()
        return True

    def _step_fast_scanned(self, lib, f, groups, all_params) -> bool:
        """The same checks as the Python passes of ``_step_fast``, with the per-tensor work done by
        the C++ helper: identity of every parameter, data pointers, which parameters have a
        gradient, each gradient's dtype / contiguity / layout / device, identity of the moment
        tensors and the step counters."""
        if len(all_params) != len(f["all_ids"]) or _FS.scan_params(all_params, f["ids_t"], f["scan_t"]) >= 0:
            return False
        scan, mask = f["scan"], f["mask"]
        # same parameters' storage, same set of parameters with a gradient, same gradient properties
        if not (np.array_equal(scan[:, 0], f["p_col"]) and np.array_equal(scan[:, 2], f["props_col"])):
            return False
        states = f["states"]
        plan = self._plans.get(f["index"])
        if plan is None or len(plan.grad_ptrs) != len(states):
            return False
        for g in groups:
            if g["centralization"] != 0:
                return False
        # moment tensors and counters as cached (a replaced tensor or an in-place edit of a counter ends
        # the fast path); the counters advance in the same pass and are taken back if the launch fails
        if _FS.check_states(states, f["ema_ids_t"], f["ema_sq_ids_t"], f["steps_t"], True, 1) >= 0:
            return False
        rows = []
        for gi, step in f["classes"]:
            g = groups[gi]
            rows.append(N.make_hyper(g["lr"], g["betas"], g["eps"], g["weight_decay"], step + 1,
                                     g["centralization"], self.reference_order, self.shared_draws))
        hyper_arr = (N.Hyper * len(rows))(*rows)
        gptrs = f["gptrs_np"]
        gptrs[:] = scan[:, 1] if f["all_grads"] else scan[mask, 1]
        index = f["index"]
        try:
            with (_NULL_CTX if torch.cuda.current_device() == index else torch.cuda.device(index)):
                stream = N.stream_ptr(index)
                N.check(lib.rt_plan_set_grads(plan.handle, gptrs.ctypes.data_as(ctypes.POINTER(N.c_void_p)), stream),
                        "rt_plan_set_grads")
                N.check(lib.rt_adamw_sr_multi(plan.handle, hyper_arr, len(rows), self.seed & (2 ** 64 - 1), stream),
                        "rt_adamw_sr_multi")
        except Exception:
            _FS.check_states(states, f["ema_ids_t"], f["ema_sq_ids_t"], f["steps_t"], False, -1)
            raise
        f["classes"] = [(gi, step + 1) for gi, step in f["classes"]]
        for bucket in self._push_marks:
            bucket.pushed = True
        self.last_step_info = dict(launches=plan.launches, resident=len(states), streamed=0, fast=True)
        if self.sync:
            torch.cuda.current_stream(index).synchronize()
        return True

    def _row_means(self, lib, index, entries, rows_of, stream):
        """Gradient centralization (adamw.py:179-184): fill a per-device scratch buffer with the
        row means of every centralized gradient; returns {entry position: (address, row_len)}."""
        if not rows_of:
            return {}
        total = sum(rows_of.values())
        scratch = self._row_scratch.get(index)
        if scratch is None or scratch.numel() < total:
            scratch = torch.empty(total, dtype=torch.float32, device=torch.device("cuda", index))
            self._row_scratch[index] = scratch
        info, off = {}, 0
        for k, rows in rows_of.items():
            grad = entries[k][1]
            row_len = grad.numel() // rows if rows else 0
            if rows and row_len:
                addr = scratch.data_ptr() + 4 * off
                N.check(lib.rt_row_means(grad.data_ptr(), N.DTYPE_CODE[grad.dtype], rows, row_len, addr, stream),
                        "rt_row_means")
                info[k] = (addr, row_len if rows > 1 else 0)
            off += rows
        return info

    def _plan_for(self, index, entries, row_info=None) -> _DevicePlan:
        row_info = row_info or {}
        signature = [(pd.data_ptr(), ema.data_ptr(), ema_sq.data_ptr(), pd.numel(), pd.dtype,
                      grad.dtype, ema.dtype, tid, hi, row_info.get(k))
                     for k, (pd, grad, ema, ema_sq, tid, hi) in enumerate(entries)]
        # peer-mapped ZeRO buffers that appear after the plan was built must be picked up
        signature.append(self._zero_buffer_count(index))
        plan = self._plans.get(index)
        if plan is not None and plan.signature == signature:
            return plan
        if plan is not None:
            torch.cuda.current_stream(index).synchronize()
            plan.close()
        descs = []
        for k, (pd, grad, ema, ema_sq, tid, hi) in enumerate(entries):
            d = N.TensorDesc()
            if k in row_info:
                d.row_mean, d.row_len = row_info[k]
            d.p, d.g, d.m, d.v = pd.data_ptr(), grad.data_ptr(), ema.data_ptr(), ema_sq.data_ptr()
            d.numel, d.index0, d.tensor_id, d.hyper_index = pd.numel(), 0, tid, hi
            d.p_dtype, d.g_dtype, d.state_dtype = (N.DTYPE_CODE[pd.dtype], N.DTYPE_CODE[grad.dtype],
                                                   N.DTYPE_CODE[ema.dtype])
            descs.append(d)
        plan = _DevicePlan(index, signature, descs)
        self._plans[index] = plan
        return plan


# The full torch behaviour (profiler range + hook dispatch) around AdamW._step, built once; only
# used by the shortcut in AdamW.step, which exists only when this torch build has every name it
# inspects (otherwise the base class wraps step() itself).
_HOOKED_STEP = Optimizer.profile_hook_step(AdamW._step) if _FAST_DISPATCH else None
