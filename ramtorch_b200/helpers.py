"""Hook-dict protocol used by ZeRO-2 for CPU-resident (``is_ramtorch``) parameters.

Only the two-attribute protocol of the reference (ramtorch/helpers.py:8-50) that
``zero2.setup_grad_sharding_hooks`` relies on and that the reference's ``Linear`` backward consumes
(ramtorch/modules/linear.py:76-94): a tensor carries ``<name>`` (an ``OrderedDict`` id -> callable)
and ``<name>_counter`` (next id).  Of the model-surgery helpers of that file only
``reattach_is_ramtorch_flags`` (helpers.py:229-253) is provided: ZeRO-1/2 here branch on the
per-tensor ``is_ramtorch`` flag, which a deserialised model has lost.
"""
from __future__ import annotations

from collections import OrderedDict
from itertools import chain
from typing import Callable

import torch
from torch import nn

ZERO2_HOOK_NAME = "_ramtorch_zero_2_hooks"


def add_custom_hooks(tensor: torch.Tensor, hook_name: str = "_custom_hooks") -> torch.Tensor:
    """Give ``tensor`` an empty hook dict and its id counter unless it has them already."""
    if not hasattr(tensor, hook_name):
        setattr(tensor, hook_name, OrderedDict())
        setattr(tensor, hook_name + "_counter", 0)
    return tensor


def register_ramtorch_hook(tensor: torch.Tensor, hook: Callable, hook_name: str) -> int:
    """Append ``hook`` to the tensor's hook dict ``hook_name``; returns the integer id under which
    it was stored (ids are never reused)."""
    add_custom_hooks(tensor, hook_name)
    counter_name = hook_name + "_counter"
    hook_id = getattr(tensor, counter_name)
    getattr(tensor, hook_name)[hook_id] = hook
    setattr(tensor, counter_name, hook_id + 1)
    return hook_id


def remove_ramtorch_hook(tensor: torch.Tensor, hook_id: int, hook_name: str) -> bool:
    """Remove a hook by id; returns whether it was present."""
    hooks = getattr(tensor, hook_name, None)
    return hooks is not None and hooks.pop(hook_id, None) is not None


def invoke_ramtorch_hooks(tensor: torch.Tensor, grad: torch.Tensor, hook_name: str = ZERO2_HOOK_NAME):
    """Run the hook dict the way the reference's backward does (linear.py:76-94): every hook sees the
    current gradient, a non-``None`` result replaces it."""
    for hook in getattr(tensor, hook_name, {}).values():
        out = hook(grad)
        if out is not None:
            grad = out
    return grad


def reattach_is_ramtorch_flags(module: nn.Module) -> nn.Module:
    """Put ``is_ramtorch = True`` back on the parameters and buffers that directly belong to any
    sub-module (``module`` itself included) which declares ``is_ramtorch = True``
    (helpers.py:229-253).

    Tensor attributes do not survive ``torch.save`` / ``torch.load`` or ``copy.deepcopy``; the
    module attribute does (``Linear`` sets it as a class-level flag, linear.py).  Call this after
    rebuilding a model and BEFORE ``create_zero_param_groups`` / ``setup_grad_sharding_hooks``:
    both treat a parameter without the flag as an ordinary HBM tensor (flat buffer + collective)
    instead of CPU storage shared by all workers (zero1.py:81, zero2.py:67-72).  Returns
    ``module``."""
    for sub in module.modules():
        if not getattr(sub, "is_ramtorch", False):
            continue
        for tensor in chain(sub.parameters(recurse=False), sub.buffers(recurse=False)):
            if isinstance(tensor, torch.Tensor):
                tensor.is_ramtorch = True
    return module


DEVICE_GRAD_ATTR = "rt_device_grad"


def accumulate_device_grad(param: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
    """Producer side of the gradient hand-off for CPU-resident (``is_ramtorch``) parameters.

    The reference's ``Linear`` backward copies each weight gradient to host memory
    (``weight_cpu.grad = w_grad.to("cpu")``, linear.py:416-427) only for ``AdamW.step`` to copy it
    back to the GPU (adamw.py:167).  A backward that calls this instead leaves the gradient in HBM:
    the first micro-batch stores it on the parameter as ``rt_device_grad``, later ones add to it in
    place (what ``Tensor.grad`` accumulation does; PyTorch itself refuses a CUDA ``.grad`` on a CPU
    tensor), ``AdamW.step`` consumes it in preference to ``p.grad`` and ``AdamW.zero_grad`` clears
    it.  ``grad`` must be a CUDA tensor of the parameter's shape that the caller will not reuse (or
    a clone).  Returns the accumulated gradient."""
    if not grad.is_cuda:
        raise ValueError("accumulate_device_grad is for gradients that live in HBM")
    if grad.shape != param.shape:
        raise ValueError("gradient and parameter shapes differ")
    held = param.__dict__.get(DEVICE_GRAD_ATTR)
    if held is None:
        held = grad.detach()
        setattr(param, DEVICE_GRAD_ATTR, held)
    else:
        held.add_(grad.detach())
    return held
