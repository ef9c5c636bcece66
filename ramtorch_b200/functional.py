"""Tensor-level wrappers over the C ABI (one call = one kernel launch sequence).

These take torch tensors only to read their device pointers, dtypes and sizes; all arithmetic
happens in ``librt_b200.so``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native as N


def _need_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: ramtorch_b200 has no CPU implementation")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _code(t: torch.Tensor, name: str) -> int:
    try:
        return N.DTYPE_CODE[t.dtype]
    except KeyError:
        raise ValueError(f"{name}: unsupported dtype {t.dtype} (bf16, fp32, fp16 only)") from None


def sr_round_bf16_(target: torch.Tensor, source: torch.Tensor, *, rand16: torch.Tensor | None = None,
                   seed: int = 0, tensor_id: int = 0, step: int = 0, stream_id: int = 0) -> torch.Tensor:
    """``target <- stochastic_round_bf16(source)`` (the arithmetic of adamw.py:13-30).

    ``rand16`` (int16/uint16, one per element) injects the draws; otherwise they come from the
    Philox stream ``(seed, tensor_id, step, stream_id)``."""
    _need_cuda(target, "target"); _need_cuda(source, "source")
    if target.dtype != torch.bfloat16 or source.dtype != torch.float32:
        raise ValueError("target must be bf16 and source fp32")
    if target.numel() != source.numel():
        raise ValueError("target and source differ in size")
    rp = None
    if rand16 is not None:
        _need_cuda(rand16, "rand16")
        if rand16.element_size() != 2 or rand16.numel() != source.numel():
            raise ValueError("rand16 must hold one 16-bit value per element")
        rp = rand16.data_ptr()
    with torch.cuda.device(source.device):
        N.check(N.lib().rt_sr_round_bf16(target.data_ptr(), source.data_ptr(), source.numel(), rp,
                                         seed & (2**64 - 1), tensor_id, step, stream_id,
                                         N.stream_ptr(source.device)), "rt_sr_round_bf16")
    return target


def row_means(g: torch.Tensor, rows: int, row_len: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 mean of each of the ``rows`` rows of ``row_len`` elements of ``g`` (``rt_row_means``)."""
    _need_cuda(g, "g")
    if rows * row_len != g.numel():
        raise ValueError("rows * row_len must equal g.numel()")
    if out is None:
        out = torch.empty(rows, dtype=torch.float32, device=g.device)
    with torch.cuda.device(g.device):
        N.check(N.lib().rt_row_means(g.data_ptr(), _code(g, "g"), rows, row_len, out.data_ptr(),
                                     N.stream_ptr(g.device)), "rt_row_means")
    return out


def adamw_sr_flat_(p, g, m, v, hyper: N.Hyper, *, seed=0, tensor_id=0, index0=0, row_mean=None, row_len=0,
                   rand=(None, None, None), taps=(None, None, None)) -> None:
    """One fused step over one device-resident tensor, in place (``rt_adamw_sr_flat``).

    ``rand`` / ``taps`` switch the call to the debug kernel: injected 16-bit draws for p, m, v and
    fp32 output buffers receiving the pre-rounding p', m', v'."""
    for t, name in ((p, "p"), (g, "g"), (m, "m"), (v, "v")):
        _need_cuda(t, name)
    n = p.numel()
    if not (g.numel() == m.numel() == v.numel() == n):
        raise ValueError("p, g, m, v differ in size")
    if m.dtype != v.dtype:
        raise ValueError("m and v must share a dtype")
    dbg = None
    if any(x is not None for x in rand) or any(x is not None for x in taps):
        dbg = N.Debug()
        for field, t in zip(("rand_p", "rand_m", "rand_v"), rand):
            if t is not None:
                _need_cuda(t, field)
                if t.element_size() != 2 or t.numel() != n:
                    raise ValueError(f"{field} must hold one 16-bit value per element")
                setattr(dbg, field, t.data_ptr())
        for field, t in zip(("f32_p", "f32_m", "f32_v"), taps):
            if t is not None:
                _need_cuda(t, field)
                if t.dtype != torch.float32 or t.numel() != n:
                    raise ValueError(f"{field} must be fp32 with one value per element")
                setattr(dbg, field, t.data_ptr())
    with torch.cuda.device(p.device):
        N.check(N.lib().rt_adamw_sr_flat(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n,
                                         _code(p, "p"), _code(g, "g"), _code(m, "m"),
                                         ctypes.byref(hyper), seed & (2**64 - 1), tensor_id, index0,
                                         None if row_mean is None else row_mean.data_ptr(), row_len,
                                         ctypes.byref(dbg) if dbg is not None else None,
                                         N.stream_ptr(p.device)), "rt_adamw_sr_flat")
