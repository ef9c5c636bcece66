"""CPU checker for the SR-AdamW step — TEST INFRASTRUCTURE, not product code.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this package; the product package never does.

The arithmetic lives in ``sr_adamw_oracle.c`` (plain C, compiled by ``build_oracle.py``); this
module is the numpy/ctypes face of it plus two tiny pure-numpy restatements (``philox_np``,
``sr_round_np``) used to cross-check the C code on small inputs.

What is pinned: the fp32 update and the (fp32 bits, r16) -> bf16 map, against the outputs of the
reference's own ``AdamW.step`` / ``copy_stochastic_`` run on the CPU (``tests/golden``).
What is not: the reference's random bit stream (torch.Generator), replaced on purpose by the
counter-based Philox stream of ``include/rt_b200.h``; Philox itself is pinned against the
Random123 known-answer vectors.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build_oracle

BF16, F32, F16 = 0, 1, 2
_NP_OF = {BF16: np.uint16, F32: np.float32, F16: np.float16}


class Hyper(ctypes.Structure):
    """Mirror of ``rt_hyper`` (include/rt_b200.h)."""

    _fields_ = [
        ("beta1", ctypes.c_float),
        ("one_minus_beta1", ctypes.c_float),
        ("beta2", ctypes.c_float),
        ("one_minus_beta2", ctypes.c_float),
        ("bias_correction2_sqrt", ctypes.c_float),
        ("eps", ctypes.c_float),
        ("decay", ctypes.c_float),
        ("neg_step_size", ctypes.c_float),
        ("centralization", ctypes.c_float),
        ("apply_decay", ctypes.c_uint32),
        ("step", ctypes.c_uint32),
        ("flags", ctypes.c_uint32),
        ("inv_bias_correction2_sqrt", ctypes.c_float),
        ("reserved", ctypes.c_uint32 * 3),
    ]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = build_oracle.build()
        L = ctypes.CDLL(path)
        vp, i64, u64, u32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64, ctypes.c_uint32
        L.rto_philox4x32_10.argtypes = [vp, vp, vp]
        L.rto_philox4x32_10.restype = None
        L.rto_draws.argtypes = [u64, u32, u32, u32, i64, i64, vp]
        L.rto_draws.restype = None
        L.rto_sr_round_bf16.argtypes = [vp, vp, vp, i64]
        L.rto_sr_round_bf16.restype = None
        L.rto_adamw_sr.argtypes = [vp, vp, vp, vp, i64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                   ctypes.POINTER(Hyper), u64, u32, i64, vp, i64,
                                   vp, vp, vp, vp, vp, vp]
        L.rto_adamw_sr.restype = ctypes.c_int
        L.rto_hyper_fill.argtypes = [ctypes.POINTER(Hyper)] + [ctypes.c_double] * 6 + [u32]
        L.rto_hyper_fill.restype = None
        L.rto_num_threads.restype = ctypes.c_int
        L.rto_set_num_threads.argtypes = [ctypes.c_int]
        L.rto_set_num_threads.restype = None
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().rto_num_threads())


def use_all_cores() -> int:
    """Let the timed baseline use every core this process may run on, whatever OMP_NUM_THREADS
    says (launchers such as torchrun export OMP_NUM_THREADS=1 to every rank)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().rto_set_num_threads(n)
    return num_threads()


def make_hyper(lr, betas, eps, weight_decay, step, centralization=0.0, shared_draws=False,
               reference_order=False) -> Hyper:
    """Per-step scalars exactly as adamw.py:173-188 forms them (Python doubles), each rounded
    once to fp32 where ATen would cast the Python scalar to the tensor's dtype."""
    beta1, beta2 = betas
    bias_correction = 1 - beta1 ** step
    bias_correction_sqrt = (1 - beta2 ** step) ** (1 / 2)
    step_size = lr / bias_correction
    h = Hyper()
    h.beta1 = beta1
    h.one_minus_beta1 = 1 - beta1
    h.beta2 = beta2
    h.one_minus_beta2 = 1 - beta2
    h.bias_correction2_sqrt = bias_correction_sqrt
    h.eps = eps
    h.decay = 1 - step_size * weight_decay
    h.neg_step_size = -step_size
    h.centralization = centralization
    h.apply_decay = 1 if weight_decay != 0 else 0
    h.step = step
    h.flags = (2 if shared_draws else 0) | (4 if reference_order else 0)
    h.inv_bias_correction2_sqrt = 1.0 / float(ctypes.c_float(bias_correction_sqrt).value)
    return h


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _check(a, dtype_code, n, name):
    want = _NP_OF[dtype_code]
    if a.dtype != want or not a.flags["C_CONTIGUOUS"] or a.size != n:
        raise ValueError(f"{name}: want contiguous {np.dtype(want)} of {n} elements, got {a.dtype} {a.shape}")


def adamw_sr(p, g, m, v, p_dtype, g_dtype, state_dtype, hyper: Hyper, seed=0, tensor_id=0,
             index0=0, row_mean=None, row_len=0, rand=(None, None, None), want_f32=False):
    """In-place step on numpy arrays (bf16 carried as uint16 bit patterns).

    Returns ``(f32_p, f32_m, f32_v)`` pre-rounding values when ``want_f32`` else ``None``."""
    n = p.size
    _check(p, p_dtype, n, "p"); _check(g, g_dtype, n, "g")
    _check(m, state_dtype, n, "m"); _check(v, state_dtype, n, "v")
    taps = [np.empty(n, np.float32) for _ in range(3)] if want_f32 else [None] * 3
    for r in rand:
        if r is not None:
            _check(r, BF16, n, "rand")
    if row_mean is not None:
        row_mean = np.ascontiguousarray(row_mean, np.float32)
    rc = lib().rto_adamw_sr(_ptr(p), _ptr(g), _ptr(m), _ptr(v), n, p_dtype, g_dtype, state_dtype,
                            ctypes.byref(hyper), seed, tensor_id, index0, _ptr(row_mean), row_len,
                            _ptr(rand[0]), _ptr(rand[1]), _ptr(rand[2]),
                            _ptr(taps[0]), _ptr(taps[1]), _ptr(taps[2]))
    if rc != 0:
        raise RuntimeError(f"rto_adamw_sr failed: {rc}")
    return tuple(taps) if want_f32 else None


def draws(seed, tensor_id, step, stream, index0, n) -> np.ndarray:
    out = np.empty(n, np.uint16)
    lib().rto_draws(seed, tensor_id, step, stream, index0, n, _ptr(out))
    return out


def sr_round_bf16(source_f32: np.ndarray, rand16: np.ndarray) -> np.ndarray:
    src = np.ascontiguousarray(source_f32, np.float32).ravel()
    r = np.ascontiguousarray(rand16, np.uint16).ravel()
    out = np.empty(src.size, np.uint16)
    lib().rto_sr_round_bf16(_ptr(out), _ptr(src), _ptr(r), src.size)
    return out


def philox_c(ctr, key) -> np.ndarray:
    c = np.asarray(ctr, np.uint32); k = np.asarray(key, np.uint32); o = np.empty(4, np.uint32)
    lib().rto_philox4x32_10(_ptr(c), _ptr(k), _ptr(o))
    return o


# ------------------------------------------------------------------ pure-numpy cross-checks
def philox_np(ctr, key, rounds=10) -> np.ndarray:
    """Philox4x32 on arrays of counters: ctr (..., 4) uint32, key (2,) uint32."""
    c = np.asarray(ctr, np.uint64) & 0xFFFFFFFF
    c0, c1, c2, c3 = (c[..., i].copy() for i in range(4))
    k0, k1 = int(key[0]), int(key[1])
    for _ in range(rounds):
        p0 = 0xD2511F53 * c0
        p1 = 0xCD9E8D57 * c2
        n0 = (p1 >> 32) ^ c1 ^ k0
        n2 = (p0 >> 32) ^ c3 ^ k1
        c0, c1, c2, c3 = n0, p1 & 0xFFFFFFFF, n2, p0 & 0xFFFFFFFF
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], -1).astype(np.uint32)


def draws_np(seed, tensor_id, step, stream, index0, n) -> np.ndarray:
    i = np.arange(index0, index0 + n, dtype=np.int64)
    ctr = np.stack([(i >> 3) & 0xFFFFFFFF, np.full(n, tensor_id), np.full(n, step), np.full(n, stream)], -1)
    out = philox_np(ctr, (seed & 0xFFFFFFFF, seed >> 32))
    j = i & 7
    w = out[np.arange(n), j >> 1]
    return np.where(j & 1, w >> 16, w & 0xFFFF).astype(np.uint16)


def sr_round_np(source_f32: np.ndarray, rand16: np.ndarray) -> np.ndarray:
    """adamw.py:13-30 in numpy: wrapping int32 add of the draw, mask, keep the high half."""
    bits = np.ascontiguousarray(source_f32, np.float32).view(np.uint32).astype(np.uint64)
    return ((((bits + rand16.astype(np.uint64)) & 0xFFFFFFFF) & 0xFFFF0000) >> 16).astype(np.uint16)


# ------------------------------------------------------------------ bf16 <-> numpy helpers
def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits_rn(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (input synthesis only)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u >> 16) & 1) + 0x7FFF
    return (((u + r) & 0xFFFFFFFF) >> 16).astype(np.uint16)
