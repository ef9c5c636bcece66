"""ctypes binding of ``librt_b200.so`` (C ABI in ``include/rt_b200.h``).

Nothing else in the package touches the shared library.  There is no CPU implementation
behind these calls: if the library has not been built the import fails with instructions.
"""
from __future__ import annotations

import ctypes
import os

import torch  # imported first on purpose: the library binds to the CUDA runtime torch loaded

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librt_b200.so")

BF16, F32, F16 = 0, 1, 2
DTYPE_CODE = {torch.bfloat16: BF16, torch.float32: F32, torch.float16: F16}

c_void_p, c_int, c_int64, c_uint64, c_uint32 = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                                ctypes.c_uint64, ctypes.c_uint32)


class Hyper(ctypes.Structure):
    _fields_ = [("beta1", ctypes.c_float), ("one_minus_beta1", ctypes.c_float),
                ("beta2", ctypes.c_float), ("one_minus_beta2", ctypes.c_float),
                ("bias_correction2_sqrt", ctypes.c_float), ("eps", ctypes.c_float),
                ("decay", ctypes.c_float), ("neg_step_size", ctypes.c_float),
                ("centralization", ctypes.c_float), ("apply_decay", c_uint32),
                ("step", c_uint32), ("flags", c_uint32),
                ("inv_bias_correction2_sqrt", ctypes.c_float), ("reserved", c_uint32 * 3)]


HYPER_SHARED_DRAWS = 2
HYPER_REFERENCE_ORDER = 4


class Debug(ctypes.Structure):
    _fields_ = [("rand_p", c_void_p), ("rand_m", c_void_p), ("rand_v", c_void_p),
                ("f32_p", c_void_p), ("f32_m", c_void_p), ("f32_v", c_void_p)]


class TensorDesc(ctypes.Structure):
    _fields_ = [("p", c_void_p), ("g", c_void_p), ("m", c_void_p), ("v", c_void_p),
                ("numel", c_int64), ("index0", c_int64), ("tensor_id", c_uint32),
                ("hyper_index", c_uint32), ("p_dtype", ctypes.c_uint8), ("g_dtype", ctypes.c_uint8),
                ("state_dtype", ctypes.c_uint8), ("reserved0", ctypes.c_uint8), ("row_len", c_uint32),
                ("row_mean", c_void_p)]


class OffloadCfg(ctypes.Structure):
    _fields_ = [("chunk_elems", c_int64), ("ring_depth", c_int), ("defer_join", c_int),
                ("staging", c_void_p), ("staging_bytes", c_int64),
                ("row_mean", c_void_p), ("row_len", c_int64)]


MAX_PEERS = 15


class Push(ctypes.Structure):
    _fields_ = [("local_base", c_void_p), ("bytes", c_int64), ("n_peers", c_int),
                ("peer_base", c_void_p * MAX_PEERS)]


class Pull(ctypes.Structure):
    _fields_ = [("local_base", c_void_p), ("bytes", c_int64), ("n_ranks", c_int), ("self_rank", c_int),
                ("base", c_void_p * (MAX_PEERS + 1))]


class Stats(ctypes.Structure):
    _fields_ = [("kernel_launches", c_uint64), ("h2d_bytes", c_uint64), ("d2h_bytes", c_uint64),
                ("h2d_copies", c_uint64), ("d2h_copies", c_uint64)]


_SIGNATURES = {
    "rt_last_error": (ctypes.c_char_p, []),
    "rt_version": (ctypes.c_char_p, []),
    "rt_hyper_fill": (c_int, [ctypes.POINTER(Hyper)] + [ctypes.c_double] * 6 + [c_uint32]),
    "rt_sr_round_bf16": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_uint64, c_uint32, c_uint32,
                                 c_uint32, c_void_p]),
    "rt_adamw_sr_flat": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                 ctypes.POINTER(Hyper), c_uint64, c_uint32, c_int64, c_void_p, c_int64,
                                 ctypes.POINTER(Debug), c_void_p]),
    "rt_selftest_exact_math": (c_int, [c_void_p, c_void_p]),
    "rt_row_means": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "rt_plan_create": (c_int, [ctypes.POINTER(c_void_p), ctypes.POINTER(TensorDesc), c_int64, c_int]),
    "rt_plan_destroy": (c_int, [c_void_p]),
    "rt_plan_set_grads": (c_int, [c_void_p, ctypes.POINTER(c_void_p), c_void_p]),
    "rt_plan_launches": (c_int, [c_void_p]),
    "rt_adamw_sr_multi": (c_int, [c_void_p, ctypes.POINTER(Hyper), c_int, c_uint64, c_void_p]),
    "rt_plan_set_push": (c_int, [c_void_p, ctypes.POINTER(Push)]),
    "rt_plan_set_pull": (c_int, [c_void_p, ctypes.POINTER(Pull)]),
    "rt_adamw_sr_multi_static": (c_int, [ctypes.POINTER(TensorDesc), c_int64, ctypes.POINTER(Hyper), c_int,
                                         c_uint64, c_void_p]),
    "rt_offload_staging_bytes": (c_int64, [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "rt_adamw_sr_offload": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                    ctypes.POINTER(Hyper), c_uint64, c_uint32,
                                    ctypes.POINTER(OffloadCfg), c_void_p]),
    "rt_offload_join": (c_int, [c_void_p]),
    "rt_host_register": (c_int, [c_void_p, c_int64]),
    "rt_host_unregister": (c_int, [c_void_p]),
    "rt_query_stats": (c_int, [ctypes.POINTER(Stats)]),
}
EXPORTS = tuple(_SIGNATURES)

_lib = None


def lib() -> ctypes.CDLL:
    """Load the library once.  Raises if it has not been built; never falls back."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing. Build it with `python -m ramtorch_b200.csrc.build` "
                "(needs nvcc; targets sm_100a). There is no CPU or PyTorch fallback.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = L
    return _lib


def check(rc: int, what: str = "librt_b200") -> None:
    if rc != 0:
        msg = lib().rt_last_error().decode(errors="replace")
        kind = ValueError if rc < 0 else RuntimeError
        raise kind(f"{what} failed ({rc}): {msg}")


def make_hyper(lr, betas, eps, weight_decay, step, centralization=0.0, reference_order=False,
               shared_draws=False) -> Hyper:
    """The per-step scalars of ``adamw.py:173-188``: Python-double arithmetic written the way the
    reference writes it, then one rounding to fp32 each (what ATen does when a Python scalar
    meets an fp32 tensor)."""
    beta1, beta2 = betas
    bias_correction = 1 - beta1 ** step
    bias_correction_sqrt = (1 - beta2 ** step) ** (1 / 2)
    step_size = lr / bias_correction
    h = Hyper()
    h.beta1, h.one_minus_beta1 = beta1, 1 - beta1
    h.beta2, h.one_minus_beta2 = beta2, 1 - beta2
    h.bias_correction2_sqrt = bias_correction_sqrt
    h.eps = eps
    h.decay = 1 - step_size * weight_decay
    h.neg_step_size = -step_size
    h.centralization = centralization
    h.apply_decay = 1 if weight_decay != 0 else 0
    h.step = step
    h.flags = (HYPER_REFERENCE_ORDER if reference_order else 0) | (HYPER_SHARED_DRAWS if shared_draws else 0)
    h.inv_bias_correction2_sqrt = 1.0 / float(ctypes.c_float(bias_correction_sqrt).value)
    return h


def stats() -> dict:
    s = Stats()
    check(lib().rt_query_stats(ctypes.byref(s)))
    return {k: int(getattr(s, k)) for k, _ in Stats._fields_}


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device) -> int:
    """The current CUDA stream of `device` (index or torch.device) as a raw handle."""
    if _RAW_STREAM is not None and isinstance(device, int):
        return _RAW_STREAM(device)      # same value, without building a torch.cuda.Stream object per call
    return torch.cuda.current_stream(device).cuda_stream


# ------------------------------------------------------------------ tracing
NVTX = os.environ.get("RT_NVTX", "0") == "1"


class _Range:
    """NVTX range around a phase of the step (RT_NVTX=1); free when tracing is off."""

    __slots__ = ("name",)

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if NVTX:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if NVTX:
            torch.cuda.nvtx.range_pop()


def trace(name: str) -> _Range:
    return _Range(name)
