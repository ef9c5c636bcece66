"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments on the host (these calls return before touching a device)."""
import ctypes
import os
import re

import pytest

from ramtorch_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "rt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rt_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = header_symbols()
    assert len(names) >= 14
    lib = ctypes.CDLL(N.LIB_PATH)
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/rt_b200.h but not exported"
    assert set(names) == set(N.EXPORTS)


def test_struct_sizes_match_header():
    assert ctypes.sizeof(N.Hyper) == 64
    assert ctypes.sizeof(N.TensorDesc) == 72
    assert ctypes.sizeof(N.Debug) == 48
    assert ctypes.sizeof(N.OffloadCfg) == 48
    assert ctypes.sizeof(N.Stats) == 40


def test_version_and_hyper_fill():
    lib = N.lib()
    assert b"sm_100a" in lib.rt_version()
    for step in (1, 11, 100):
        a = N.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, step)
        b = N.Hyper()
        assert lib.rt_hyper_fill(ctypes.byref(b), 1e-4, 0.9, 0.999, 1e-8, 0.01, 0.0, step) == 0
        assert bytes(a) == bytes(b)


def test_argument_errors_are_reported_before_any_launch():
    lib = N.lib()
    h = N.make_hyper(1e-3, (0.9, 0.999), 1e-8, 0.0, 1)
    buf = (ctypes.c_uint8 * 64)()
    ptr = ctypes.addressof(buf)
    hp = ctypes.byref(h)
    assert lib.rt_adamw_sr_flat(None, ptr, ptr, ptr, 8, 0, 0, 0, hp, 0, 0, 0, None, 0, None, None) == -1
    assert b"non-null" in lib.rt_last_error()
    assert lib.rt_adamw_sr_flat(ptr, ptr, ptr, ptr, 8, 0, 7, 0, hp, 0, 0, 0, None, 0, None, None) == -2
    assert lib.rt_adamw_sr_flat(ptr, ptr, ptr, ptr, -1, 0, 0, 0, hp, 0, 0, 0, None, 0, None, None) == -3
    assert lib.rt_adamw_sr_flat(ptr, ptr, ptr, ptr, 8, 0, 0, 0, hp, 0, 0, 4, None, 0, None, None) == -3
    assert lib.rt_adamw_sr_flat(ptr + 1, ptr, ptr, ptr, 8, 0, 0, 0, hp, 0, 0, 0, None, 0, None, None) == -4
    assert lib.rt_adamw_sr_flat(ptr, ptr, ptr, ptr, 8, 0, 0, 0, None, 0, 0, 0, None, 0, None, None) == -1
    assert lib.rt_sr_round_bf16(None, ptr, 8, None, 0, 0, 0, 0, None) == -1
    assert lib.rt_plan_destroy(None) == -5
    assert lib.rt_offload_staging_bytes(12, 3, 0, 0, 0, 1, 1, 1, 1) == -6
    assert lib.rt_offload_staging_bytes(1024, 3, 0, 0, 1, 1, 0, 1, 1) == 3 * (2048 + 4096 + 4096)
    with pytest.raises(ValueError):
        N.check(-3)


def test_zero_length_calls_are_noops():
    lib = N.lib()
    h = N.make_hyper(1e-3, (0.9, 0.999), 1e-8, 0.0, 1)
    buf = (ctypes.c_uint8 * 64)()
    ptr = ctypes.addressof(buf)
    assert lib.rt_adamw_sr_flat(ptr, ptr, ptr, ptr, 0, 0, 0, 0, ctypes.byref(h), 0, 0, 0, None, 0, None, None) == 0
    assert lib.rt_sr_round_bf16(ptr, ptr, 0, None, 0, 0, 0, 0, None) == 0
