"""The multi-tensor step that never allocates (``rt_adamw_sr_multi_static``).

Who needs it: a program that has given all of its device memory to its own pool, or that runs the
optimizer inside a phase where the CUDA allocator must not be called, cannot use ``rt_plan_create``
(which keeps its tables in ``cudaMalloc`` memory).  The static entry point keeps the same tables in a
fixed array inside the library image instead.  Here it is called through the C ABI on two steps in
a row and must reproduce, bit for bit, what the plan-based entry point writes for the same inputs.
This file is named so that pytest collects it last."""
import ctypes

import numpy as np
import pytest
import torch

from ramtorch_b200 import _native as N

HP = dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


def _descs(tensors):
    arr = (N.TensorDesc * len(tensors))()
    for k, (p, g, m, v) in enumerate(tensors):
        d = arr[k]
        d.p, d.g, d.m, d.v = p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr()
        d.numel, d.index0, d.tensor_id, d.hyper_index = p.numel(), 0, 100 + k, k % 2
        d.p_dtype, d.g_dtype, d.state_dtype = N.DTYPE_CODE[p.dtype], N.DTYPE_CODE[g.dtype], N.DTYPE_CODE[m.dtype]
    return arr


def _make(dev, seed):
    gen = torch.Generator().manual_seed(seed)
    spec = [(64, torch.bfloat16, torch.bfloat16), (8192 * 3 + 5, torch.bfloat16, torch.float32),
            (1000, torch.float32, torch.float32), (40000, torch.bfloat16, torch.bfloat16),
            (7, torch.bfloat16, torch.float32), (123457, torch.bfloat16, torch.bfloat16)]
    out = []
    for n, pdt, sdt in spec:
        p = (torch.randn(n, generator=gen) * 0.02).to(pdt).to(dev)
        g = (torch.randn(n, generator=gen) * 1e-3).to(pdt).to(dev)
        m = (torch.randn(n, generator=gen) * 1e-3).to(sdt).to(dev)
        v = (torch.randn(n, generator=gen) * 1e-6).abs().to(sdt).to(dev)
        out.append((p, g, m, v))
    return out


def _bits(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16 if t.element_size() == 2 else torch.int32).numpy()


@pytest.mark.gpu
def test_static_entry_point_matches_the_plan_entry_point_on_two_consecutive_steps():
    lib = N.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    a, b = _make(dev, 5), _make(dev, 5)          # two identical copies of the same problem
    da, db = _descs(a), _descs(b)
    stream = N.stream_ptr(dev)
    plan = ctypes.c_void_p()
    N.check(lib.rt_plan_create(ctypes.byref(plan), da, len(a), 0), "rt_plan_create")
    try:
        for step in (7, 8):                      # two calls in a row share the static tables
            hyper = (N.Hyper * 2)(N.make_hyper(step=step, **HP),
                                  N.make_hyper(step=step, **{**HP, "lr": 3e-4, "weight_decay": 0.0}))
            N.check(lib.rt_adamw_sr_multi(plan, hyper, 2, 99, stream), "rt_adamw_sr_multi")
            N.check(lib.rt_adamw_sr_multi_static(db, len(b), hyper, 2, 99, stream), "rt_adamw_sr_multi_static")
            torch.cuda.synchronize()
            for (pa, _, ma, va), (pb, _, mb, vb) in zip(a, b):
                assert np.array_equal(_bits(pa), _bits(pb))
                assert np.array_equal(_bits(ma), _bits(mb))
                assert np.array_equal(_bits(va), _bits(vb))
        assert not np.array_equal(_bits(a[0][0]), _bits(_make(dev, 5)[0][0]))   # the steps did change p
    finally:
        lib.rt_plan_destroy(plan)


def test_static_entry_point_rejects_requests_beyond_its_fixed_tables():
    """Host-side checks only: nothing is launched, so this part needs no GPU."""
    lib = N.lib()
    buf = (ctypes.c_uint8 * 64)()
    ptr = ctypes.addressof(buf)
    h = (N.Hyper * 1)(N.make_hyper(step=1, **HP))
    too_many = (N.TensorDesc * 1025)()
    assert lib.rt_adamw_sr_multi_static(too_many, 1025, h, 1, 0, None) == -3
    assert b"at most 1024 tensors" in lib.rt_last_error()
    one = (N.TensorDesc * 1)()
    one[0].p = one[0].g = one[0].m = one[0].v = ptr
    one[0].numel = 8192 * 65536 + 1            # one chunk more than the chunk table holds
    assert lib.rt_adamw_sr_multi_static(one, 1, h, 1, 0, None) == -3
    assert b"65536 chunks" in lib.rt_last_error()
    assert lib.rt_adamw_sr_multi_static(one, 1, h, 65, 0, None) == -3
    assert lib.rt_adamw_sr_multi_static(one, 0, h, 1, 0, None) == 0
