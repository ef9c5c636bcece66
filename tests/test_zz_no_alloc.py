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


def _np_bits(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).ravel().copy()
    return t.numpy().ravel().copy()


@pytest.mark.gpu
def test_static_entry_point_against_the_cpu_checker_and_without_touching_the_allocator():
    """The same call checked on its own terms: its output equals the CPU checker's bit for bit
    (ragged sizes with scalar tails, three dtype combinations, six hyper rows -- more than ride
    along as kernel arguments on the plan path), a second call with a different, shorter tensor
    list reuses the shared tables correctly, and neither call changes what the CUDA allocator or
    PyTorch's caching allocator hold."""
    import oracle
    lib = N.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = N.stream_ptr(dev)
    code = {torch.bfloat16: oracle.BF16, torch.float32: oracle.F32}

    def run(tensors, step, seed):
        rows = [dict(HP, lr=1e-4 * (k + 1), weight_decay=0.01 * (k % 2)) for k in range(6)]
        hyper = (N.Hyper * 6)(*[N.make_hyper(step=step, **r) for r in rows])
        descs = _descs(tensors)
        for k in range(len(tensors)):
            descs[k].hyper_index = k % 6
        want = []
        for k, (p, g, m, v) in enumerate(tensors):       # the checker's answer, before the GPU overwrites the inputs
            hp, hg, hm, hv = (_np_bits(t) for t in (p, g, m, v))
            oracle.adamw_sr(hp, hg, hm, hv, code[p.dtype], code[g.dtype], code[m.dtype],
                            oracle.make_hyper(step=step, **rows[k % 6]), seed=seed, tensor_id=100 + k)
            want.append((hp, hm, hv))
        torch.cuda.synchronize()
        free0, alloc0, reserved0 = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
        N.check(lib.rt_adamw_sr_multi_static(descs, len(tensors), hyper, 6, seed, stream), "rt_adamw_sr_multi_static")
        torch.cuda.synchronize()
        after = (torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev))
        for (p, _, m, v), (wp, wm, wv) in zip(tensors, want):
            assert np.array_equal(_np_bits(p), wp) and np.array_equal(_np_bits(m), wm) and np.array_equal(_np_bits(v), wv)
        return (free0, alloc0, reserved0), after

    first = _make(dev, 11)
    run(first, 3, 1234)                 # warm-up call: looks up the array's address, loads the kernels' code
    before, after = run(first, 4, 1234)
    assert before == after              # nothing allocated or freed by the call, by anyone
    shorter = _make(dev, 12)[1:4]       # a different, shorter list right behind it on the same stream
    before, after = run(shorter, 9, 77)
    assert before == after


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
    # a hyper row that asks for centralization needs the tensor's row means, as on the plan path
    one[0].numel = 64
    c = (N.Hyper * 1)(N.make_hyper(step=1, centralization=0.5, **HP))
    assert lib.rt_adamw_sr_multi_static(one, 1, c, 1, 0, None) == -6
    assert b"row_mean" in lib.rt_last_error()
    # flag bits the library does not know are refused, not ignored
    bad = (N.Hyper * 1)(N.make_hyper(step=1, **HP))
    bad[0].flags = 1
    assert lib.rt_adamw_sr_multi_static(one, 1, bad, 1, 0, None) == -6
