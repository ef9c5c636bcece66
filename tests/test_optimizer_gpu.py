"""GPU: the drop-in ``AdamW`` class against the CPU checker over several steps, on ragged
multi-tensor lists, with HBM-resident and host-resident (streamed) parameters and moments."""
import numpy as np
import pytest
import torch

import oracle
from util import CODE, bits_equal, to_numpy

pytestmark = pytest.mark.gpu
KIND = {torch.bfloat16: "bf16", torch.float32: "f32", torch.float16: "f16"}


def make_params(shapes, dtype, device, seed=0, pin=False):
    g = torch.Generator().manual_seed(seed)
    out = []
    for s in shapes:
        t = (torch.randn(s, generator=g) * 0.02).to(dtype)
        if device == "cpu":
            t = t.pin_memory() if pin else t
        else:
            t = t.to(device)
        out.append(t)
    return out


def make_grads(shapes, dtype, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return [(torch.randn(s, generator=g) * 1e-3).to(dtype) for s in shapes]


class Mirror:
    """The same optimisation carried out by the CPU checker, tensor by tensor."""

    def __init__(self, params, state_dtype, seed, ids=None, shared_draws=True, **hp):
        self.shared_draws = shared_draws      # AdamW's default
        self.p = [to_numpy(p) for p in params]
        self.kp = [KIND[p.dtype] for p in params]
        self.ks = KIND[state_dtype]
        sdt = np.uint16 if self.ks == "bf16" else (np.float32 if self.ks == "f32" else np.float16)
        self.m = [np.zeros(p.size, sdt) for p in self.p]
        self.v = [np.zeros(p.size, sdt) for p in self.p]
        self.step = [0] * len(params)
        self.seed, self.hp = seed, hp
        self.ids = ids or list(range(len(params)))

    def apply(self, grads, skip=()):
        for k, g in enumerate(grads):
            if k in skip:
                continue
            self.step[k] += 1
            h = oracle.make_hyper(self.hp["lr"], self.hp["betas"], self.hp["eps"], self.hp["weight_decay"], self.step[k],
                                  shared_draws=self.shared_draws)
            oracle.adamw_sr(self.p[k], to_numpy(g), self.m[k], self.v[k], CODE[self.kp[k]], CODE[KIND[g.dtype]],
                            CODE[self.ks], h, seed=self.seed, tensor_id=self.ids[k])


SHAPES = [(64,), (1000,), (37, 111), (8192,), (3, 5, 7), (1,), (20000,), (129, 64)]
HP = dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


def check(opt, params, mirror):
    for k, p in enumerate(params):
        assert bits_equal(to_numpy(p), mirror.p[k]) == 0, f"param {k}"
        st = opt.state[p]
        assert st["step"] == mirror.step[k]
        assert bits_equal(to_numpy(st["ema"]), mirror.m[k]) == 0, f"ema {k}"
        assert bits_equal(to_numpy(st["ema_squared"]), mirror.v[k]) == 0, f"ema_squared {k}"
        assert st["ema"].shape == p.shape and st["ema_squared"].shape == p.shape


@pytest.mark.parametrize("shared", [True, False], ids=["shared-draws", "independent-draws"])
@pytest.mark.parametrize("state_dtype", [torch.bfloat16, torch.float32])
def test_resident_multi_tensor_steps(state_dtype, shared):
    from ramtorch_b200 import AdamW
    params = make_params(SHAPES, torch.bfloat16, "cuda")
    opt = AdamW(params, dtype=state_dtype, storage_device="cuda", seed=11, shared_draws=shared, **HP)
    mirror = Mirror(params, state_dtype, 11, shared_draws=shared, **HP)
    for s in range(4):
        grads = make_grads(SHAPES, torch.bfloat16, s)
        skip = {2} if s == 1 else set()   # a parameter without a gradient is skipped, its step stays
        for k, (p, g) in enumerate(zip(params, grads)):
            p.grad = None if k in skip else g.cuda()
        opt.step()
        mirror.apply(grads, skip)
        check(opt, params, mirror)
    assert opt.last_step_info["launches"] == 1
    assert opt.last_step_info["resident"] == len(SHAPES)


def test_mixed_dtypes_use_one_launch_per_combination():
    from ramtorch_b200 import AdamW
    shapes = SHAPES[:6]
    dts = [torch.bfloat16, torch.float32, torch.bfloat16, torch.float16, torch.float32, torch.bfloat16]
    params = [make_params([s], dt, "cuda", seed=k)[0] for k, (s, dt) in enumerate(zip(shapes, dts))]
    opt = AdamW(params, dtype=torch.float32, storage_device="cuda", **HP)
    mirror = Mirror(params, torch.float32, 0, **HP)
    for s in range(2):
        grads = [make_grads([sh], dt, 10 * s + k)[0] for k, (sh, dt) in enumerate(zip(shapes, dts))]
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step()
        mirror.apply(grads)
        check(opt, params, mirror)
    assert opt.last_step_info["launches"] == 3


def test_param_groups_with_their_own_hyper_parameters_and_lr_schedule():
    from ramtorch_b200 import AdamW
    a = make_params(SHAPES[:3], torch.bfloat16, "cuda", seed=1)
    b = make_params(SHAPES[3:6], torch.bfloat16, "cuda", seed=2)
    opt = AdamW([{"params": a, "weight_decay": 0.0}, {"params": b, "lr": 3e-4}],
                dtype=torch.bfloat16, storage_device="cuda", seed=5, **HP)
    ma = Mirror(a, torch.bfloat16, 5, ids=[0, 1, 2], **{**HP, "weight_decay": 0.0})
    mb = Mirror(b, torch.bfloat16, 5, ids=[3, 4, 5], **{**HP, "lr": 3e-4})
    for s in range(3):
        ga, gb = make_grads(SHAPES[:3], torch.bfloat16, s), make_grads(SHAPES[3:6], torch.bfloat16, 50 + s)
        for p, g in zip(a + b, ga + gb):
            p.grad = g.cuda()
        # a scheduler mutates group["lr"] between steps (re-read every step, adamw.py:174)
        opt.param_groups[1]["lr"] = 3e-4 * (0.5 ** s)
        mb.hp["lr"] = 3e-4 * (0.5 ** s)
        opt.step()
        ma.apply(ga); mb.apply(gb)
        check(opt, a, ma); check(opt, b, mb)


def test_default_pinned_cpu_state_streams_and_matches_resident_state():
    """storage_device="cpu" (the reference default): moments in pinned host RAM, parameters in
    HBM.  Same seed -> bit-identical to the all-resident run."""
    from ramtorch_b200 import AdamW
    shapes = SHAPES + [(300001,)]
    params = make_params(shapes, torch.bfloat16, "cuda")
    opt = AdamW(params, **HP, seed=3, offload_chunk_elems=65536)   # dtype=bf16, storage_device="cpu"
    assert all(opt.state[p]["ema"].is_pinned() and opt.state[p]["ema"].device.type == "cpu" for p in params)
    mirror = Mirror(params, torch.bfloat16, 3, **HP)
    for s in range(3):
        grads = make_grads(shapes, torch.bfloat16, s)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step()
        mirror.apply(grads)
        check(opt, params, mirror)
    assert opt.last_step_info["streamed"] == len(shapes)


@pytest.mark.parametrize("pin", [True, False])
def test_cpu_parameters_and_gradients_stream_through_the_gpu(pin):
    """Parameters, gradients and moments all in host RAM (the ramtorch.Linear convention)."""
    import warnings
    from ramtorch_b200 import AdamW
    shapes = [(1000,), (70001,), (64, 33), (200000,)]
    params = make_params(shapes, torch.bfloat16, "cpu", pin=pin)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = AdamW(params, dtype=torch.float32, **HP, seed=9, offload_chunk_elems=32768, offload_ring_depth=2)
        mirror = Mirror(params, torch.float32, 9, **HP)
        for s in range(3):
            grads = make_grads(shapes, torch.bfloat16, s)
            for p, g in zip(params, grads):
                p.grad = g.pin_memory() if pin else g
            opt.step()
            mirror.apply(grads)
            check(opt, params, mirror)


def test_state_dict_round_trip_and_late_parameters():
    from ramtorch_b200 import AdamW
    params = make_params(SHAPES[:4], torch.bfloat16, "cuda")
    opt = AdamW(params, dtype=torch.bfloat16, storage_device="cuda", **HP)
    mirror = Mirror(params, torch.bfloat16, 0, **HP)
    grads = make_grads(SHAPES[:4], torch.bfloat16, 0)
    for p, g in zip(params, grads):
        p.grad = g.cuda()
    opt.step(); mirror.apply(grads)
    sd = opt.state_dict()
    assert set(sd["state"][0].keys()) == {"step", "ema", "ema_squared"}
    opt2 = AdamW(params, dtype=torch.bfloat16, storage_device="cuda", **HP)
    opt2.load_state_dict(sd)
    grads = make_grads(SHAPES[:4], torch.bfloat16, 1)
    for p, g in zip(params, grads):
        p.grad = g.cuda()
    opt2.step(); mirror.apply(grads)
    check(opt2, params, mirror)
    # a group added after construction gets its state lazily and the next free tensor id
    late = make_params([(555,)], torch.bfloat16, "cuda", seed=77)
    opt2.add_param_group({"params": late})
    ml = Mirror(late, torch.bfloat16, 0, ids=[4], **HP)
    gl = make_grads([(555,)], torch.bfloat16, 5)
    for p in params:
        p.grad = None
    late[0].grad = gl[0].cuda()
    opt2.step(); ml.apply(gl)
    check(opt2, late, ml)


def test_errors():
    from ramtorch_b200 import AdamW
    p = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    opt = AdamW([p], storage_device="cuda")
    p.grad = torch.sparse_coo_tensor(torch.tensor([[1]]), torch.tensor([1.0]), (16,), device="cuda").to(torch.bfloat16)
    with pytest.raises(RuntimeError, match="sparse"):
        opt.step()
    q = torch.zeros(16, dtype=torch.float64, device="cuda")
    opt = AdamW([q], storage_device="cuda")
    q.grad = torch.zeros_like(q)
    with pytest.raises(ValueError):
        opt.step()


def test_copy_stochastic_drop_in():
    from ramtorch_b200 import copy_stochastic_
    src = torch.randn(4097, device="cuda")
    dst = torch.empty(4097, dtype=torch.bfloat16, device="cuda")
    copy_stochastic_(dst, src, seed=53)
    r = oracle.draws(53, 0, 0, 0, 0, 4097)
    assert (to_numpy(dst) == oracle.sr_round_bf16(src.cpu().numpy(), r)).all()


@pytest.mark.parametrize("where", ["all-in-hbm", "moments-on-host", "everything-on-host"])
@pytest.mark.parametrize("name", ["step_bf16_centralized_2d.npz", "step_bf16_centralized_1d.npz"])
def test_centralization_through_the_optimizer_against_the_reference_fixture(name, where):
    """adamw.py:179-184 via ``AdamW(centralization=c)``: one step from the recorded inputs lands
    within the fp32 tolerance of what the reference produced (its row means are summed in another
    order, so bit equality is not expected).  With the reference's default ``storage_device="cpu"``
    the moments, and in the last case parameter and gradient too, are streamed in chunks much
    shorter than the tensor: the row means come from a pass over the whole gradient first."""
    from ramtorch_b200 import AdamW
    from util import TORCH_DT, load_golden, to_torch
    d = load_golden(name)
    meta = d["meta"]
    dev = torch.device("cuda") if where != "everything-on-host" else torch.device("cpu")
    shape = tuple(meta["shape"])
    p = to_torch(d["in_p"], meta["p_dtype"], dev).reshape(shape)
    p.grad = to_torch(d["in_g"], meta["g_dtype"], dev).reshape(shape)
    if where == "everything-on-host":
        p, g = p.pin_memory(), p.grad.pin_memory()
        p.grad = g
    opt = AdamW([p], lr=meta["lr"], betas=tuple(meta["betas"]), eps=meta["eps"], weight_decay=meta["weight_decay"],
                centralization=meta["centralization"], dtype=TORCH_DT[meta["state_dtype"]],
                storage_device="cuda" if where == "all-in-hbm" else "cpu", offload_chunk_elems=1024)
    st = opt.state[p]
    st["ema"].copy_(to_torch(d["in_m"], meta["state_dtype"], dev).reshape(shape))
    st["ema_squared"].copy_(to_torch(d["in_v"], meta["state_dtype"], dev).reshape(shape))
    st["step"] = meta["step"] - 1
    opt.step()
    assert opt.last_step_info["streamed"] == (0 if where == "all-in-hbm" else 1)
    # compare with the reference's recorded tensors after the step: bf16 results within one step,
    # fp32 moments within 1e-6 of the update's scale
    for got_t, key in ((p, "out_p"), (st["ema"], "out_m"), (st["ema_squared"], "out_v")):
        got, want = to_numpy(got_t), d[key]
        if got.dtype == np.uint16:
            diff = np.abs(got.astype(np.int64) - want.astype(np.int64))
            assert diff.max() <= 1 and (diff != 0).mean() < 0.6   # different draws: p, m, v each either floor or ceil
        else:
            old = d["in_" + key[-1]].astype(np.float64)
            den = np.maximum(np.abs(old), np.abs(want.astype(np.float64) - old))
            assert (np.abs(got.astype(np.float64) - want) <= 2e-6 * den + 1e-30).all()


def test_device_gradient_handoff_for_cpu_parameters():
    """A CPU-resident parameter whose gradient stays in HBM (``p.rt_device_grad``) is streamed with
    6 B/element in instead of 8 and gives the same result as a host gradient."""
    from ramtorch_b200 import AdamW, _native as N
    shapes = [(70001,), (64, 33)]
    params = make_params(shapes, torch.bfloat16, "cpu", pin=True)
    opt = AdamW(params, dtype=torch.bfloat16, **HP, seed=4, offload_chunk_elems=32768)
    mirror = Mirror(params, torch.bfloat16, 4, **HP)
    for s in range(2):
        grads = make_grads(shapes, torch.bfloat16, s)
        for p, g in zip(params, grads):
            p.rt_device_grad = g.cuda()
        before = N.stats()["h2d_bytes"]
        opt.step()
        moved = N.stats()["h2d_bytes"] - before
        assert moved == sum(6 * p.numel() for p in params)      # p, ema, ema_squared; no gradient bytes
        mirror.apply(grads)
        check(opt, params, mirror)


def test_checkpoint_round_trip_with_pinned_host_moments():
    """state_dict() keeps the reference's per-tensor layout although the pinned moments share two
    allocations; loading it (the base class moves state next to the parameters) and continuing gives
    the same bits as never having stopped."""
    import io
    from ramtorch_b200 import AdamW
    shapes = SHAPES[:5]
    params = make_params(shapes, torch.bfloat16, "cuda")
    opt = AdamW(params, **HP, seed=6)                      # bf16 moments, storage_device="cpu" (pinned)
    mirror = Mirror(params, torch.bfloat16, 6, **HP)
    for s in range(2):
        grads = make_grads(shapes, torch.bfloat16, s)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step(); mirror.apply(grads)
    buf = io.BytesIO()
    torch.save(opt.state_dict(), buf)
    buf.seek(0)
    loaded = torch.load(buf, weights_only=False)
    assert [tuple(loaded["state"][k]["ema"].shape) for k in range(len(shapes))] == [tuple(s) for s in shapes]
    opt2 = AdamW(params, **HP, seed=6)
    opt2.load_state_dict(loaded)
    for s in range(2, 4):
        grads = make_grads(shapes, torch.bfloat16, s)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt2.step(); mirror.apply(grads)
        check(opt2, params, mirror)


def test_empty_and_zero_dim_parameters():
    from ramtorch_b200 import AdamW
    shapes = [(0,), (), (3, 0, 5), (17,)]
    params = make_params(shapes, torch.bfloat16, "cuda", seed=3)
    opt = AdamW(params, dtype=torch.bfloat16, storage_device="cuda", **HP)
    mirror = Mirror(params, torch.bfloat16, 0, **HP)
    for s in range(2):
        grads = make_grads(shapes, torch.bfloat16, s)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step(); mirror.apply(grads)
        check(opt, params, mirror)


def test_step_hooks_and_lr_schedulers_keep_working():
    """step() bypasses torch's per-call profiler wrapper when nothing is registered; hooks, LR
    schedulers and the profiler range must behave as with any torch optimizer."""
    from ramtorch_b200 import AdamW
    p = make_params([(1000,)], torch.bfloat16, "cuda")[0]
    opt = AdamW([p], dtype=torch.bfloat16, storage_device="cuda", **HP)
    sched = torch.optim.lr_scheduler.StepLR(opt, step_size=1, gamma=0.5)
    mirror = Mirror([p], torch.bfloat16, 0, **HP)
    seen = []
    h1 = opt.register_step_pre_hook(lambda o, a, k: seen.append("pre"))
    h2 = opt.register_step_post_hook(lambda o, a, k: seen.append("post"))
    for s in range(3):
        g = make_grads([(1000,)], torch.bfloat16, s)
        p.grad = g[0].cuda()
        mirror.hp["lr"] = opt.param_groups[0]["lr"]
        opt.step(); sched.step()
        mirror.apply(g)
        check(opt, [p], mirror)
    assert seen == ["pre", "post"] * 3
    assert abs(opt.param_groups[0]["lr"] - HP["lr"] * 0.125) < 1e-12
    h1.remove(); h2.remove()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as prof:
        p.grad = make_grads([(1000,)], torch.bfloat16, 9)[0].cuda()
        opt.step()
    assert any("Optimizer.step#AdamW.step" in e.key for e in prof.key_averages())
    assert seen == ["pre", "post"] * 3


def test_more_hyper_rows_than_ride_along_with_a_launch():
    """Up to four (group, step) rows travel as kernel arguments; more go through the device table."""
    from ramtorch_b200 import AdamW
    shapes = [(300,), (4100,), (17,), (9000,), (64, 3), (2048,)]
    params = make_params(shapes, torch.bfloat16, "cuda", seed=8)
    lrs = [1e-4 * (k + 1) for k in range(len(shapes))]
    opt = AdamW([{"params": [p], "lr": lr} for p, lr in zip(params, lrs)], dtype=torch.bfloat16,
                storage_device="cuda", seed=2, **{k: v for k, v in HP.items() if k != "lr"})
    mirrors = [Mirror([p], torch.bfloat16, 2, ids=[k], **{**HP, "lr": lr}) for k, (p, lr) in enumerate(zip(params, lrs))]
    for s in range(3):
        grads = make_grads(shapes, torch.bfloat16, s)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step()
        for k, mir in enumerate(mirrors):
            mir.apply([grads[k]])
            check(opt, [params[k]], mir)


def test_large_all_bf16_tensor_takes_the_long_cta_path_bit_exactly():
    """2^29 + 8200 elements with bf16 moments: the plan gives this tensor CTAs of four 8192-element
    pieces; slices recomputed by the checker at their own index0 must match bit for bit."""
    from ramtorch_b200 import AdamW
    dev = torch.device("cuda")
    n = (1 << 29) + 8200
    gen = torch.Generator(device=dev).manual_seed(1)
    p = (torch.randn(n, device=dev, generator=gen) * 0.02).bfloat16()
    p.grad = (torch.randn(n, device=dev, generator=gen) * 1e-3).bfloat16()
    opt = AdamW([p], dtype=torch.bfloat16, storage_device=dev, seed=13, **HP)
    st = opt.state[p]
    st["ema"].copy_(torch.randn(n, device=dev, generator=gen) * 1e-3)
    st["ema_squared"].copy_((torch.randn(n, device=dev, generator=gen) * 1e-6).abs())
    st["step"] = 41
    p0, m0, v0 = p.clone(), st["ema"].clone(), st["ema_squared"].clone()
    opt.step()
    h = oracle.make_hyper(HP["lr"], HP["betas"], HP["eps"], HP["weight_decay"], 42, shared_draws=True)
    for lo in (0, 8 * 4097, 32768 * 1000 + 8192, n // 2 + 24, n - 65536):
        sl = slice(lo, min(n, lo + 65536))
        ps, gs, ms, vs = (to_numpy(t[sl]) for t in (p0, p.grad, m0, v0))
        oracle.adamw_sr(ps, gs, ms, vs, oracle.BF16, oracle.BF16, oracle.BF16, h, seed=13, tensor_id=0, index0=lo)
        assert bits_equal(ps, to_numpy(p[sl])) == 0
        assert bits_equal(ms, to_numpy(st["ema"][sl])) == 0
        assert bits_equal(vs, to_numpy(st["ema_squared"][sl])) == 0


def test_streamed_call_rejects_a_short_staging_buffer_before_copying_anything():
    """Host-side fault injection: a staging ring that is too small for the requested chunk is an
    argument error (nothing copied, nothing launched, tensors untouched)."""
    import ctypes
    from ramtorch_b200 import _native as N
    lib = N.lib()
    n = 100000
    p = torch.zeros(n, dtype=torch.bfloat16).pin_memory()
    g = torch.ones(n, dtype=torch.bfloat16).pin_memory()
    m = torch.zeros(n, dtype=torch.bfloat16).pin_memory()
    v = torch.zeros(n, dtype=torch.bfloat16).pin_memory()
    need = lib.rt_offload_staging_bytes(32768, 3, 0, 0, 0, 1, 1, 1, 1)
    staging = torch.empty(need // 2, dtype=torch.uint8, device="cuda")
    cfg = N.OffloadCfg(32768, 3, 0, staging.data_ptr(), staging.numel())
    h = N.make_hyper(1e-3, (0.9, 0.999), 1e-8, 0.0, 1)
    before = N.stats()
    rc = lib.rt_adamw_sr_offload(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n, 0, 0, 0,
                                 ctypes.byref(h), 0, 0, ctypes.byref(cfg), N.stream_ptr(torch.device("cuda", 0)))
    assert rc == -6 and b"staging buffer too small" in lib.rt_last_error()
    after = N.stats()
    assert after == before
    torch.cuda.synchronize()
    assert float(p.float().abs().sum()) == 0 and float(m.float().abs().sum()) == 0


def test_streamed_centralized_step_is_bit_identical_to_the_resident_one():
    """Same tensors, same seed: centralization through the chunked host pipeline (moments pinned on
    the host, chunks that cut rows in the middle) gives exactly the resident result."""
    from ramtorch_b200 import AdamW
    shapes = [(257, 130), (1000,), (64, 3, 5)]
    results = []
    for storage in ("cuda", "cpu"):
        params = make_params(shapes, torch.bfloat16, "cuda")
        opt = AdamW(params, centralization=0.5, dtype=torch.bfloat16, storage_device=storage, seed=12,
                    offload_chunk_elems=4096, **HP)
        for s in range(3):
            for p, g in zip(params, make_grads(shapes, torch.bfloat16, s)):
                p.grad = g.cuda()
            opt.step()
        results.append([to_numpy(p) for p in params] + [to_numpy(opt.state[p]["ema_squared"]) for p in params])
    for a, b in zip(*results):
        assert bits_equal(a, b) == 0


@pytest.mark.parametrize("helper", ["c++ list scan", "python passes"])
def test_load_state_dict_in_place_after_the_fast_path_is_armed(helper, monkeypatch):
    """Two steps arm the repeat-step cache; load_state_dict() then swaps every state dict and tensor.
    The following steps must use the loaded moments and counters, not the cached ones.  Run with
    the C++ helper that walks the parameter list and with the Python passes it replaces."""
    import copy
    from ramtorch_b200 import AdamW
    from ramtorch_b200.stochastic_optimizers import adamw as adamw_module
    if helper == "python passes":
        monkeypatch.setattr(adamw_module, "_FS", None)
    elif adamw_module._FS is None:
        pytest.skip("_fastscan.so has not been built")
    shapes = SHAPES[:6]
    params = make_params(shapes, torch.bfloat16, "cuda")
    opt = AdamW(params, dtype=torch.bfloat16, storage_device="cuda", seed=9, **HP)
    mirror = Mirror(params, torch.bfloat16, 9, **HP)

    def run(step_seed):
        grads = make_grads(shapes, torch.bfloat16, step_seed)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step()
        mirror.apply(grads)

    run(0)
    snapshot = copy.deepcopy(opt.state_dict())                       # state after step 1 ...
    kept = ([a.copy() for a in mirror.m], [a.copy() for a in mirror.v], list(mirror.step))
    run(1); run(2)
    assert opt.last_step_info.get("fast")                            # ... the cache is armed by now
    opt.load_state_dict(snapshot)                                     # back to the moments of step 1
    mirror.m, mirror.v, mirror.step = kept
    run(3)
    assert not opt.last_step_info.get("fast")
    check(opt, params, mirror)
    run(4)
    check(opt, params, mirror)
    # an in-place edit of a counter is noticed too
    run(5)
    assert opt.last_step_info.get("fast")
    opt.state[params[0]]["step"] = 40
    mirror.step[0] = 40
    run(6)
    check(opt, params, mirror)
    # ... and so are a gradient that disappears and a gradient of another dtype
    run(7); run(8)
    assert opt.last_step_info.get("fast")
    grads = make_grads(shapes, torch.bfloat16, 9)
    for k, (p, g) in enumerate(zip(params, grads)):
        p.grad = None if k == 2 else g.cuda()
    opt.step()
    mirror.apply(grads, skip=(2,))
    assert not opt.last_step_info.get("fast")
    check(opt, params, mirror)


def test_a_rejected_step_leaves_every_counter_where_it_was():
    from ramtorch_b200 import AdamW
    params = make_params([(64,), (4, 32)], torch.bfloat16, "cuda")
    params[1] = params[1].t()                                  # a non-contiguous parameter is refused
    opt = AdamW(params, dtype=torch.bfloat16, storage_device="cuda", **HP)
    for p in params:
        p.grad = torch.zeros(p.shape, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="contiguous"):
        opt.step()
    assert [opt.state[p]["step"] for p in params] == [0, 0]


def _shared_storage_owner(weight, grad, seed):
    """Child process = the owning rank: steps the shared CPU weight through the streamed path."""
    from ramtorch_b200 import AdamW
    torch.cuda.set_device(0)
    assert weight.is_shared() and not weight.is_pinned()
    weight.is_ramtorch = True
    weight.grad = grad
    opt = AdamW([weight], dtype=torch.bfloat16, seed=seed, offload_chunk_elems=8192, **HP)
    opt.step()
    assert weight.is_pinned()                      # re-pinned in place by the optimizer (rt_host_register)
    assert opt.last_step_info["streamed"] == 1
    opt.release_host_memory()


def test_shared_cpu_parameter_storage_is_repinned_and_updated_in_place_for_the_other_ranks():
    """Parameter consumption after the step (linear.py:168-188 reads ``weight_cpu`` again; the
    workers share its storage through ``mp.spawn`` pickling, README.md:177-182): the owner's step
    writes the new values into the shared pages, so a process that never ran the optimizer sees
    them without any redistribution (zero1.py:81 skips such parameters).  In the worker the storage
    arrives unpinned; the optimizer page-locks it where it lies."""
    import torch.multiprocessing as mp
    n, seed = 50001, 17
    weight = make_params([(n,)], torch.bfloat16, "cpu")[0].share_memory_()
    grad = make_grads([(n,)], torch.bfloat16, 0)[0].share_memory_()
    before = to_numpy(weight).copy()
    ctx = mp.get_context("spawn")
    child = ctx.Process(target=_shared_storage_owner, args=(weight, grad, seed))
    child.start()
    child.join(timeout=300)
    assert child.exitcode == 0
    want, m, v = before.copy(), np.zeros(n, np.uint16), np.zeros(n, np.uint16)
    oracle.adamw_sr(want, to_numpy(grad), m, v, oracle.BF16, oracle.BF16, oracle.BF16,
                    oracle.make_hyper(HP["lr"], HP["betas"], HP["eps"], HP["weight_decay"], 1, shared_draws=True),
                    seed=seed, tensor_id=0)
    got = to_numpy(weight)                          # read by this process, which ran no optimizer
    assert bits_equal(got, want) == 0 and bits_equal(got, before) > 0


def test_gradient_producer_keeps_micro_batch_gradients_in_hbm():
    """Stand-in for the patched ``Linear`` backward (linear.py:401-430): instead of copying each
    weight gradient to the host it calls ``accumulate_device_grad``.  Over two micro-batches the
    gradient accumulates in HBM, ``step`` consumes it without moving gradient bytes over the link,
    ``zero_grad`` clears it, and the result equals a host-side accumulation."""
    from ramtorch_b200 import AdamW, _native as N
    from ramtorch_b200.helpers import accumulate_device_grad
    shapes = [(4099,), (64, 33)]
    params = make_params(shapes, torch.bfloat16, "cpu", pin=True)
    opt = AdamW(params, dtype=torch.bfloat16, **HP, seed=4, offload_chunk_elems=32768)
    mirror = Mirror(params, torch.bfloat16, 4, **HP)
    for s in range(2):
        micro = [make_grads(shapes, torch.bfloat16, 10 * s + k) for k in range(2)]
        for batch in micro:                                   # "backward" of each micro-batch
            for p, g in zip(params, batch):
                accumulate_device_grad(p, g.cuda())
        total = [a + b for a, b in zip(*micro)]               # bf16 accumulation, as Tensor.grad would
        for p, t in zip(params, total):
            assert p.grad is None and torch.equal(p.rt_device_grad.cpu(), t)
        before = N.stats()["h2d_bytes"]
        opt.step()
        assert N.stats()["h2d_bytes"] - before == sum(6 * p.numel() for p in params)
        mirror.apply(total)
        check(opt, params, mirror)
        opt.zero_grad()
        assert all(p.rt_device_grad is None for p in params)
    for p, g in zip(params, make_grads(shapes, torch.bfloat16, 99)):
        accumulate_device_grad(p, g.cuda())
    opt.zero_grad(set_to_none=False)
    assert all(float(p.rt_device_grad.abs().sum()) == 0 for p in params)
