"""GPU: the CUDA kernels, called through the C ABI, against the CPU checker and the fixtures
produced by the reference.  Integer/bit results must be identical; fp32 pre-rounding values are
held to 1e-6 relative (cancellation-safe denominator) and in practice match bit for bit because
every operation of the contract is a correctly rounded IEEE operation on both sides."""
import numpy as np
import pytest
import torch

import oracle
from util import CODE, TORCH_DT, bits_equal, load_golden, step_cases, synth, to_numpy, to_torch

pytestmark = pytest.mark.gpu
F = None


def setup_module(module):
    global F
    from ramtorch_b200 import functional
    F = functional


def _hyper_pair(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, wd=0.01, step=11, shared=False, ref=False):
    from ramtorch_b200 import _native as N
    return (N.make_hyper(lr, betas, eps, wd, step, shared_draws=shared, reference_order=ref),
            oracle.make_hyper(lr, betas, eps, wd, step, shared_draws=shared, reference_order=ref))


ORDERS = pytest.mark.parametrize("ref", [False, True], ids=["default-order", "reference-order"])


def run_both(n, kp, kg, ks, *, seed=3, tensor_id=5, index0=0, step=11, wd=0.01, misalign=0,
             inject=False, taps=False, data_seed=0, shared=False, ref=False):
    """Run the CUDA kernel and the checker on the same seeded inputs; return both results."""
    p, g, m, v = synth(n, kp, kg, ks, data_seed)
    hn, ho = _hyper_pair(step=step, wd=wd, shared=shared, ref=ref)
    dev = torch.device("cuda")

    def dev_tensor(arr, kind):
        # optional misalignment: place the data `misalign` elements into a larger buffer
        t = to_torch(arr, kind)
        big = torch.zeros(n + misalign + 8, dtype=t.dtype, device=dev)
        view = big[misalign:misalign + n]
        view.copy_(t)
        return big, view

    bp, tp = dev_tensor(p, kp); bg, tg = dev_tensor(g, kg)
    bm, tm = dev_tensor(m, ks); bv, tv = dev_tensor(v, ks)
    rand_np = (None, None, None)
    rand_t = (None, None, None)
    if inject:
        rng = np.random.default_rng(99)
        rand_np = tuple(rng.integers(0, 65536, n, dtype=np.uint16) for _ in range(3))
        rand_t = tuple(torch.from_numpy(r.view(np.int16).copy()).to(dev) for r in rand_np)
    taps_t = tuple(torch.empty(n, dtype=torch.float32, device=dev) for _ in range(3)) if taps else (None,) * 3
    F.adamw_sr_flat_(tp, tg, tm, tv, hn, seed=seed, tensor_id=tensor_id, index0=index0,
                     rand=rand_t, taps=taps_t)
    torch.cuda.synchronize()
    f32 = oracle.adamw_sr(p, g, m, v, CODE[kp], CODE[kg], CODE[ks], ho, seed=seed, tensor_id=tensor_id,
                          index0=index0, rand=rand_np, want_f32=True)
    got = tuple(to_numpy(t) for t in (tp, tm, tv))
    # guard elements around the views must be untouched
    for big in (bp, bm, bv):
        assert float(big[:misalign].float().abs().sum()) == 0
        assert float(big[misalign + n:].float().abs().sum()) == 0
    return got, (p, m, v), f32, tuple(None if t is None else t.cpu().numpy() for t in taps_t)


SIZES = [1, 7, 8, 9, 255, 2048, 4095, 4096, 4099, 8192, 8193, 100003, (1 << 20) + 13]


@ORDERS
@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("kinds", [("bf16", "bf16", "bf16"), ("bf16", "bf16", "f32")])
def test_production_kernel_is_bit_exact_with_checker(n, kinds, ref):
    got, want, _, _ = run_both(n, *kinds, ref=ref)
    for a, b in zip(got, want):
        assert bits_equal(a, b) == 0


@ORDERS
@pytest.mark.parametrize("kp", ["bf16", "f32", "f16"])
@pytest.mark.parametrize("kg", ["bf16", "f32", "f16"])
@pytest.mark.parametrize("ks", ["bf16", "f32", "f16"])
def test_every_dtype_combination(kp, kg, ks, ref):
    got, want, _, _ = run_both(20011, kp, kg, ks, wd=0.0 if kp == "f16" else 0.01, ref=ref)
    for a, b in zip(got, want):
        assert bits_equal(a, b) == 0


def test_packed_square_root_and_reciprocal_are_correctly_rounded_on_every_input():
    """The kernels build sqrt(v') and 1/den for two elements at a time from the hardware
    approximations and packed fused multiply-adds.  The library's self-test compares them with the
    IEEE built-ins on all 2^32 bit patterns: no mismatch inside the ranges the fast path accepts."""
    from ramtorch_b200 import _native as N
    dev = torch.device("cuda")
    counts = torch.zeros(4, dtype=torch.int64, device=dev)
    N.check(N.lib().rt_selftest_exact_math(counts.data_ptr(), N.stream_ptr(dev)), "rt_selftest_exact_math")
    torch.cuda.synchronize()
    sqrt_in_range, rcp_in_range, sqrt_any, rcp_any = counts.tolist()
    assert sqrt_in_range == 0 and rcp_in_range == 0
    # the counters are live: outside the fast range (zeros, denormals, infinities, negatives) the
    # pair routines do differ from the built-ins, which is why those inputs take the built-ins
    assert sqrt_any > 0 and rcp_any > 0


@pytest.mark.parametrize("misalign", [1, 3, 4])
@pytest.mark.parametrize("kinds", [("bf16", "bf16", "bf16"), ("bf16", "f32", "f32")])
def test_misaligned_views_take_the_scalar_path_with_identical_results(misalign, kinds):
    got, want, _, _ = run_both(10007, *kinds, misalign=misalign)
    for a, b in zip(got, want):
        assert bits_equal(a, b) == 0


def test_index0_offsets_select_the_same_draws_as_the_whole_tensor():
    # a tensor updated in two slices (as the streaming path and ZeRO shards do) equals the
    # tensor updated at once
    n, cut = 50000, 16384
    whole, _, _, _ = run_both(n, "bf16", "bf16", "bf16")
    p, g, m, v = synth(n, "bf16", "bf16", "bf16", 0)
    hn, _ = _hyper_pair()
    dev = torch.device("cuda")
    ts = [to_torch(a, "bf16", dev) for a in (p, g, m, v)]
    for lo, hi in ((0, cut), (cut, n)):
        F.adamw_sr_flat_(*(t[lo:hi] for t in ts), hn, seed=3, tensor_id=5, index0=lo)
    torch.cuda.synchronize()
    for a, t in zip(whole, (ts[0], ts[2], ts[3])):
        assert bits_equal(a, to_numpy(t)) == 0


@ORDERS
@pytest.mark.parametrize("kinds", [("bf16", "bf16", "bf16"), ("bf16", "bf16", "f32"), ("f32", "f32", "f32")])
def test_debug_kernel_taps_and_injected_draws(kinds, ref):
    n = 30001
    got, want, f32_want, taps = run_both(n, *kinds, inject=True, taps=True, ref=ref)
    # fp32 pre-rounding update: the required tolerance is 1e-6 relative; in fact the bits are identical
    for a, b in zip(taps, f32_want):
        assert bits_equal(a, b) == 0
    # identical random bits -> bit-exact results
    for a, b in zip(got, want):
        assert bits_equal(a, b) == 0
    # and the bf16 outputs are the integer map applied to the kernel's own fp32 values
    p, g, m, v = synth(n, *kinds, 0)
    if kinds[0] == "bf16":
        rng = np.random.default_rng(99)
        rp = rng.integers(0, 65536, n, dtype=np.uint16)
        assert (oracle.sr_round_np(taps[0], rp) == got[0]).all()


def test_debug_and_production_kernels_agree():
    a, _, _, _ = run_both(12345, "bf16", "bf16", "bf16", taps=True)
    b, _, _, _ = run_both(12345, "bf16", "bf16", "bf16")
    for x, y in zip(a, b):
        assert bits_equal(x, y) == 0


@ORDERS
@pytest.mark.parametrize("name", step_cases())
def test_golden_steps_on_gpu(name, ref):
    """The reference's own recorded steps: same inputs, the reference's draws injected."""
    d = load_golden(name)
    meta = d["meta"]
    if meta.get("centralization", 0):
        pytest.skip("centralization is exercised through the optimizer class")
    from ramtorch_b200 import _native as N
    kp, kg, ks = meta["p_dtype"], meta["g_dtype"], meta["state_dtype"]
    dev = torch.device("cuda")
    tp, tg, tm, tv = (to_torch(d["in_" + k], kind, dev) for k, kind in zip("pgmv", (kp, kg, ks, ks)))
    h = N.make_hyper(meta["lr"], tuple(meta["betas"]), meta["eps"], meta["weight_decay"], meta["step"],
                     reference_order=ref)
    rand = tuple(None if ("r16_" + k) not in d else torch.from_numpy(d["r16_" + k].view(np.int16).copy()).to(dev)
                 for k in "pmv")
    taps = tuple(torch.empty(tp.numel(), dtype=torch.float32, device=dev) for _ in range(3))
    F.adamw_sr_flat_(tp, tg, tm, tv, h, rand=rand, taps=taps)
    torch.cuda.synchronize()
    # against the checker: identical
    p, g, m, v = (d["in_" + k].copy() for k in "pgmv")
    ho = oracle.make_hyper(meta["lr"], tuple(meta["betas"]), meta["eps"], meta["weight_decay"], meta["step"],
                           reference_order=ref)
    f32 = oracle.adamw_sr(p, g, m, v, CODE[kp], CODE[kg], CODE[ks], ho,
                          rand=tuple(d.get("r16_" + k) for k in "pmv"), want_f32=True)
    for t, want in zip((tp, tm, tv), (p, m, v)):
        assert bits_equal(to_numpy(t), want) == 0
    for t, want in zip(taps, f32):
        assert bits_equal(t.cpu().numpy(), want) == 0
    # against the reference's recorded fp32 values: 1e-6 relative, safe denominator
    if "f32_p" in d:
        old = oracle.bf16_bits_to_f32(d["in_p"]).astype(np.float64)
        ref = d["f32_p"].astype(np.float64)
        den = np.maximum(np.abs(old), np.abs(ref - old))
        rel = np.abs(taps[0].cpu().numpy().astype(np.float64) - ref) / np.where(den > 0, den, 1)
        assert rel.max() <= 1e-6
    if "f32_m" in d:
        assert bits_equal(taps[1].cpu().numpy(), d["f32_m"]) == 0
        assert bits_equal(taps[2].cpu().numpy(), d["f32_v"]) == 0
    # against the reference's final tensors: at most one bf16 step apart, almost all identical
    for t, key in zip((tp, tm, tv), ("out_p", "out_m", "out_v")):
        got, want = to_numpy(t), d[key]
        if got.dtype == np.uint16:
            diff = np.abs(got.astype(np.int64) - want.astype(np.int64))
            assert diff.max() <= 1 and (diff != 0).mean() <= 2e-3


@pytest.mark.parametrize("name", ["sr_edge.npz", "sr_random.npz"])
def test_sr_round_golden_on_gpu(name):
    d = load_golden(name)
    dev = torch.device("cuda")
    src = torch.from_numpy(d["source_bits"].astype(np.uint32).view(np.float32).copy()).to(dev)
    r = torch.from_numpy(d["r16"].view(np.int16).copy()).to(dev)
    out = torch.empty(src.numel(), dtype=torch.bfloat16, device=dev)
    F.sr_round_bf16_(out, src, rand16=r)
    got, want = to_numpy(out), d["target_bits"]
    want_nan = (want & 0x7FFF) > 0x7F80
    assert (((got & 0x7FFF) > 0x7F80) == want_nan).all()
    assert (got[~want_nan] == want[~want_nan]).all()
    assert (got == oracle.sr_round_bf16(src.cpu().numpy(), d["r16"])).all()


@pytest.mark.parametrize("n", [1, 8, 1000, 65536 + 3])
def test_sr_round_philox_stream_matches_checker(n):
    dev = torch.device("cuda")
    x = torch.randn(n, generator=torch.Generator().manual_seed(n)).to(dev)
    out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    F.sr_round_bf16_(out, x, seed=2**40 + 17, tensor_id=9, step=33, stream_id=2)
    r = oracle.draws(2**40 + 17, 9, 33, 2, 0, n)
    assert (to_numpy(out) == oracle.sr_round_bf16(x.cpu().numpy(), r)).all()


def test_stochastic_rounding_is_unbiased_over_a_million_trials():
    """out in {floor, ceil} of the fp32 value and the mean over 10^6 roundings within 3 sigma."""
    dev = torch.device("cuda")
    n = 1_000_000
    for value in (1.00212, -0.0123456, 3.14159e-5):
        x = torch.full((n,), value, dtype=torch.float32, device=dev)
        out = torch.empty(n, dtype=torch.bfloat16, device=dev)
        F.sr_round_bf16_(out, x, seed=1234, tensor_id=1, step=5)
        o = out.float().cpu().numpy().astype(np.float64)
        x32 = np.float32(value)
        bits = np.array([x32]).view(np.uint32)[0]
        lo = np.array([bits & 0xFFFF0000], np.uint32).view(np.float32)[0]
        hi = np.array([(bits & 0xFFFF0000) + 0x10000], np.uint32).view(np.float32)[0]
        assert set(np.unique(o)) <= {float(lo), float(hi)}
        f = (bits & 0xFFFF) / 65536.0
        ulp = abs(float(hi) - float(lo))
        sigma = ulp * np.sqrt(f * (1 - f) / n)
        assert abs(o.mean() - float(x32)) <= 3 * sigma + 1e-30


def test_shared_draws_stay_unbiased_and_couple_only_the_documented_lanes():
    """RT_HYPER_SHARED_DRAWS (the optimizer class's default): one Philox block serves p, ema and
    ema_squared of a group of eight, ema reading two lanes further and ema_squared four.  Over 2^20
    elements with identical inputs: each of the three roundings is unbiased within 3 sigma; the
    three roundings OF ONE ELEMENT are uncorrelated; and the pairs that do share a draw -- p[i] with
    ema[i-2] and ema_squared[i-4] inside a group -- are coupled exactly as much as two thresholds on
    one uniform number are: corr = (min(fa, fb) - fa fb) / sqrt(fa (1 - fa) fb (1 - fb))."""
    from ramtorch_b200 import _native as N
    n, step = 1 << 20, 100
    dev = torch.device("cuda")
    const = dict(p=0.0123, g=7.3e-4, m=-4.1e-4, v=3.3e-7)
    bits16 = {k: oracle.f32_to_bf16_bits_rn(np.full(n, x, np.float32)) for k, x in const.items()}
    hn = N.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, step, shared_draws=True)
    ho = oracle.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, step, shared_draws=True)
    tp, tg, tm, tv = (to_torch(bits16[k], "bf16", dev) for k in "pgmv")
    F.adamw_sr_flat_(tp, tg, tm, tv, hn, seed=2024, tensor_id=3)
    torch.cuda.synchronize()
    small = {k: bits16[k][:8].copy() for k in "pgmv"}
    f32 = oracle.adamw_sr(small["p"], small["g"], small["m"], small["v"], oracle.BF16, oracle.BF16, oracle.BF16, ho,
                          seed=2024, tensor_id=3, want_f32=True)
    floor16, frac = {}, {}
    for name, x in zip("pmv", f32):
        b = int(np.array([x[0]], np.float32).view(np.uint32)[0])
        floor16[name], frac[name] = b >> 16, (b & 0xFFFF) / 65536.0
        assert 0.05 < frac[name] < 0.95                       # a fraction worth testing

    def round_ups(tensors):
        """1.0 where an element was rounded up; also checks floor/ceil and the mean (3 sigma)."""
        up = {}
        for name, t in zip("pmv", tensors):
            out = to_numpy(t).astype(np.int64)
            assert set(np.unique(out)) <= {floor16[name], floor16[name] + 1}   # floor or ceil of the fp32 value
            up[name] = (out != floor16[name]).astype(np.float64)
            sigma = np.sqrt(frac[name] * (1 - frac[name]) / n)
            assert abs(up[name].mean() - frac[name]) <= 3 * sigma, name
        return up

    def corr(a, b):
        return float(np.corrcoef(a, b)[0, 1])

    def shifted(x, lanes):        # x[i] <- x[(i - lanes) within its group of eight]
        return x.reshape(-1, 8)[:, (np.arange(8) - lanes) % 8].ravel()

    noise = 4.0 / np.sqrt(n)
    up = round_ups((tp, tm, tv))
    # same element, different tensors: different draws
    assert abs(corr(up["p"], up["m"])) <= noise and abs(corr(up["p"], up["v"])) <= noise and abs(corr(up["m"], up["v"])) <= noise
    # the coupled pairs
    for other, lanes in (("m", 2), ("v", 4)):
        fa, fb = frac["p"], frac[other]
        want = (min(fa, fb) - fa * fb) / np.sqrt(fa * (1 - fa) * fb * (1 - fb))
        assert abs(corr(up["p"], shifted(up[other], lanes)) - want) <= noise, other
    # with independent blocks (flags = 0) the same pairs are uncorrelated
    hn.flags = 0
    tp, tg, tm, tv = (to_torch(bits16[k], "bf16", dev) for k in "pgmv")
    F.adamw_sr_flat_(tp, tg, tm, tv, hn, seed=2024, tensor_id=3)
    torch.cuda.synchronize()
    ind = round_ups((tp, tm, tv))
    assert abs(corr(ind["p"], shifted(ind["m"], 2))) <= noise and abs(corr(ind["p"], shifted(ind["v"], 4))) <= noise


def test_large_flat_tensor_spot_checked_against_checker():
    """2^27 elements (fp32 moments, the roofline configuration's dtypes): whole-buffer
    properties plus slices recomputed by the checker at their own index0."""
    n = 1 << 27
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    p = (torch.randn(n, device=dev, generator=g) * 0.02).bfloat16()
    gr = (torch.randn(n, device=dev, generator=g) * 1e-3).bfloat16()
    m = torch.randn(n, device=dev, generator=g) * 1e-3
    v = (torch.randn(n, device=dev, generator=g) * 1e-6).abs()
    p0, m0, v0 = p.clone(), m.clone(), v.clone()
    hn, ho = _hyper_pair(step=100)
    F.adamw_sr_flat_(p, gr, m, v, hn, seed=7, tensor_id=0)
    torch.cuda.synchronize()
    # whole-buffer check against a plain PyTorch fp32 evaluation of the same update: moments within
    # fp32 rounding, parameters within one bf16 step of the unrounded value
    assert torch.isfinite(p.float()).all() and torch.isfinite(m).all() and torch.isfinite(v).all()
    g32 = gr.float()
    m_ref = m0 * 0.9 + g32 * (1 - 0.9)
    v_ref = v0 * 0.999 + g32 * g32 * (1 - 0.999)
    assert float(((m - m_ref).abs() / (m0.abs() + g32.abs() + 1e-30)).max()) <= 1e-6
    assert float(((v - v_ref).abs() / (v0.abs() + g32 * g32 + 1e-30)).max()) <= 1e-6
    ss = 1e-4 / (1 - 0.9 ** 100)
    den = v.sqrt() / ((1 - 0.999 ** 100) ** 0.5) + 1e-8
    p_ref = p0.float() * (1 - ss * 0.01) - ss * m / den
    ulp = torch.maximum(p_ref.abs(), p.float().abs()) * 2.0 ** -7
    assert bool(((p.float() - p_ref).abs() <= ulp + 1e-30).all())
    del g32, m_ref, v_ref, den, p_ref, ulp
    for lo in (0, 8 * 12345, n // 2 + 64, n - 65536):
        hi = lo + 65536
        ps, gs, ms, vs = (to_numpy(t[lo:hi]) for t in (p0, gr, m0, v0))
        oracle.adamw_sr(ps, gs, ms, vs, oracle.BF16, oracle.BF16, oracle.F32, ho, seed=7, tensor_id=0, index0=lo)
        assert bits_equal(ps, to_numpy(p[lo:hi])) == 0
        assert bits_equal(ms, to_numpy(m[lo:hi])) == 0
        assert bits_equal(vs, to_numpy(v[lo:hi])) == 0


@pytest.mark.parametrize("kinds", [("bf16", "bf16", "bf16"), ("bf16", "bf16", "f32"), ("f32", "f32", "f32")])
@pytest.mark.parametrize("step", [1, 11, 100])
def test_default_order_stays_within_the_fp32_tolerance_of_the_reference_order(kinds, step):
    """The default operation order (multiply-add by 1/bc, reciprocal of den) against the reference's
    order (two divisions): moments bit-identical, p' within 1e-6 relative (cancellation-safe
    denominator), bf16 parameters in {floor, ceil} of the kernel's own fp32."""
    from ramtorch_b200 import _native as N
    n = 200003
    kp, kg, ks = kinds
    p, g, m, v = synth(n, kp, kg, ks, 4, warm=step > 1)
    dev = torch.device("cuda")
    hn = N.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, step)
    ho_ref = oracle.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, step, reference_order=True)
    tp, tg, tm, tv = (to_torch(a, k, dev) for a, k in zip((p, g, m, v), (kp, kg, ks, ks)))
    taps = tuple(torch.empty(n, dtype=torch.float32, device=dev) for _ in range(3))
    rng = np.random.default_rng(5)
    rand_np = tuple(rng.integers(0, 65536, n, dtype=np.uint16) for _ in range(3))
    rand_t = tuple(torch.from_numpy(r.view(np.int16).copy()).to(dev) for r in rand_np)
    F.adamw_sr_flat_(tp, tg, tm, tv, hn, rand=rand_t, taps=taps)
    torch.cuda.synchronize()
    p_old = (oracle.bf16_bits_to_f32(p) if kp == "bf16" else p).astype(np.float64)
    po, mo, vo = p.copy(), m.copy(), v.copy()
    fp, fm, fv = oracle.adamw_sr(po, g, mo, vo, CODE[kp], CODE[kg], CODE[ks], ho_ref, rand=rand_np, want_f32=True)
    assert bits_equal(taps[1].cpu().numpy(), fm) == 0
    assert bits_equal(taps[2].cpu().numpy(), fv) == 0
    got = taps[0].cpu().numpy().astype(np.float64)
    den = np.maximum(np.abs(p_old), np.abs(fp.astype(np.float64) - p_old))
    rel = np.abs(got - fp) / np.where(den > 0, den, 1)
    assert rel.max() <= 1e-6, rel.max()
    if kp == "bf16":
        assert (oracle.sr_round_np(taps[0].cpu().numpy(), rand_np[0]) == to_numpy(tp)).all()
        # same draws, fp32 values a few ulps apart: at most one bf16 step, almost always none
        d = np.abs(to_numpy(tp).astype(np.int64) - po.astype(np.int64))
        assert d.max() <= 1 and (d != 0).mean() < 1e-3


@pytest.mark.parametrize("shape", [(37, 111), (1, 1000), (5000, 8), (100003,), (64, 4096)])
@pytest.mark.parametrize("kind", ["bf16", "f32"])
def test_row_means_kernel(shape, kind):
    g = torch.randn(shape, generator=torch.Generator().manual_seed(7)) * 1e-3 + 2e-4
    g = g.to(TORCH_DT[kind]).cuda()
    rows = shape[0] if len(shape) >= 2 else 1
    got = F.row_means(g.reshape(-1), rows, g.numel() // rows).cpu().numpy().astype(np.float64)
    want = g.double().reshape(rows, -1).mean(dim=1).cpu().numpy()
    scale = g.double().abs().reshape(rows, -1).mean(dim=1).cpu().numpy()
    assert (np.abs(got - want) <= 2e-6 * scale + 1e-12).all()


@pytest.mark.parametrize("shape", [(37, 111), (64, 4096), (100003,)])
def test_centralized_step_is_bit_exact_given_the_same_row_means(shape):
    from ramtorch_b200 import _native as N
    n = int(np.prod(shape))
    p, g, m, v = synth(n, "bf16", "bf16", "bf16", 12)
    dev = torch.device("cuda")
    tp, tg, tm, tv = (to_torch(a, "bf16", dev) for a in (p, g, m, v))
    rows = shape[0] if len(shape) >= 2 else 1
    row_len = n // rows
    means = F.row_means(tg, rows, row_len)
    hn = N.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, 5, centralization=0.5)
    ho = oracle.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, 5, centralization=0.5)
    F.adamw_sr_flat_(tp, tg, tm, tv, hn, seed=2, tensor_id=9, row_mean=means, row_len=row_len if rows > 1 else 0)
    torch.cuda.synchronize()
    oracle.adamw_sr(p, g, m, v, oracle.BF16, oracle.BF16, oracle.BF16, ho, seed=2, tensor_id=9,
                    row_mean=means.cpu().numpy(), row_len=row_len if rows > 1 else 0)
    for t, want in zip((tp, tm, tv), (p, m, v)):
        assert bits_equal(to_numpy(t), want) == 0


@pytest.mark.parametrize("kinds", [("bf16", "bf16", "bf16"), ("f32", "bf16", "bf16"), ("f16", "f32", "bf16"),
                                   ("bf16", "bf16", "f32")])
@pytest.mark.parametrize("n,misalign", [(100003, 0), (8200, 3), (5, 0)])
def test_shared_draws_layout_is_bit_exact_with_checker(kinds, n, misalign):
    """RT_HYPER_SHARED_DRAWS: one Philox block per eight elements, rotated per stream; vector,
    scalar and tail paths must pick the same lanes as the checker."""
    got, want, _, _ = run_both(n, *kinds, shared=True, misalign=misalign)
    for a, b in zip(got, want):
        assert bits_equal(a, b) == 0
    # the debug kernel follows the same layout
    got2, _, _, _ = run_both(n, *kinds, shared=True, misalign=misalign, taps=True)
    for a, b in zip(got2, want):
        assert bits_equal(a, b) == 0
    if kinds[2] == "bf16":
        # and it differs from the independent layout in the moments, not in the parameter
        indep, _, _, _ = run_both(n, *kinds, shared=False, misalign=misalign)
        assert bits_equal(got[0], indep[0]) == 0
        if n > 1000:
            assert bits_equal(got[1], indep[1]) > 0


def test_special_values_follow_ieee_like_the_checker():
    """Zeros, denormals, infinities and NaNs in every input: wherever the fp32 update is a number the
    CUDA result is bit-identical to the checker's; where it is a NaN both sides produce a NaN."""
    from ramtorch_b200 import _native as N
    specials = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x007F, 0x0080, 0x3F80, 0xBF80, 0x7F7F, 0xFF7F,
                         0x7F80, 0xFF80, 0x7FC0, 0x3A83, 0x0400, 0x7E00], dtype=np.uint16)
    grid = np.array(np.meshgrid(specials, specials, specials, specials, indexing="ij")).reshape(4, -1)
    p, g, m, v = (np.ascontiguousarray(a) for a in grid)
    v = v & 0x7FFF                                           # second moments are never negative
    n = p.size
    dev = torch.device("cuda")
    tp, tg, tm, tv = (to_torch(a, "bf16", dev) for a in (p, g, m, v))
    taps = tuple(torch.empty(n, dtype=torch.float32, device=dev) for _ in range(3))
    hn, ho = _hyper_pair(step=3)
    F.adamw_sr_flat_(tp, tg, tm, tv, hn, seed=1, tensor_id=1, taps=taps)
    tp2, tg2, tm2, tv2 = (to_torch(a, "bf16", dev) for a in (p, g, m, v))
    F.adamw_sr_flat_(tp2, tg2, tm2, tv2, hn, seed=1, tensor_id=1)      # production kernel
    torch.cuda.synchronize()
    po, mo, vo = p.copy(), m.copy(), v.copy()
    f32 = oracle.adamw_sr(po, g, mo, vo, oracle.BF16, oracle.BF16, oracle.BF16, ho, seed=1, tensor_id=1, want_f32=True)
    for tap, ref, out_dbg, out_prod, want in zip(taps, f32, (tp, tm, tv), (tp2, tm2, tv2), (po, mo, vo)):
        got32 = tap.cpu().numpy()
        nan = np.isnan(ref)
        assert (np.isnan(got32) == nan).all()
        assert bits_equal(got32[~nan], ref[~nan]) == 0
        assert bits_equal(to_numpy(out_dbg)[~nan], want[~nan]) == 0
        assert bits_equal(to_numpy(out_prod)[~nan], want[~nan]) == 0
    assert nan.any() and (~nan).sum() > n // 4


def _self_peered_step(n, offsets, dev, ranks=3, self_rank=0, pull_grads=True):
    """Drive the ZeRO peer paths of the kernel on ONE GPU through the C ABI: the "peers" are other
    buffers of the same device (a peer pointer is just an address).  This rank is `self_rank` of
    `ranks`; the other ranks' gradient copies are pulled and summed in rank order, and the updated
    parameters are pushed into ranks - 1 more parameter buffers.  (The number of ranks decides how
    many shared-memory slots the gradient staging ring gets: 4 up to five ranks, 2 at eight.)"""
    import ctypes
    from ramtorch_b200 import _native as N
    lib = N.lib()
    gen = torch.Generator(device=dev).manual_seed(3)
    total = offsets[-1][0] + offsets[-1][1]
    pflat = (torch.randn(total, device=dev, generator=gen) * 0.02).bfloat16()
    p0 = pflat.clone()
    gflats = [(torch.randn(total, device=dev, generator=gen) * 1e-3).bfloat16() for _ in range(ranks)]
    pcopies = [torch.zeros(total, dtype=torch.bfloat16, device=dev) for _ in range(ranks - 1)]
    m = (torch.randn(total, device=dev, generator=gen) * 1e-3).bfloat16()
    v = (torch.randn(total, device=dev, generator=gen) * 1e-6).abs().bfloat16()
    m0, v0 = m.clone(), v.clone()
    descs = (N.TensorDesc * len(offsets))()
    for k, (off, cnt) in enumerate(offsets):
        d = descs[k]
        d.p, d.g = pflat.data_ptr() + 2 * off, gflats[self_rank].data_ptr() + 2 * off
        d.m, d.v = m.data_ptr() + 2 * off, v.data_ptr() + 2 * off
        d.numel, d.tensor_id = cnt, 40 + k
        d.p_dtype = d.g_dtype = d.state_dtype = N.BF16
    plan = ctypes.c_void_p()
    N.check(lib.rt_plan_create(ctypes.byref(plan), descs, len(offsets), 0), "rt_plan_create")
    try:
        push = N.Push()
        push.local_base, push.bytes, push.n_peers = pflat.data_ptr(), 2 * total, ranks - 1
        for k, c in enumerate(pcopies):
            push.peer_base[k] = c.data_ptr()
        N.check(lib.rt_plan_set_push(plan, ctypes.byref(push)), "rt_plan_set_push")
        if pull_grads:
            pull = N.Pull()
            pull.local_base, pull.bytes, pull.n_ranks, pull.self_rank = gflats[self_rank].data_ptr(), 2 * total, ranks, self_rank
            for r in range(ranks):
                pull.base[r] = gflats[r].data_ptr()
            N.check(lib.rt_plan_set_pull(plan, ctypes.byref(pull)), "rt_plan_set_pull")
        else:
            gflats = [gflats[self_rank]]          # redistribution only: the gradient is this rank's own
        hyper = (N.Hyper * 1)(N.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, 7, shared_draws=True))
        N.check(lib.rt_adamw_sr_multi(plan, hyper, 1, 5, N.stream_ptr(dev)), "rt_adamw_sr_multi")
        torch.cuda.synchronize()
    finally:
        lib.rt_plan_destroy(plan)
    return pflat, p0, gflats, pcopies, m, m0, v, v0


def _check_self_peered(offsets, result, spots):
    pflat, p0, gflats, pcopies, m, m0, v, v0 = result
    ho = oracle.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, 7, shared_draws=True)
    for c in pcopies:
        for off, cnt in offsets:                          # every "peer" received the new parameters
            assert torch.equal(c[off:off + cnt], pflat[off:off + cnt])
    for k, (off, cnt) in enumerate(offsets):
        for lo in spots(cnt):
            hi = min(cnt, lo + 65536)
            sl = slice(off + lo, off + hi)
            g32 = gflats[0][sl].float()
            for r in range(1, len(gflats)):
                g32 = g32 + gflats[r][sl].float()              # rank order, fp32
            ps, ms, vs = to_numpy(p0[sl]), to_numpy(m0[sl]), to_numpy(v0[sl])
            oracle.adamw_sr(ps, g32.cpu().numpy(), ms, vs, oracle.BF16, oracle.F32, oracle.BF16, ho, seed=5,
                            tensor_id=40 + k, index0=lo)
            assert bits_equal(ps, to_numpy(pflat[sl])) == 0
            assert bits_equal(ms, to_numpy(m[sl])) == 0
            assert bits_equal(vs, to_numpy(v[sl])) == 0


@pytest.mark.parametrize("pull_grads", [True, False], ids=["push+pull", "push-only"])
@pytest.mark.parametrize("ranks,self_rank", [(3, 0), (2, 1), (6, 3), (8, 5), (16, 15)])
def test_peer_push_and_gradient_pull_paths_on_one_gpu(ranks, self_rank, pull_grads):
    dev = torch.device("cuda", 0)
    sizes = [64, 8192 * 3 + 5, 100000, 7, 20000, 2048 * 9 + 8]
    offsets, cur = [], 0
    for s in sizes:
        offsets.append((cur, s))
        cur += (s + 127) // 128 * 128
    _check_self_peered(offsets, _self_peered_step(cur, offsets, dev, ranks, self_rank, pull_grads), lambda cnt: [0])


def test_peer_paths_with_long_ctas_on_a_large_tensor():
    """2^29 + 8200 elements: enough elements for the launch to use its longer CTAs (16384 elements), with a ragged end."""
    dev = torch.device("cuda", 0)
    n = (1 << 29) + 8200
    offsets = [(0, n)]
    for pull_grads in (True, False):
        res = _self_peered_step(n, offsets, dev, pull_grads=pull_grads)
        _check_self_peered(offsets, res, lambda cnt: [0, 8 * 4097, 32768 * 1000 + 8192, cnt // 2 + 24, cnt - 65536])
        del res
