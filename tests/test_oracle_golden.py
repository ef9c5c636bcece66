"""CPU: the C checker against the fixtures produced by running the reference (tests/golden)."""
import json
import os

import numpy as np
import pytest

import oracle
from util import CODE, GOLDEN, bits_equal, load_golden, step_cases


def test_philox_known_answers():
    # Random123 kat_vectors, philox4x32 with 10 rounds
    kat = [([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
           ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
           ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
            [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1])]
    for ctr, key, want in kat:
        assert oracle.philox_c(ctr, key).tolist() == want
        assert oracle.philox_np(np.array([ctr]), key)[0].tolist() == want


def test_draw_layout_matches_numpy_restatement():
    for seed, tid, step, stream, i0, n in [(0, 0, 1, 0, 0, 64), (2**40 + 5, 3, 7, 2, 8, 1000),
                                           (2**64 - 1, 2**32 - 1, 2**32 - 1, 1, 16, 100)]:
        assert (oracle.draws(seed, tid, step, stream, i0, n) ==
                oracle.draws_np(seed, tid, step, stream, i0, n)).all()


@pytest.mark.parametrize("name", ["sr_edge.npz", "sr_random.npz"])
def test_sr_round_matches_reference(name):
    d = load_golden(name)
    src = d["source_bits"].astype(np.uint32).view(np.float32)
    want = d["target_bits"]
    # A rounded value that is a NaN keeps its payload here; the reference's final
    # Tensor.copy_ canonicalises NaN payloads in an ATen-build-dependent way (0xFFFF on this
    # CPU build).  Everything else, including overflow to inf and -0.0, must match bit for bit.
    want_nan = (want & 0x7FFF) > 0x7F80
    for got in (oracle.sr_round_bf16(src, d["r16"]), oracle.sr_round_np(src, d["r16"])):
        got_nan = (got & 0x7FFF) > 0x7F80
        assert (got_nan == want_nan).all()
        assert (got[~want_nan] == want[~want_nan]).all()


def _row_mean(d):
    meta = d["meta"]
    c = meta.get("centralization", 0)
    if not c:
        return None, 0
    g = d["in_g"]
    g32 = oracle.bf16_bits_to_f32(g) if meta["g_dtype"] == "bf16" else g.astype(np.float32)
    shape = meta["shape"]
    if len(shape) == 1:
        return np.array([g32.mean(dtype=np.float32)], np.float32), 0
    rows = g32.reshape(shape[0], -1)
    return rows.mean(axis=1, dtype=np.float32), rows.shape[1]


def safe_rel(got, want, old, scale_floor=0.0):
    """|got - want| relative to max(|old|, |want - old|): the cancellation-safe denominator."""
    den = np.maximum(np.abs(old.astype(np.float64)), np.abs(want.astype(np.float64) - old))
    den = np.maximum(den, scale_floor)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    return np.where(den > 0, err / np.where(den > 0, den, 1), err)


@pytest.mark.parametrize("ref", [False, True], ids=["default-order", "reference-order"])
@pytest.mark.parametrize("name", step_cases())
def test_step_matches_reference(name, ref):
    d = load_golden(name)
    meta = d["meta"]
    pd, gd, sd = CODE[meta["p_dtype"]], CODE[meta["g_dtype"]], CODE[meta["state_dtype"]]
    h = oracle.make_hyper(meta["lr"], tuple(meta["betas"]), meta["eps"], meta["weight_decay"],
                          meta["step"], meta.get("centralization", 0), reference_order=ref)
    p, g, m, v = (d["in_" + k].copy() for k in "pgmv")
    rand = tuple(d.get("r16_" + k) for k in "pmv")
    row_mean, row_len = _row_mean(d)
    fp, fm, fv = oracle.adamw_sr(p, g, m, v, pd, gd, sd, h, rand=rand, row_mean=row_mean,
                                 row_len=row_len, want_f32=True)
    centralized = row_mean is not None
    # fp32 pre-rounding values: the reference's, where it rounds stochastically (taps), else its outputs
    ref_m = d["f32_m"] if "f32_m" in d else d["out_m"].astype(np.float32)
    ref_v = d["f32_v"] if "f32_v" in d else d["out_v"].astype(np.float32)
    ref_p = d["f32_p"] if "f32_p" in d else d["out_p"].astype(np.float32)
    f16 = meta["state_dtype"] == "f16"
    if not centralized and not f16:
        # moments: bit-exact with the reference's vectorised CPU kernels
        assert bits_equal(fm, ref_m) == 0
        assert bits_equal(fv, ref_v) == 0
    if not f16 and meta["p_dtype"] != "f16":
        # p': within 1e-6 in either operation order.  In the reference's order the only difference
        # left is that the reference's ATen build evaluates sqrt with a 0.5035-ulp routine and the
        # checker with the correctly rounded one: a few elements land one fp32 ulp apart.
        old_p = (oracle.bf16_bits_to_f32(d["in_p"]) if meta["p_dtype"] == "bf16" else d["in_p"]).astype(np.float64)
        rel = safe_rel(fp, ref_p, old_p)
        assert rel.max() <= 1e-6, rel.max()
        if not centralized and ref:
            assert bits_equal(fp, ref_p) <= max(2, fp.size // 500)
    # final tensors with the reference's own draws injected
    tol_elems = 0 if not centralized else None
    for key, arr in (("out_p", p), ("out_m", m), ("out_v", v)):
        want = d[key]
        if arr.dtype == np.uint16:
            diff = np.abs(arr.astype(np.int64) - want.astype(np.int64))
            assert diff.max() <= 1  # never more than one bf16 step apart
            if tol_elems == 0:
                assert (diff != 0).mean() <= 2e-3
        elif arr.dtype == np.float16:
            assert np.abs(arr.astype(np.float32) - want.astype(np.float32)).max() <= 2 * np.spacing(np.abs(want).max().astype(np.float16)).astype(np.float32) + 1e-7
        else:
            old = d["in_" + key[-1]].astype(np.float64)
            assert safe_rel(arr, want, old).max() <= 1e-6


def test_hyper_fill_agrees_with_python_restatement():
    import ctypes
    for step in (1, 2, 11, 100, 100000):
        a = oracle.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, step)
        b = oracle.Hyper()
        oracle.lib().rto_hyper_fill(ctypes.byref(b), 1e-4, 0.9, 0.999, 1e-8, 0.01, 0.0, step)
        assert bytes(a) == bytes(b)


def test_zero1_golden_is_round_robin_per_group():
    with open(os.path.join(GOLDEN, "zero1_ownership.json")) as f:
        cases = json.load(f)
    for c in cases:
        w, k = c["world_size"], 0
        for gi, n in enumerate(c["group_sizes"]):
            for j in range(n):
                assert k in c["ownership"][str(j % w)][gi]
                k += 1


def test_shared_draws_layout_is_the_rotated_block_of_stream_zero():
    """RT_HYPER_SHARED_DRAWS in the checker: element i of stream s takes draw ((i & 7) + 2 s) & 7 of
    the stream-0 block of its group -- restated here with the numpy Philox."""
    n, seed, tid, step, index0 = 1000, 77, 3, 9, 16
    h = oracle.make_hyper(1e-4, (0.9, 0.999), 1e-8, 0.01, step, shared_draws=True)
    rng = np.random.default_rng(0)
    p = oracle.f32_to_bf16_bits_rn(rng.normal(0, 0.02, n).astype(np.float32))
    g = oracle.f32_to_bf16_bits_rn(rng.normal(0, 1e-3, n).astype(np.float32))
    m = oracle.f32_to_bf16_bits_rn(rng.normal(0, 1e-3, n).astype(np.float32))
    v = oracle.f32_to_bf16_bits_rn(np.abs(rng.normal(0, 1e-6, n)).astype(np.float32))
    p1, m1, v1 = p.copy(), m.copy(), v.copy()
    fp, fm, fv = oracle.adamw_sr(p1, g, m1, v1, oracle.BF16, oracle.BF16, oracle.BF16, h, seed=seed,
                                 tensor_id=tid, index0=index0, want_f32=True)
    i = np.arange(index0, index0 + n)
    block = oracle.draws_np(seed, tid, step, 0, (index0 // 8) * 8, ((index0 + n + 7) // 8) * 8 - (index0 // 8) * 8)
    base = (index0 // 8) * 8
    for s, (f32, out) in enumerate(((fp, p1), (fm, m1), (fv, v1))):
        lane = (i & ~7) | (((i & 7) + 2 * s) & 7)
        r = block[lane - base]
        assert (oracle.sr_round_np(f32, r) == out).all()


def test_bench_workload_generators_match_the_configs():
    import bench
    shapes = bench.llama_shapes()
    assert len(shapes) == 291
    assert sum(int(np.prod(s)) for s in shapes) == 6_738_415_616
    ragged = bench.ragged_shapes()
    assert len(ragged) == 20000
    total = sum(int(np.prod(s)) for s in ragged)
    assert 7.4e9 < total < 7.6e9                      # log-uniform(64, 4194304) x 20000, as specified
    assert all(len(s) == 1 for s in ragged if np.prod(s) < 16384)


def test_alias_package_serves_the_reference_import_paths():
    import ramtorch
    import ramtorch_b200
    from ramtorch.stochastic_optimizers.adamw import AdamW, copy_stochastic_
    from ramtorch.zero1 import broadcast_zero_params, create_zero_param_groups
    from ramtorch.zero2 import setup_grad_sharding_hooks
    assert AdamW is ramtorch_b200.AdamW and ramtorch.AdamW is AdamW
    assert create_zero_param_groups is ramtorch_b200.zero1.create_zero_param_groups
    assert setup_grad_sharding_hooks is ramtorch_b200.zero2.setup_grad_sharding_hooks
    with pytest.raises(AttributeError):
        ramtorch.Linear
