"""CPU: host-side logic of the drop-in optimizer that needs no GPU -- constructor contract, state
layout, tensor-id bookkeeping, hyper-parameter scalars, and the loud failure without a device."""
import pytest
import torch

import oracle
from ramtorch_b200 import AdamW, _native as N
from ramtorch_b200.stochastic_optimizers.adamw import _grad_of
from ramtorch_b200.zero1 import create_zero_param_groups

CPU = torch.device("cpu")      # the non-string form: unpinned state, as in the reference (adamw.py:91)


def test_constructor_contract_matches_the_reference():
    p = torch.zeros(3, 5, dtype=torch.bfloat16)
    q = torch.zeros(7, dtype=torch.float32)
    opt = AdamW([p, q], storage_device=CPU)
    assert opt.defaults == dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, centralization=0)
    assert (opt.chunk_size, opt.optim_state_dtype, opt.optim_state_device) == (64, torch.bfloat16, CPU)
    for t in (p, q):
        st = opt.state[t]
        assert set(st) == {"step", "ema", "ema_squared"} and st["step"] == 0
        for key in ("ema", "ema_squared"):
            assert st[key].shape == t.shape and st[key].dtype == torch.bfloat16 and st[key].device.type == "cpu"
            assert float(st[key].float().abs().sum()) == 0
    sd = opt.state_dict()
    assert sorted(sd["state"]) == [0, 1] and set(sd["param_groups"][0]) >= {"lr", "betas", "eps", "weight_decay", "centralization"}


def test_bad_arguments_are_rejected_at_construction():
    p = torch.zeros(4)
    with pytest.raises(ValueError):
        AdamW([p], dtype=torch.float64, storage_device=CPU)
    with pytest.raises(ValueError):
        AdamW([p], storage_device=CPU, offload_chunk_elems=12)
    with pytest.raises(ValueError):
        AdamW([p], storage_device=CPU, offload_ring_depth=1)


def test_tensor_ids_follow_group_order_or_the_zero_plan():
    a, b, c, d = (torch.zeros(2) for _ in range(4))
    opt = AdamW([{"params": [a, b]}, {"params": [c]}], storage_device=CPU)
    assert [opt._tensor_ids[t] for t in (a, b, c)] == [0, 1, 2]
    opt.add_param_group({"params": [d]})
    assert opt._tensor_ids[d] == 3 and not opt.state[d]        # late parameters get their state lazily
    # ZeRO: the ids are the global positions, whatever the rank
    rpg = create_zero_param_groups([{"params": [a, b, c]}, {"params": [d]}], 2)
    o0, o1 = AdamW(rpg[0], storage_device=CPU), AdamW(rpg[1], storage_device=CPU)
    assert [o0._tensor_ids[t] for t in (a, c)] == [0, 2] and o0._tensor_ids[d] == 3
    assert o1._tensor_ids[b] == 1
    with pytest.raises(ValueError):
        AdamW([{"params": [a, b], "rt_param_ids": [0]}], storage_device=CPU)


def test_step_fails_loudly_without_a_cuda_device():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    p = torch.zeros(8, dtype=torch.bfloat16)
    p.grad = torch.zeros_like(p)
    opt = AdamW([p], storage_device=CPU)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        opt.step()
    assert opt.state[p]["step"] == 0


@pytest.mark.parametrize("step", [1, 2, 11, 100, 54321])
@pytest.mark.parametrize("wd", [0.0, 0.01])
def test_native_and_checker_scalars_are_identical(step, wd):
    for shared in (False, True):
        for ref in (False, True):
            a = N.make_hyper(1e-4, (0.9, 0.999), 1e-8, wd, step, shared_draws=shared, reference_order=ref)
            b = oracle.make_hyper(1e-4, (0.9, 0.999), 1e-8, wd, step, shared_draws=shared, reference_order=ref)
            assert bytes(a) == bytes(b)
            assert a.flags == (N.HYPER_SHARED_DRAWS if shared else 0) | (N.HYPER_REFERENCE_ORDER if ref else 0)
    assert abs(a.inv_bias_correction2_sqrt * a.bias_correction2_sqrt - 1) < 1e-6


def test_device_gradient_attribute_only_applies_to_cpu_parameters():
    p = torch.zeros(4)
    p.grad = torch.ones(4)
    assert _grad_of(p) is p.grad
    p.rt_device_grad = torch.full((4,), 2.0)
    assert _grad_of(p) is p.rt_device_grad
    p.rt_device_grad = None
    assert _grad_of(p) is p.grad


def test_reattach_is_ramtorch_flags_marks_the_tensors_of_flagged_modules_only():
    """helpers.py:229-253: parameters and buffers that directly belong to a module declaring
    ``is_ramtorch = True`` get the flag back; everything else is left alone."""
    import copy
    from ramtorch_b200.helpers import reattach_is_ramtorch_flags

    class Bouncing(torch.nn.Linear):
        is_ramtorch = True

    model = torch.nn.Sequential(Bouncing(4, 4), torch.nn.LayerNorm(4), torch.nn.Sequential(Bouncing(4, 2, bias=False)))
    model[0].register_buffer("scale", torch.ones(1))
    for p in model[0].parameters():
        p.is_ramtorch = True
    clone = copy.deepcopy(model)                         # tensor attributes do not survive this (nor torch.save)
    assert not any(getattr(p, "is_ramtorch", False) for p in clone.parameters())
    assert reattach_is_ramtorch_flags(clone) is clone
    flagged = {n for n, p in clone.named_parameters() if getattr(p, "is_ramtorch", False)}
    assert flagged == {"0.weight", "0.bias", "2.0.weight"}
    assert getattr(clone[0].scale, "is_ramtorch", False) and not hasattr(clone[1].weight, "is_ramtorch")


def test_byte_balanced_ownership_keeps_the_dict_shape_and_evens_out_the_segments():
    from ramtorch_b200._shard_plan import plan_for
    from ramtorch_b200.zero1 import create_zero_param_groups
    sizes = [1000, 8, 8, 8, 900, 8, 8, 8, 1100, 8, 8, 8]          # round-robin by count gives rank 0 every big tensor
    norms = [torch.zeros(3) for _ in range(2)]
    params = [torch.zeros(n) for n in sizes]
    groups = [{"params": norms, "weight_decay": 0.0}, {"params": params, "tag": "w"}]
    by_count = create_zero_param_groups(groups, 4)
    by_bytes = create_zero_param_groups(groups, 4, balance="bytes")
    for rpg in (by_count, by_bytes):
        assert sorted(rpg) == [0, 1, 2, 3] and all(len(rpg[r]) == 2 for r in rpg)
        assert all(rpg[r][1]["tag"] == "w" and rpg[r][0]["weight_decay"] == 0.0 for r in rpg)
        owned = [id(p) for r in rpg for g in rpg[r] for p in g["params"]]
        assert sorted(owned) == sorted(map(id, norms + params))                    # every tensor exactly once
        ids = sorted(i for r in rpg for g in rpg[r] for i in g["rt_param_ids"])
        assert ids == list(range(len(norms) + len(params)))                        # global positions, whatever the owner
    load = lambda rpg: [sum(p.numel() for g in rpg[r] for p in g["params"]) for r in rpg]
    assert max(load(by_count)) == 3003 and max(load(by_bytes)) <= 1100 + 16
    assert plan_for(by_bytes).buckets and max(load(by_bytes)) < max(load(by_count)) / 2
    # the same position keeps the same id in both assignments: the random bits do not depend on the owner
    pos = {id(p): i for r in by_count for g in by_count[r] for p, i in zip(g["params"], g["rt_param_ids"])}
    assert all(pos[id(p)] == i for r in by_bytes for g in by_bytes[r] for p, i in zip(g["params"], g["rt_param_ids"]))
    with pytest.raises(ValueError):
        create_zero_param_groups(groups, 4, balance="size")


def test_device_gradient_producer_validates_its_arguments():
    from ramtorch_b200.helpers import accumulate_device_grad
    p = torch.zeros(4)
    with pytest.raises(ValueError, match="HBM"):
        accumulate_device_grad(p, torch.ones(4))
