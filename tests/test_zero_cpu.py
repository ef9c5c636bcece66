"""CPU: the ZeRO-1 / ZeRO-2 host logic on gloo ranks (world_size 2 and 3) and against the ownership
maps recorded from the reference.  No GPU and no optimizer kernel involved: the "optimizer" here
is a plain in-place edit of the parameters a rank owns."""
import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ramtorch_b200 import helpers
from ramtorch_b200._shard_plan import ShardPlan, plan_for
from ramtorch_b200.zero1 import PARAM_IDS_KEY, broadcast_zero_params, create_zero_param_groups
from ramtorch_b200.zero2 import setup_grad_sharding_hooks
from util import GOLDEN


def test_ownership_matches_the_reference_fixtures():
    with open(os.path.join(GOLDEN, "zero1_ownership.json")) as f:
        cases = json.load(f)
    for c in cases:
        groups, k = [], 0
        for gi, n in enumerate(c["group_sizes"]):
            params = [torch.zeros(1) for _ in range(n)]
            for t in params:
                t.tag = k
                k += 1
            groups.append({"params": params, "lr": 0.1 * (gi + 1), "foo": f"g{gi}"})
        rpg = create_zero_param_groups(groups, c["world_size"])
        assert sorted(rpg) == list(range(c["world_size"]))
        for r, gl in rpg.items():
            assert [[p.tag for p in g["params"]] for g in gl] == c["ownership"][str(r)]
            for g, extra in zip(gl, c["extra_keys"][str(r)]):
                assert {k2: v for k2, v in g.items() if k2 not in ("params", PARAM_IDS_KEY)} == extra
                # ids are the global positions, so they equal the tags assigned above
                assert g[PARAM_IDS_KEY] == [p.tag for p in g["params"]]
        # references, not copies
        assert rpg[0][0]["params"][0] is groups[0]["params"][0] if c["group_sizes"][0] else True


def test_flat_layout_is_owner_ordered_equal_segments_and_keeps_values():
    params = [torch.arange(n, dtype=torch.float32) + 100 * k for k, n in enumerate([5, 300, 7, 64, 1])]
    before = [p.clone() for p in params]
    rpg = create_zero_param_groups([{"params": params}], 2)
    plan = plan_for(rpg)
    assert plan is plan_for(rpg)
    (bucket,) = plan.buckets.values()
    assert bucket.segment % 64 == 0 and bucket.segment >= 5 + 7 + 1
    plan.flatten_params()
    for p, b, owner, off in zip(bucket.params, [before[0], before[2], before[4], before[1], before[3]],
                                bucket.owner, bucket.offset):
        assert torch.equal(p, b)
        assert owner * bucket.segment <= off < (owner + 1) * bucket.segment
        assert off % 64 == 0
        assert p.data_ptr() == bucket.flat.data_ptr() + 4 * off
    # a hand-built plain dict works too
    plain = {0: [{"params": [torch.ones(3)]}], 1: [{"params": [torch.ones(4)]}]}
    assert isinstance(plan_for(plain), ShardPlan) and plan_for(plain) is plan_for(plain)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("balance", ["count", "bytes"])
def test_gradient_pieces_cover_every_gradient_once_and_stay_balanced(world, balance, monkeypatch):
    """Layout of the flat gradient buffer for a Llama-like list (meta tensors, no memory): every
    gradient lies in exactly one piece, inside its owner's part; parts of a piece are equally long;
    pieces follow the order in which backward completes the parameters; and a piece is never mostly
    padding (the rule that keeps one huge tensor from forming a piece of empty parts)."""
    monkeypatch.setenv("RT_ZERO2_BUCKET_MB", "8")
    shapes = [(3200, 512)] + [s for _ in range(6) for s in [(512, 512)] * 4 + [(1376, 512)] * 2 + [(512, 1376), (512,), (512,)]]
    shapes += [(512,), (3200, 512)]
    params = [torch.empty(s, dtype=torch.bfloat16, device="meta") for s in shapes]
    rpg = create_zero_param_groups([{"params": params}], world, balance=balance)
    plan = plan_for(rpg)
    (b,) = plan.buckets.values()
    total = plan._layout_grad_pieces(b)
    spans = sorted((b.goffset[k], b.goffset[k] + p.numel()) for k, p in enumerate(b.params))
    assert all(x[1] <= y[0] for x, y in zip(spans, spans[1:])) and spans[-1][1] <= total
    useful = sum(p.numel() for p in params)
    if balance == "bytes":
        assert total <= 1.35 * useful                               # bounded padding overall
    held = [0] * len(b.subs)
    for k, p in enumerate(b.params):
        held[b.sub_of[k]] += (p.numel() + 127) // 128 * 128
    for sub, inside in list(zip(b.subs, held))[:-1]:                # every piece but the (merged) last
        assert (sub.part * world - inside) * 8 < sub.part * world
    for k, p in enumerate(b.params):
        sub = b.subs[b.sub_of[k]]
        lo = sub.start + b.owner[k] * sub.part
        assert lo <= b.goffset[k] and b.goffset[k] + p.numel() <= lo + sub.part
        assert b.goffset[k] % 128 == 0                               # 256-byte aligned views
    assert [s.start for s in b.subs] == sorted(s.start for s in b.subs)
    assert all(b.subs[i].start + b.subs[i].part * world == b.subs[i + 1].start for i in range(len(b.subs) - 1))
    # backward order: a parameter registered later never sits in a later piece than one registered earlier
    by_order = sorted(range(len(b.params)), key=lambda k: b.order[k])
    pieces_in_registration_order = [b.sub_of[k] for k in by_order]
    assert pieces_in_registration_order == sorted(pieces_in_registration_order, reverse=True)
    if world == 2:
        assert len(b.subs) >= 2                                      # 44 MB of gradients, 8 MiB target


def test_hook_dict_protocol():
    t = torch.zeros(2)
    a = helpers.register_ramtorch_hook(t, lambda g: g * 2, "_ramtorch_zero_2_hooks")
    b = helpers.register_ramtorch_hook(t, lambda g: None, "_ramtorch_zero_2_hooks")
    assert (a, b) == (0, 1) and t._ramtorch_zero_2_hooks_counter == 2
    assert list(t._ramtorch_zero_2_hooks) == [0, 1]
    assert torch.equal(helpers.invoke_ramtorch_hooks(t, torch.ones(2)), torch.full((2,), 2.0))
    assert helpers.remove_ramtorch_hook(t, 0, "_ramtorch_zero_2_hooks")
    assert helpers.register_ramtorch_hook(t, lambda g: g, "_ramtorch_zero_2_hooks") == 2


# ------------------------------------------------------------------------------------------
# multi-process part
# ------------------------------------------------------------------------------------------
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(13, 32), torch.nn.Tanh(), torch.nn.Linear(32, 7, bias=False),
                               torch.nn.Tanh(), torch.nn.Linear(7, 3))


def _deep_model(seed=0):
    """Six weight matrices of (nearly) the same size: consecutive tensors balance the ranks' parts
    quickly, so small gradient pieces really are cut."""
    torch.manual_seed(seed)
    layers = [torch.nn.Linear(13, 16, bias=False)]
    for _ in range(5):
        layers += [torch.nn.Tanh(), torch.nn.Linear(16, 16, bias=False)]
    return torch.nn.Sequential(*layers)


def _worker(rank, world, port, scenario, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        result = SCENARIOS[scenario](rank, world)
        out.put((rank, "ok", result))
    except Exception as e:  # report instead of hanging the other ranks' collectives
        out.put((rank, "error", f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def _spawn(scenario, world):
    import queue
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in procs:
            results.append(out.get(timeout=180))      # a worker that died must not hang the test
    except queue.Empty:
        for p in procs:
            if p.is_alive():
                p.terminate()
        pytest.fail(f"only {len(results)} of {world} workers reported (exit codes {[p.exitcode for p in procs]})")
    for p in procs:
        p.join(timeout=60)
    return sorted(results)


def _scenario_full_loop(rank, world, make=_model):
    """ZeRO-2 reduce + owner-only update + ZeRO-1 redistribution over two steps with gradient
    accumulation, compared with a single-process run on the summed gradients."""
    model, ref = make(), make()
    groups = [{"params": [p for n, p in model.named_parameters() if n.endswith("bias")], "tag": "b"},
              {"params": [p for n, p in model.named_parameters() if n.endswith("weight")], "tag": "w"}]
    rpg = create_zero_param_groups(groups, world)
    handles = setup_grad_sharding_hooks(rpg, rank)
    assert len(handles) == sum(len(g["params"]) for g in groups)
    mine = [p for g in rpg[rank] for p in g["params"]]
    for step in range(2):
        for micro in range(2):                   # gradient accumulation: two backward passes
            for r in range(world):               # the reference run sees every rank's batch
                x = torch.randn(4, 13, generator=torch.Generator().manual_seed(100 * step + 10 * micro + r))
                if r == rank:
                    model(x).square().sum().backward()
                ref(x).square().sum().backward()
        from ramtorch_b200.zero2 import finish_grad_sync
        finish_grad_sync()
        # owner's gradient = SUM over ranks (and over micro-batches)
        ref_params = dict(ref.named_parameters())
        for n, p in model.named_parameters():
            if any(p is q for q in mine):
                assert torch.allclose(p.grad, ref_params[n].grad, rtol=1e-5, atol=1e-6), n
        with torch.no_grad():
            for p in mine:                       # stand-in optimizer: owners update their tensors
                p.data.sub_(0.1 * p.grad)
            for p in ref.parameters():
                p.sub_(0.1 * p.grad)
        assert broadcast_zero_params(rpg) is None
        for (n, p), q in zip(model.named_parameters(), ref.parameters()):
            assert torch.allclose(p, q, rtol=1e-5, atol=1e-6), n
        if step == 0:
            model.zero_grad(set_to_none=True)    # drops the flat views; the hooks fold them back
        else:
            model.zero_grad(set_to_none=False)
        ref.zero_grad()
    return True


def _scenario_small_pieces(rank, world):
    """The same loop with gradient pieces of 256 bytes: several reduce-scatters per backward, launched
    as their pieces complete, with a partial backward (unused head) in between."""
    os.environ["RT_ZERO2_BUCKET_MB"] = str(256 / (1 << 20))
    try:
        from ramtorch_b200._shard_plan import plan_for as _pf
        ok = _scenario_full_loop(rank, world, make=_deep_model)
        # and the layout really was cut up: rebuild the plan of an equal model to look at it
        model = _deep_model()
        rpg = create_zero_param_groups([{"params": list(model.parameters())}], world)
        setup_grad_sharding_hooks(rpg, rank)
        (bucket,) = _pf(rpg).buckets.values()
        pieces = len(bucket.subs)
        covered = sorted((bucket.goffset[k], bucket.goffset[k] + p.numel()) for k, p in enumerate(bucket.params))
        disjoint = all(a[1] <= b[0] for a, b in zip(covered, covered[1:]))
        for p in model.parameters():
            assert p.grad.data_ptr() == bucket.gflat.data_ptr() + 4 * bucket.goffset[[id(q) for q in bucket.params].index(id(p))]
        # a backward that leaves the last layer out: step time reduces every piece on every rank
        from ramtorch_b200.zero2 import finish_grad_sync
        x = torch.randn(4, 13, generator=torch.Generator().manual_seed(rank))
        model[:5](x).square().sum().backward()
        finish_grad_sync()
        first = model[0].weight
        mine = any(first is q for g in rpg[rank] for q in g["params"])
        total = torch.zeros_like(first)
        for r in range(world):
            ref = _deep_model()
            xr = torch.randn(4, 13, generator=torch.Generator().manual_seed(r))
            ref[:5](xr).square().sum().backward()
            total += ref[0].weight.grad
        partial_ok = (not mine) or torch.allclose(first.grad, total, rtol=1e-5, atol=1e-6)
        return True if (ok and pieces >= 2 and disjoint and partial_ok) else (ok, pieces, disjoint, partial_ok)
    finally:
        os.environ.pop("RT_ZERO2_BUCKET_MB", None)


def _scenario_plan_mismatch(rank, world):
    """A rank whose parameter list differs must be caught on the host before any data collective."""
    params = [torch.zeros(4), torch.zeros(6 if rank == 0 else 8)]
    rpg = create_zero_param_groups([{"params": params}], world)
    try:
        broadcast_zero_params(rpg)
    except RuntimeError as e:
        return "differ" in str(e)
    return False


def _scenario_ramtorch_hooks(rank, world):
    """CPU-shared parameters keep the hook-dict protocol and the per-tensor synchronous reduce."""
    w = torch.nn.Parameter(torch.zeros(5))
    w.is_ramtorch = True
    plain = torch.nn.Parameter(torch.ones(3) * (rank + 1))
    rpg = create_zero_param_groups([{"params": [w, plain]}], world)
    handles = setup_grad_sharding_hooks(rpg, rank)
    assert isinstance(handles[0], int) and hasattr(w, "_ramtorch_zero_2_hooks")
    grad = torch.full((5,), float(rank + 1))
    out = helpers.invoke_ramtorch_hooks(w, grad)
    total = float(sum(range(1, world + 1)))
    owner_ok = (rank != 0) or bool((out == total).all())
    broadcast_zero_params(rpg)                   # skips w, redistributes `plain` from rank 1
    return owner_ok and bool((plain == 2.0).all()) and bool((w == 0).all())


def _scenario_rank_leaves(rank, world):
    """Failure made on the host: rank 1 leaves between steps (no collective in flight).  Rank 0's
    next redistribution must end with an exception within the process-group timeout, not hang."""
    params = [torch.zeros(4), torch.ones(6)]
    rpg = create_zero_param_groups([{"params": params}], world)
    broadcast_zero_params(rpg)                   # one healthy step with everybody present
    if rank == 1:
        return True                              # leaves: the worker tears its process group down
    import time
    t0 = time.time()
    try:
        for _ in range(3):
            broadcast_zero_params(rpg)
            time.sleep(0.5)
    except Exception as e:                        # gloo: connection closed / reset / timed out
        return time.time() - t0 < 30 and isinstance(e, (RuntimeError, ValueError))
    return False


SCENARIOS = {"rank_leaves": _scenario_rank_leaves, "full_loop": _scenario_full_loop, "plan_mismatch": _scenario_plan_mismatch,
             "ramtorch_hooks": _scenario_ramtorch_hooks, "small_pieces": _scenario_small_pieces}


@pytest.mark.parametrize("scenario,world", [("full_loop", 2), ("full_loop", 3), ("small_pieces", 2), ("small_pieces", 3),
                                            ("plan_mismatch", 2), ("ramtorch_hooks", 2), ("rank_leaves", 2)])
def test_gloo_ranks(scenario, world):
    results = _spawn(scenario, world)
    assert len(results) == world
    for rank, status, payload in results:
        assert status == "ok", f"rank {rank}: {payload}"
        assert payload is True, f"rank {rank} returned {payload}"


def test_world_size_one_needs_no_process_group():
    """The single-process case of the README loop: every call is a no-op or purely local."""
    model = _model()
    rpg = create_zero_param_groups([{"params": list(model.parameters())}], 1)
    handles = setup_grad_sharding_hooks(rpg, 0)
    assert len(handles) == len(list(model.parameters()))
    model(torch.randn(4, 13)).square().sum().backward()
    want = [p.grad.clone() for p in model.parameters()]
    from ramtorch_b200.zero2 import finish_grad_sync
    finish_grad_sync()
    assert broadcast_zero_params(rpg) is None
    for p, g in zip(model.parameters(), want):
        assert torch.equal(p.grad, g)
    # the parameters were packed into the flat buffer without changing their values
    fresh = _model()
    for p, q in zip(model.parameters(), fresh.parameters()):
        assert torch.equal(p, q)
