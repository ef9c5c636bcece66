"""GPU (needs >= 2 devices): the whole ZeRO loop — flat reduce-scatter of gradients, owner-only fused
SR-AdamW step, flat all-gather of parameters — on NCCL ranks, against a single-process run of the
same optimizer on the summed gradients.  With the same seed the parameters must come out
bit-identical whatever the world size (the random bits are keyed by global parameter id)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

SHAPES = [(257, 64), (64,), (1000, 33), (33,), (4096,), (8, 8, 8), (70001, 1), (5,), (129, 128)]
HP = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
STEPS = 5


def _params(device):
    """bf16 weights and fp32 vectors (norm scales are often kept in fp32): two flat buckets, of which
    only the larger one is peer-mapped."""
    g = torch.Generator().manual_seed(0)
    return [torch.nn.Parameter((torch.randn(s, generator=g) * 0.02).to(torch.float32 if len(s) == 1 else torch.bfloat16)
                               .to(device)) for s in SHAPES]


def _grad(step, rank, k, shape, exact=True):
    g = torch.Generator().manual_seed(1000 * step + 10 * rank + k)
    if not exact and len(shape) > 1:
        # random values for the (bf16, peer-mapped) weights only: the fp32 vectors go through NCCL,
        # whose summation order is unspecified beyond two ranks
        return (torch.randn(shape, generator=g) * 1e-3).bfloat16()
    # multiples of 2^-14 with few significant bits: sums of up to 8 ranks are exact in bf16, so the
    # order in which NCCL adds them cannot matter
    return (torch.randint(-8, 9, shape, generator=g).float() * 2.0 ** -14).bfloat16()


def _groups(params):
    return [{"params": [p for p in params if p.dim() == 1], "weight_decay": 0.0},
            {"params": [p for p in params if p.dim() > 1]}]


def _worker(rank, world, port, out, mode, exact):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    fused = mode != "all-gather"
    os.environ["RT_ZERO_FUSED_PUSH"] = "1" if fused else "0"
    os.environ["RT_ZERO2_FUSED_PULL"] = "1" if mode == "peer-push+grad-pull" else "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from ramtorch_b200 import AdamW
        from ramtorch_b200.zero1 import broadcast_zero_params, create_zero_param_groups
        from ramtorch_b200.zero2 import setup_grad_sharding_hooks
        params = _params(dev)
        rpg = create_zero_param_groups(_groups(params), world)
        setup_grad_sharding_hooks(rpg, rank)
        opt = AdamW(rpg[rank], dtype=torch.bfloat16, storage_device=dev, seed=21, **HP)
        for step in range(STEPS):
            # a "backward": every parameter receives this rank's gradient through autograd; on odd
            # steps in two micro-batches (gradient accumulation) whose halves add up exactly
            grads = [_grad(step, rank, k, p.shape, exact).to(dev, p.dtype) for k, p in enumerate(params)]
            if step % 2 == 1 and exact:
                halves = [(g * 0.5, g - g * 0.5) for g in grads]      # powers of two: exact in bf16
                for part in (0, 1):
                    sum((p * h[part]).sum() for p, h in zip(params, halves)).backward()
            else:
                sum((p * g).sum() for p, g in zip(params, grads)).backward()
            opt.step()
            broadcast_zero_params(rpg)
            for p in params:
                p.grad = None if step % 2 == 0 else p.grad.zero_()
        torch.cuda.synchronize()
        from ramtorch_b200._shard_plan import plan_for
        buckets = {str(b.dtype): b for b in plan_for(rpg).buckets.values()}
        big, small = buckets["torch.bfloat16"], buckets["torch.float32"]
        assert str(big.mode) == ("push" if fused else "None") and small.peer_ptrs is None and small.mode is None
        assert (big.gpeer_ptrs is not None) == (mode == "peer-push+grad-pull") and small.gpeer_ptrs is None
        out.put((rank, "ok", [p.detach().float().cpu() for p in params]))
    except Exception as e:
        import traceback
        out.put((rank, "error", traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _single_process(world, exact=True, fp32_sum=False):
    """The same optimisation in one process on the summed gradients.  ``fp32_sum``: the sum is kept
    in fp32, accumulated in rank order -- what the fused reduction computes; otherwise it is rounded
    to bf16 like an NCCL reduction of bf16 buffers."""
    from ramtorch_b200 import AdamW
    dev = torch.device("cuda", 0)
    params = _params(dev)
    if fp32_sum:
        for p in params:
            p.grad_dtype = None
    opt = AdamW(_groups(params), dtype=torch.bfloat16, storage_device=dev, seed=21, **HP)
    for step in range(STEPS):
        for k, p in enumerate(params):
            total = _grad(step, 0, k, p.shape, exact).float()
            for r in range(1, world):
                total = total + _grad(step, r, k, p.shape, exact).float()
            if p.dtype == torch.float32:
                p.grad = total.to(dev)           # fp32 bucket: NCCL sums fp32 (exact here, or two ranks)
            else:
                p.grad = (total if fp32_sum else total.bfloat16()).to(dev)
        opt.step()
    return [p.detach().float().cpu() for p in params]


def _collect(out, procs, deadline_s=300.0):
    """One report per worker, or a failure naming the workers that died or ran out of time: a
    worker that exits before reporting must not leave the test waiting on the queue forever."""
    import queue
    import time
    results, t_end = [], time.monotonic() + deadline_s
    while len(results) < len(procs):
        try:
            results.append(out.get(timeout=2.0))
            continue
        except queue.Empty:
            pass
        reported = {r[0] for r in results}
        dead = [k for k, p in enumerate(procs) if not p.is_alive() and k not in reported]
        if dead or time.monotonic() > t_end:
            try:                                  # a report may have arrived between the two checks
                while True:
                    results.append(out.get(timeout=1.0))
            except queue.Empty:
                pass
            reported = {r[0] for r in results}
            missing = [k for k in range(len(procs)) if k not in reported]
            if not missing:
                break
            for p in procs:
                if p.is_alive():
                    p.terminate()
            why = "exited without reporting" if dead else f"did not report within {deadline_s:.0f} s"
            pytest.fail(f"workers {missing} {why} (exit codes {[procs[k].exitcode for k in missing]})")
    return sorted(results, key=lambda r: r[0])


@pytest.mark.parametrize("mode,exact", [("peer-push", True), ("all-gather", True), ("peer-push+grad-pull", True),
                                        ("peer-push+grad-pull", False)])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_zero_loop_matches_single_process(world, mode, exact):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, world, port, out, mode, exact)) for r in range(world)]
    for p in procs:
        p.start()
    results = _collect(out, procs)
    for p in procs:
        p.join(timeout=120)
    want = _single_process(world, exact, fp32_sum=(mode == "peer-push+grad-pull"))
    for rank, status, payload in results:
        assert status == "ok", f"rank {rank}: {payload}"
        for k, (a, b) in enumerate(zip(payload, want)):
            assert torch.equal(a, b), f"rank {rank} parameter {k} differs from the single-process run"
