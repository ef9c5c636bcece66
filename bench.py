#!/usr/bin/env python
"""Benchmark of the SR-AdamW optimizer step (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: a 1,073,741,824-element bf16 parameter shard per GPU with fp32 moments, gradients
~N(0,1e-3), step counter at 100 (the "pure memory-bound roofline case").  A step is one
``AdamW.step()`` over that shard; with N > 1 every rank owns one such shard of an N-times larger
flat parameter space (ZeRO-1) and the step ends with the all-gather of the updated parameters.

  value     params updated / s, inputs resident in HBM, CUDA-event timed, max over ranks
  e2e       same metric with parameters, gradients and moments in pinned HOST memory, streamed
            through the GPU by ``AdamW.step()`` (copies inside the timed region)
  roofline  algorithmic bytes (22 B/element) / kernel time against the measured HBM copy peak
  cpu_baseline / --impl reference
            the CPU restatement of the reference step (oracle/, C + OpenMP, all host threads) on
            a bounded sample of the same workload
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sr_adamw_params_per_s"
UNIT = "params/s"
ELEMS_PER_GPU = 1 << 30
BYTES_PER_ELEM = 22            # read p2 g2 m4 v4, write p2 m4 v4
HP = dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
START_STEP = 99                # the timed steps start at t = 100
# DRAM bytes per element of the fused kernel (bf16 p/g, fp32 moments) measured with ncu
# (dram__bytes_read.sum + dram__bytes_write.sum over one launch of 2^27 elements, see profiles/);
# traffic is proportional to the element count, so it is scaled to the launch timed here.
NCU_DRAM_BYTES_PER_ELEM = 21.6
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML on a thread while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index, period=0.004):
        self.rows, self.stop_flag, self.ok = [], False, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            ids = [v for v in vis.split(",") if v.strip().isdigit()]
            phys = int(ids[index]) if index < len(ids) else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.period = period
            self.ok = True
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception as e:  # no NVML: report that instead of numbers
            self.err = repr(e)

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.rows.append((time.time(), sm, rs))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self, t0, t1):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + self.err]}
        self.stop_flag = True
        self.thread.join(timeout=1.0)
        rows = [r for r in self.rows if t0 <= r[0] <= t1] or self.rows[-3:]
        sm = sorted(r[1] for r in rows)
        reasons = set()
        for _, _, rs in rows:
            for bit, name in self.REASONS.items():
                if rs & bit:
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_sm,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(seconds=12.0, sample_elems=1 << 26, warmup=1, steps=None):
    """The CPU restatement of the reference step on all host threads, on a sample of the
    workload (same dtypes and distributions)."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(0)
    n = sample_elems

    def normal(scale):
        out = np.empty(n, np.float32)
        blk = 1 << 22
        for lo in range(0, n, blk):
            out[lo:lo + blk] = rng.standard_normal(min(blk, n - lo), dtype=np.float32) * scale
        return out

    p = oracle.f32_to_bf16_bits_rn(normal(0.02))
    g = oracle.f32_to_bf16_bits_rn(normal(1e-3))
    m = normal(1e-3)
    v = np.abs(normal(1e-6))
    threads = oracle.use_all_cores()
    times, k = [], 0
    t_end = time.time() + seconds
    while True:
        h = oracle.make_hyper(HP["lr"], HP["betas"], HP["eps"], HP["weight_decay"], START_STEP + 1 + k)
        t0 = time.perf_counter()
        oracle.adamw_sr(p, g, m, v, oracle.BF16, oracle.BF16, oracle.F32, h, seed=0, tensor_id=0)
        dt = time.perf_counter() - t0
        k += 1
        if k > warmup:
            times.append(dt)
        if steps is not None:
            if len(times) >= steps:
                break
        elif time.time() > t_end and len(times) >= 3:
            break
    mean = sum(times) / len(times)
    return {"value": n / mean, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{n} elements (1/{ELEMS_PER_GPU // n} of one shard), bf16 p/g + fp32 moments, "
                      f"{len(times)} steps of the C+OpenMP restatement in oracle/, {threads} threads",
            "ms_per_step": mean * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_baseline(steps=args.steps, warmup=max(args.warmup, 1))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "config 2: bf16 parameter shard with fp32 moments, t=100, on host cores",
                       "elements_per_step": 1 << 26},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def synth_on_device(n, device, seed, state_dtype=None):
    import torch
    state_dtype = state_dtype or torch.float32
    g = torch.Generator(device=device).manual_seed(seed)
    blk = 1 << 28
    p = torch.empty(n, dtype=torch.bfloat16, device=device)
    grad = torch.empty(n, dtype=torch.bfloat16, device=device)
    m = torch.empty(n, dtype=state_dtype, device=device)
    v = torch.empty(n, dtype=state_dtype, device=device)
    for lo in range(0, n, blk):
        hi = min(n, lo + blk)
        p[lo:hi] = torch.randn(hi - lo, device=device, generator=g) * 0.02
        grad[lo:hi] = torch.randn(hi - lo, device=device, generator=g) * 1e-3
        m[lo:hi] = torch.randn(hi - lo, device=device, generator=g) * 1e-3
        v[lo:hi] = (torch.randn(hi - lo, device=device, generator=g) * 1e-6).abs()
    return p, grad, m, v


def host_mem_available_bytes():
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except Exception:
        pass
    return 0


def llama_shapes():
    """The 291 weight tensors of a 32-layer Llama-style decoder (hidden 4096, MLP 11008, vocab
    32000) in module order: embedding, then per layer q k v o gate up down and two norms, the final
    norm, the output head.  6,738,415,616 elements."""
    shapes = [(32000, 4096)]
    for _ in range(32):
        shapes += [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)] + [(4096,)] * 2
    shapes += [(4096,), (32000, 4096)]
    return shapes


def ragged_shapes(count=20000, lo=64, hi=4194304, seed=0):
    """Sizes log-uniform in [lo, hi]; 1-D below 16384 elements, otherwise (size // 1024, 1024)
    rounded down (2-D weights)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    sizes = np.floor(np.exp(rng.uniform(np.log(lo), np.log(hi), count))).astype(np.int64)
    return [(int(s),) if s < 16384 else (int(s) // 1024, 1024) for s in sizes]


def link_ceiling(device, nbytes=1 << 30, reps=4):
    """Pinned cudaMemcpyAsync rates of this box: each direction alone and both at once (GB/s)."""
    import torch
    h_in = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    h_out = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=device)
    d_out = torch.empty(nbytes, dtype=torch.uint8, device=device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def run(h2d, d2h, n):
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        for _ in range(n):
            if h2d:
                with torch.cuda.stream(s_in):
                    d_in.copy_(h_in, non_blocking=True)
            if d2h:
                with torch.cuda.stream(s_out):
                    h_out.copy_(d_out, non_blocking=True)
        torch.cuda.synchronize(device)
        return nbytes * n / (time.perf_counter() - t0) / 1e9

    run(True, True, 1)
    return {"h2d_alone_gbs": run(True, False, reps), "d2h_alone_gbs": run(False, True, reps),
            "both_each_gbs": run(True, True, reps)}


WORKLOADS = {
    "c2": "config 2: one 2^30-element bf16 parameter shard per GPU, fp32 moments, bf16 grads ~N(0,1e-3), t=100",
    "bf16": "2^30-element bf16 parameter shard per GPU, bf16 moments (14 B/element), t=100",
    "c1": "config 1: 16,777,216-element bf16 parameter, bf16 moments, t=11, rotating over 12 buffer sets",
    "c3": "config 3: Llama-style 32-layer decoder shapes (291 tensors, 6.74e9 elements), bf16 moments, ZeRO-1",
    "c5": "config 5: 20,000 ragged bf16 tensors, sizes log-uniform in [64, 4194304], bf16 moments, ZeRO-1",
    "list": "a list of --list-count equal bf16 tensors of --elems elements each, bf16 moments (for profiling the "
            "multi-tensor path on a small case)",
    "c4": "config 4: 8e9 bf16 parameters + bf16 moments in pinned host RAM (60 tensors of 2^27 elements, split "
          "over the ranks), gradients in pinned host RAM too (where the reference's Linear leaves them), streamed "
          "in 256 MiB chunks per tensor through a 2-slot ring",
}


def run_c4(args, device, rank, world, warmup):
    """Host-offloaded step: parameters and moments in pinned CPU RAM, streamed through the GPU."""
    import torch
    import torch.distributed as dist
    from ramtorch_b200 import AdamW, _native as N
    n_tensors, n_each = 60, 1 << 27
    mine = [k for k in range(n_tensors) if k % world == rank]
    budget = host_mem_available_bytes() // max(world, 1)
    while len(mine) * n_each * 8 * 1.2 > budget and len(mine) > 1:
        mine = mine[:-1]
    params = [torch.empty(n_each, dtype=torch.bfloat16, pin_memory=True) for _ in mine]
    opt = AdamW(params, dtype=torch.bfloat16, storage_device="cpu", seed=0, offload_chunk_elems=n_each,
                offload_ring_depth=2, fast_math=args.fast_math, shared_draws=not args.independent_draws, **HP)
    scratch = torch.empty(n_each, dtype=torch.float32, device=device)
    for p in params:
        st = opt.state[p]
        p.copy_(scratch.normal_(0, 0.02)); st["ema"].copy_(scratch.normal_(0, 1e-3))
        st["ema_squared"].copy_(scratch.normal_(0, 1e-6).abs_())
        st["step"] = START_STEP
        if args.grads_in_hbm:
            p.rt_device_grad = torch.empty(n_each, dtype=torch.bfloat16, device=device).normal_(0, 1e-3)
        else:
            p.grad = torch.empty(n_each, dtype=torch.bfloat16, pin_memory=True)
            p.grad.copy_(scratch.normal_(0, 1e-3))
    del scratch
    ceiling = link_ceiling(device) if rank == 0 else None
    steps = max(1, min(args.steps, 3))
    opt.step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(device.index) if rank == 0 else None
    s0 = N.stats()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        opt.step()
        _ = float(params[0][0])
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    s1 = N.stats()
    ms = e0.elapsed_time(e1) / steps
    elems = torch.tensor([float(len(mine) * n_each)], device=device, dtype=torch.float64)
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
        dist.all_reduce(elems, op=dist.ReduceOp.SUM)
    total = int(elems.item())
    h2d = (s1["h2d_bytes"] - s0["h2d_bytes"]) / steps
    d2h = (s1["d2h_bytes"] - s0["d2h_bytes"]) / steps
    if rank == 0:
        value = total / (ms * 1e-3)
        link = {"h2d_gbs_per_gpu": h2d / (ms * 1e-3) / 1e9, "d2h_gbs_per_gpu": d2h / (ms * 1e-3) / 1e9,
                "ceiling": ceiling, "pcie_gen5_x16_nominal_gbs_per_direction": 63.0}
        link["frac_of_measured_bidirectional"] = ((link["h2d_gbs_per_gpu"] + link["d2h_gbs_per_gpu"]) /
                                                  (2 * ceiling["both_each_gbs"]))
        e2e = {"value": value, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": ms}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": 1,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": WORKLOADS["c4"] + ("; variant: gradients kept in HBM" if args.grads_in_hbm else ""),
                           "elements_per_step": total,
                           "l2": "streamed chunks of 1 GiB per slot far exceed L2",
                           "parallelism": f"tensors round-robin over {world} ranks" if world > 1 else "single"},
                "roofline": {"bound": "host link", "achieved": link["h2d_gbs_per_gpu"] + link["d2h_gbs_per_gpu"],
                             "peak": 2 * ceiling["both_each_gbs"], "unit": "GB/s",
                             "frac": link["frac_of_measured_bidirectional"], "traffic": None,
                             "peak_source": "pinned cudaMemcpyAsync both directions at once, same run"},
                "link": link, "e2e": e2e, "cpu_baseline": None,
                "gpu_launches": int(s1["kernel_launches"] - s0["kernel_launches"]),
                "clocks": sampler.stop(t0, t1) if sampler else None}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--elems", type=int, default=ELEMS_PER_GPU, help="elements per GPU for c2/bf16 (default 2^30)")
    ap.add_argument("--list-count", type=int, default=64, help="number of tensors of the 'list' workload")
    ap.add_argument("--e2e-steps", type=int, default=4)
    ap.add_argument("--fast-math", action="store_true", help="approximate sqrt/reciprocal in p' (off by default)")
    ap.add_argument("--independent-draws", action="store_true",
                    help="three independent Philox blocks per eight elements instead of one shared block "
                         "(AdamW(shared_draws=False)); only matters for bf16 moments")
    ap.add_argument("--grads-in-hbm", action="store_true",
                    help="c4 only: gradients of the CPU parameters stay in HBM (p.rt_device_grad)")
    ap.add_argument("--with-grad-sync", action="store_true",
                    help="N > 1: include the ZeRO-2 gradient reduction in every timed step")
    ap.add_argument("--fused-grad-pull", action="store_true",
                    help="N > 1: no reduce-scatter; the optimizer kernel sums the ranks' gradients over NVLink")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from ramtorch_b200 import AdamW, _native as N
    from ramtorch_b200.zero1 import broadcast_zero_params, create_zero_param_groups

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    warmup = max(args.warmup, 3)
    wl = args.workload
    state_dtype = torch.float32 if wl == "c2" else torch.bfloat16
    bytes_per_elem = 22 if wl == "c2" else 14
    start_step = 10 if wl == "c1" else START_STEP

    if wl == "c4":
        return run_c4(args, device, rank, world, warmup)

    # ---------------------------------------------------------------- resident step (value)
    # Every workload is a list of parameters in ONE group handed to create_zero_param_groups, so
    # the reference's round-robin (parameter k -> rank k % world) decides ownership.  A rank
    # holds all parameters (they are replicated) but gradients and moments only for the ones it owns.
    steppers, rpgs = [], []

    def make_set(shapes, seed):
        params = [torch.empty(s, dtype=torch.bfloat16, device=device).normal_(0, 0.02) for s in shapes]
        rpg = create_zero_param_groups([{"params": params}], world)
        owned = rpg[rank][0]["params"]
        opt = AdamW(rpg[rank], dtype=state_dtype, storage_device=device, seed=seed, sync=False,
                    fast_math=args.fast_math, shared_draws=not args.independent_draws, **HP)
        for p in owned:
            p.grad = torch.empty_like(p).normal_(0, 1e-3)
            st = opt.state[p]
            st["ema"].normal_(0, 1e-3)
            st["ema_squared"].normal_(0, 1e-6).abs_()
            st["step"] = start_step
        if world > 1:
            broadcast_zero_params(rpg)   # builds the flat buffer and re-points the parameters into it
        rpgs.append(rpg)
        steppers.append(opt)
        return sum(p.numel() for p in owned)

    if wl in ("c2", "bf16"):
        # one shard per rank: `world` equal tensors, rank r owns tensor r
        owned_elems = make_set([(args.elems,)] * world, 0)
    elif wl == "c1":
        owned_elems = [make_set([(1 << 24,)] * world, k) for k in range(12)][0]
    elif wl == "c3":
        owned_elems = make_set(llama_shapes(), 0)
    elif wl == "list":
        owned_elems = make_set([(args.elems,)] * args.list_count, 0)
    else:
        owned_elems = make_set(ragged_shapes(), 0)
    torch.cuda.synchronize()

    grad_sync = world > 1 and (args.with_grad_sync or args.fused_grad_pull)
    if grad_sync:
        from ramtorch_b200.zero2 import reduce_gradients_now, setup_grad_sharding_hooks
        if args.fused_grad_pull:
            os.environ["RT_ZERO2_FUSED_PULL"] = "1"
        for rpg in rpgs:
            for grp_list in rpg.values():
                for grp in grp_list:
                    for p in grp["params"]:
                        p.requires_grad_(True)
            setup_grad_sharding_hooks(rpg, rank)   # flat gradient buffer; every p.grad becomes a view of it
            from ramtorch_b200._shard_plan import plan_for as _pf
            for bk in _pf(rpg).buckets.values():
                bk.gflat.normal_(0, 1e-3)          # every rank holds a gradient for every parameter

    rs_events = []

    def one_step(k):
        if grad_sync:
            reduce_gradients_now(rpgs[k % len(rpgs)])
            if rs_events is not None and len(rs_events) < 4096:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                rs_events.append(e)
        steppers[k % len(steppers)].step()

    def redistribute(k):
        if world > 1:
            broadcast_zero_params(rpgs[k % len(rpgs)])

    for k in range(max(warmup, len(steppers))):
        one_step(k); redistribute(k)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local) if rank == 0 else None
    rs_events.clear()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    launches0 = N.stats()["kernel_launches"]
    t_wall0 = time.time()
    ev[0].record()
    for k in range(args.steps):
        one_step(k)
        ev[2 * k + 1].record()
        redistribute(k)
        ev[2 * k + 2].record()
    host_ms = (time.time() - t_wall0) * 1e3 / args.steps
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    launches = N.stats()["kernel_launches"] - launches0
    total_ms = ev[0].elapsed_time(ev[2 * args.steps])
    upd_ms = sum(ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(args.steps)) / args.steps
    ag_ms = sum(ev[2 * k + 1].elapsed_time(ev[2 * k + 2]) for k in range(args.steps)) / args.steps
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    sync_ms = None
    if grad_sync and len(rs_events) == args.steps:
        # part of t_update spent in the gradient reduction (NCCL reduce-scatter, or the barrier of the fused path)
        sync_ms = sum(ev[2 * k].elapsed_time(rs_events[k]) for k in range(args.steps)) / args.steps
    elems = torch.tensor([float(owned_elems)], device=device, dtype=torch.float64)
    if world > 1:
        t = torch.tensor([total_ms, upd_ms, ag_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, upd_ms, ag_ms = t.tolist()
        dist.all_reduce(elems, op=dist.ReduceOp.SUM)
    total_elems = int(elems.item())
    ms_per_step = total_ms / args.steps
    value = total_elems / (ms_per_step * 1e-3)

    # the kernel's own duration: steps are enqueued back to back, so the update interval between
    # consecutive events is the kernel (plus a 48-byte hyper-parameter copy); per rank, slowest rank
    peak, which = measured_peak()
    per_rank = total_elems / world
    achieved = bytes_per_elem * per_rank / (upd_ms * 1e-3) / 1e9
    traffic = NCU_DRAM_BYTES_PER_ELEM * per_rank if (wl == "c2" and NCU_DRAM_BYTES_PER_ELEM) else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": which, "traffic": traffic,
                "algorithmic_bytes": bytes_per_elem * per_rank, "kernel_ms": upd_ms,
                "frac_of_nominal_8TBs": achieved / 8000.0}
    if world > 1:
        from ramtorch_b200._shard_plan import plan_for as _plan_for
        if all(bk.mode == "push" for bk in _plan_for(rpgs[0]).buckets.values()):
            # fused update + redistribution: the kernel also stores every updated bf16 parameter into
            # the other ranks' buffers, so its target time is the slower of the HBM time and the
            # NVLink time (bytes leaving this GPU / measured peer-copy rate per direction)
            nvlink_peak = 770.0
            # parameters pushed to the peers, plus (fused reduction) this rank's gradients read by the peers
            egress = 2.0 * per_rank * (world - 1) * (2 if args.fused_grad_pull else 1)
            t_hbm = bytes_per_elem * per_rank / (peak * 1e9)
            t_link = egress / (nvlink_peak * 1e9)
            target = max(t_hbm, t_link)
            roofline = {"bound": "nvlink" if t_link > t_hbm else "hbm",
                        "achieved": egress / (upd_ms * 1e-3) / 1e9 if t_link > t_hbm else achieved,
                        "peak": nvlink_peak if t_link > t_hbm else peak, "unit": "GB/s",
                        "frac": target / (upd_ms * 1e-3), "traffic": None, "kernel_ms": upd_ms,
                        "peak_source": "measured peer copy, 770 GB/s per direction per GPU"
                                       if t_link > t_hbm else which,
                        "nvlink_egress_bytes": egress, "hbm_algorithmic_bytes": bytes_per_elem * per_rank,
                        "target_ms": target * 1e3}

    redistribution = None
    if world > 1:
        from ramtorch_b200._shard_plan import plan_for
        modes = sorted({str(bk.mode) for bk in plan_for(rpgs[0]).buckets.values()})
        redistribution = {"push": "fused peer stores from the optimizer kernel + barrier",
                          "gather": "NCCL all-gather"}.get(modes[0], modes[0]) if len(modes) == 1 else str(modes)

    # ---------------------------------------------------------------- ZeRO-2 reduce-scatter (N > 1)
    rs_ms = None
    if world > 1 and not grad_sync:
        from ramtorch_b200.zero2 import reduce_gradients_now, setup_grad_sharding_hooks
        for grp_list in rpgs[0].values():
            for grp in grp_list:
                for p in grp["params"]:
                    p.requires_grad_(True)
        setup_grad_sharding_hooks(rpgs[0], rank)   # flat gradient buffer, p.grad become views of it
        for _ in range(2):
            reduce_gradients_now(rpgs[0])
        torch.cuda.synchronize(); dist.barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(5):
            reduce_gradients_now(rpgs[0])
        r1.record(); torch.cuda.synchronize()
        t = torch.tensor([r0.elapsed_time(r1) / 5], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rs_ms = t.item()

    # ---------------------------------------------------------------- end to end from host memory
    e2e = None
    if not args.no_e2e and wl == "c2":
        n = args.elems
        for opt in steppers:
            for p in opt.state:
                p.grad = None
        steppers.clear(); rpgs.clear()
        del opt
        torch.cuda.empty_cache()
        n_host = n
        budget = host_mem_available_bytes() // max(world, 1)
        while n_host * 12 * 1.3 > budget and n_host > (1 << 24):
            n_host //= 2
        hp_, hg = (torch.empty(n_host, dtype=torch.bfloat16, pin_memory=True) for _ in range(2))
        # storage_device="cpu" (the reference default): moments in pinned host memory
        hopt = AdamW([hp_], dtype=torch.float32, storage_device="cpu", seed=0, **HP)
        hst = hopt.state[hp_]
        dp, dg, dm, dv = synth_on_device(n_host, device, seed=100 + rank)
        for h, d in ((hp_, dp), (hg, dg), (hst["ema"], dm), (hst["ema_squared"], dv)):
            h.copy_(d)
        hst["step"] = START_STEP
        del dp, dg, dm, dv
        torch.cuda.empty_cache()
        hp_.grad = hg
        hopt.step()   # warm-up: creates the pipeline streams and the staging ring
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s0 = N.stats()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            hopt.step()              # returns when the results are back in host memory
            _ = float(hp_[0])        # host read of the step's result
        e1.record()
        torch.cuda.synchronize()
        s1 = N.stats()
        e2e_ms = e0.elapsed_time(e1) / args.e2e_steps
        if world > 1:
            t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = t.item()
        h2d = (s1["h2d_bytes"] - s0["h2d_bytes"]) // args.e2e_steps
        d2h = (s1["d2h_bytes"] - s0["d2h_bytes"]) // args.e2e_steps
        e2e = {"value": n_host * world / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_ms, "elements_per_gpu": n_host,
               "h2d_gbs": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs": d2h / (e2e_ms * 1e-3) / 1e9,
               "steps": args.e2e_steps, "chunk_elems": hopt.offload_chunk_elems,
               "ring_depth": hopt.offload_ring_depth}
        if rank == 0:
            del hopt, hst, hp_, hg
            e2e["link_ceiling"] = link_ceiling(device)
            e2e["frac_of_measured_bidirectional_link"] = ((e2e["h2d_gbs"] + e2e["d2h_gbs"]) /
                                                          (2 * e2e["link_ceiling"]["both_each_gbs"]))

    base = None
    if rank == 0 and world == 1 and not args.no_cpu and wl == "c2":
        base = cpu_baseline()

    if rank == 0:
        label = WORKLOADS[wl]
        if world > 1:
            label += "; ZeRO-1 all-gather of the updated parameters inside the step"
        l2 = ("rotating over 12 buffer sets of 128 MiB (1.5 GiB > L2)" if wl == "c1" else
              "per-GPU inputs far exceed L2; no flush needed")
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak" if wl in ("c2", "bf16", "c1") else "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": label, "elements_per_step": total_elems, "l2": l2,
                           "math": "fast (approx sqrt/rcp in p')" if args.fast_math else "exact (IEEE sqrt/div)",
                           "draws": "independent Philox blocks" if args.independent_draws else "one Philox block shared by p, m, v",
                           "parallelism": f"zero1x{world}" if world > 1 else "single"},
                "roofline": roofline, "e2e": e2e, "cpu_baseline": base, "gpu_launches": int(launches),
                "clocks": clocks, "t_update_ms": upd_ms, "t_all_gather_ms": ag_ms if world > 1 else 0.0,
                "t_reduce_scatter_ms": rs_ms, "t_grad_sync_inside_update_ms": sync_ms,
                "zero1_redistribution": redistribution,
                "zero2_reduction": (None if world == 1 else
                                    "inside t_update: fused peer loads in the optimizer kernel" if args.fused_grad_pull else
                                    "inside t_update: NCCL reduce-scatter before the kernel" if grad_sync else
                                    "outside the timed step (t_reduce_scatter_ms measured separately)"),
                "host_ms_per_step": host_ms}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
