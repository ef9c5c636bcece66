#!/usr/bin/env python
"""Benchmark of the SR-AdamW optimizer step (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload ("c2"): a 1,073,741,824-element bf16 parameter shard per GPU with fp32 moments,
gradients ~N(0,1e-3), step counter at 100 (the "pure memory-bound roofline case").  A step is one
``AdamW.step()`` over that shard; with N > 1 every rank owns one such shard of an N-times larger
flat parameter space (ZeRO-1) and the step ends with the redistribution of the updated parameters.

  value     params updated / s, inputs resident in HBM, CUDA-event timed, max over ranks
  e2e       same metric with parameters, gradients and moments in pinned HOST memory, streamed
            through the GPU by ``AdamW.step()`` (copies inside the timed region)
  roofline  algorithmic bytes (22 B/element) / kernel time against the measured HBM copy peak
  variants  (N = 1) the other configurations of the same path, each with a 20-step and a >= 1 s
            figure: all-bf16 shard (default / independent draws / reference order), config 1,
            config 3, config 5, config 4
  parity_check (N > 1) a small seeded ZeRO-1/2 loop in three modes, every rank's parameters compared
            bit for bit with the CPU checker before anything is timed
  cpu_baseline / --impl reference
            the CPU restatement of the reference step (oracle/, C + OpenMP, all host threads) on
            the full shard when host memory allows
"""
from __future__ import annotations

import argparse
import ctypes
import gc
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sr_adamw_params_per_s"
UNIT = "params/s"
ELEMS_PER_GPU = 1 << 30
HP = dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
START_STEP = 99                # the timed steps start at t = 100
# DRAM bytes per element of the fused kernel (bf16 p/g, fp32 moments) measured with ncu
# (dram__bytes_read.sum + dram__bytes_write.sum over one launch of 2^27 elements, see profiles/);
# traffic is proportional to the element count, so it is scaled to the launch timed here.
NCU_DRAM_BYTES_PER_ELEM = 21.6
FALLBACK_HBM_GBS = 6650.0
NVLINK_FALLBACK_GBS = 770.0    # peer-copy rate per direction per GPU when it cannot be measured here


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

    def window(self, t0, t1):
        """Median SM clock and the throttle reasons seen between two wall-clock times."""
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + self.err]}
        rows = [r for r in list(self.rows) if t0 <= r[0] <= t1] or list(self.rows)[-3:]
        sm = sorted(r[1] for r in rows)
        reasons = set()
        for _, _, rs in rows:
            for bit, name in self.REASONS.items():
                if rs & bit:
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_sm,
                "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self, t0=None, t1=None):
        out = self.window(t0, t1) if t0 is not None else None
        if self.ok:
            self.stop_flag = True
            self.thread.join(timeout=1.0)
        return out


def host_mem_available_bytes():
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) * 1024
    except Exception:
        pass
    return 0


# ---------------------------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------------------------
def cpu_baseline(steps=3, warmup=1, sample_elems=None):
    """The CPU restatement of the reference step on all host threads, on the full 2^30-element shard
    of the headline workload when host memory allows (23.6 GB of arrays), else on the largest
    power-of-two fraction that fits.  Same dtypes and distributions; inputs are synthesised block
    by block with numpy."""
    import numpy as np
    import oracle
    n = sample_elems or ELEMS_PER_GPU
    avail = host_mem_available_bytes()
    why = None
    while avail and n * 12 * 1.6 > avail and n > (1 << 24):
        n //= 2
        why = f"host MemAvailable {avail / 2**30:.0f} GiB"
    threads = oracle.use_all_cores()
    p = np.empty(n, np.uint16); g = np.empty(n, np.uint16)
    m = np.empty(n, np.float32); v = np.empty(n, np.float32)
    blk = 1 << 22
    local = threading.local()

    def fill(lo):
        # independent Gaussian blocks seeded by position, generated in parallel into per-thread
        # scratch (numpy releases the GIL); bf16 by round-to-nearest-even on the fp32 bit pattern
        if not hasattr(local, "z"):
            local.z = np.empty(blk, np.float32)
            local.u = np.empty(blk, np.uint32)
        rng = np.random.default_rng(lo + 1)
        hi = min(n, lo + blk)
        z, u = local.z[:hi - lo], local.u[:hi - lo]

        def to_bf16(scale, out):
            rng.standard_normal(out=z, dtype=np.float32)
            np.multiply(z, np.float32(scale), out=z)
            zb = z.view(np.uint32)
            np.right_shift(zb, 16, out=u); np.bitwise_and(u, 1, out=u); np.add(u, 0x7FFF, out=u)
            np.add(u, zb, out=u); np.right_shift(u, 16, out=u)
            out[...] = u

        to_bf16(0.02, p[lo:hi])
        to_bf16(1e-3, g[lo:hi])
        rng.standard_normal(out=m[lo:hi], dtype=np.float32)
        np.multiply(m[lo:hi], np.float32(1e-3), out=m[lo:hi])
        rng.standard_normal(out=v[lo:hi], dtype=np.float32)
        np.multiply(v[lo:hi], np.float32(1e-6), out=v[lo:hi])
        np.abs(v[lo:hi], out=v[lo:hi])

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=max(1, min(threads, 32))) as ex:
        list(ex.map(fill, range(0, n, blk)))
    times = []
    for k in range(warmup + steps):
        h = oracle.make_hyper(HP["lr"], HP["betas"], HP["eps"], HP["weight_decay"], START_STEP + 1 + k,
                              reference_order=True)     # the reference's own operation order
        t0 = time.perf_counter()
        oracle.adamw_sr(p, g, m, v, oracle.BF16, oracle.BF16, oracle.F32, h, seed=0, tensor_id=0)
        dt = time.perf_counter() - t0
        if k >= warmup:
            times.append(dt)
    mean = sum(times) / len(times)
    frac = "the full shard" if n == ELEMS_PER_GPU else f"1/{ELEMS_PER_GPU // n} of one shard ({why})"
    return {"value": n / mean, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{n} elements ({frac}), bf16 p/g + fp32 moments, {len(times)} steps of the "
                      f"C+OpenMP restatement in oracle/, {threads} threads",
            "ms_per_step": mean * 1e3, "elements": n}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_baseline(steps=max(1, min(args.steps, 5)), warmup=1)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOADS["c2"] + ", on host cores",
                       "elements_per_step": base["elements"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
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
          "in 256 MiB chunks per tensor",
}


def link_ceiling(device, nbytes=1 << 30, reps=4, world=1, mix=(1, 1)):
    """Pinned cudaMemcpyAsync rates of this box: each direction alone, both at once with equal
    bytes, and both at once with the workload's own byte ratio `mix` = (bytes in, bytes out) --
    the time of that last run is what a perfect pipeline of the streamed step would need, so its
    total rate (`mix_total_gbs`) is the ceiling the step is held against.  With world > 1 every
    rank measures at the same time (between barriers), which is what the ranks of a streamed step
    get: they share the host's memory and PCIe root complexes."""
    import torch
    import torch.distributed as dist
    h_in = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    h_out = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=device)
    d_out = torch.empty(nbytes, dtype=torch.uint8, device=device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def run(h2d, d2h, n, n_in=nbytes, n_out=nbytes):
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            if h2d:
                with torch.cuda.stream(s_in):
                    d_in[:n_in].copy_(h_in[:n_in], non_blocking=True)
            if d2h:
                with torch.cuda.stream(s_out):
                    h_out[:n_out].copy_(d_out[:n_out], non_blocking=True)
        torch.cuda.synchronize(device)
        dt = time.perf_counter() - t0
        return ((n_in if h2d else 0) + (n_out if d2h else 0)) * n / dt / 1e9

    run(True, True, 1)
    big = max(mix)
    n_in, n_out = (int(nbytes * mix[0] / big) // 256 * 256, int(nbytes * mix[1] / big) // 256 * 256)
    out = {"h2d_alone_gbs": run(True, False, reps), "d2h_alone_gbs": run(False, True, reps),
           "both_each_gbs": run(True, True, reps) / 2, "mix_total_gbs": run(True, True, reps, n_in, n_out),
           "mix": list(mix), "ranks_measuring_at_once": world}
    if world > 1:
        keys = ("h2d_alone_gbs", "d2h_alone_gbs", "both_each_gbs", "mix_total_gbs")
        t = torch.tensor([out[k] for k in keys], device=device, dtype=torch.float64)
        lo = t.clone(); dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        out["min_over_ranks"] = dict(zip(keys, lo.tolist()))
        out["sum_over_ranks"] = dict(zip(keys, t.tolist()))
    return out


def link_frac(h2d_gbs, d2h_gbs, ceiling, world):
    """Achieved host-link traffic (both directions) over what concurrent pinned copies with the same
    byte ratio reach in the same run (slowest rank when several measure at once)."""
    top = ceiling["min_over_ranks"]["mix_total_gbs"] if world > 1 else ceiling["mix_total_gbs"]
    return (h2d_gbs + d2h_gbs) / top, top


def nvlink_ceiling(device, rank, world, chunk_bytes=256 << 20, reps=8):
    """Peer-copy rate per direction per GPU, all ranks at once: rank r copies 256 MiB chunks into
    the receive buffer of rank r+1 (a ring, so every GPU sends to one peer and receives from one)
    with cudaMemcpyAsync between the same two barriers.  Returns GB/s leaving (= entering) one GPU,
    min over ranks.  (Copying to ALL peers at once through the copy engines was tried as the
    ceiling and rejected: at 4 ranks it reaches 375 GB/s per GPU while the optimizer kernel's own
    peer stores move 684 GB/s -- the copy engines, not the links, limit that pattern.)"""
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm
    recv = symm.empty(chunk_bytes, dtype=torch.uint8, device=device)
    handle = symm.rendezvous(recv, dist.group.WORLD)
    ptrs = [int(q) for q in handle.buffer_ptrs]
    src = torch.empty(chunk_bytes, dtype=torch.uint8, device=device)
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    rt.cudaMemcpyAsync.restype = ctypes.c_int
    stream = torch.cuda.Stream(device)
    peer = (rank + 1) % world

    def burst(n):
        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        for _ in range(n):
            rc = rt.cudaMemcpyAsync(ptrs[peer], src.data_ptr(), chunk_bytes, 4, stream.cuda_stream)   # 4 = cudaMemcpyDefault
            if rc != 0:
                raise RuntimeError(f"cudaMemcpyAsync to peer {peer} failed: {rc}")
        torch.cuda.synchronize(device)
        return chunk_bytes * n / (time.perf_counter() - t0) / 1e9

    burst(1)
    gbs = burst(reps)
    t = torch.tensor([gbs], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    dist.barrier()
    del recv, handle
    return {"gbs_per_direction_per_gpu": t.item(), "pattern": f"ring of {world} ranks, every rank to its right neighbour at once, "
            f"{chunk_bytes >> 20} MiB chunks, cudaMemcpyAsync, min over ranks"}


# ---------------------------------------------------------------------------------------------
# parity check of the multi-GPU path (N > 1), before anything is timed
# ---------------------------------------------------------------------------------------------
PARITY_SHAPES = [(257, 64), (64,), (1000, 33), (33,), (4096,), (8, 8, 8), (70001, 1), (5,), (129, 128)]
PARITY_HP = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
PARITY_STEPS = 5


def _parity_grad(step, rank, k, shape):
    """Multiples of 2^-14 with few significant bits: sums over up to 16 ranks are exact in bf16, so
    neither NCCL's summation order nor its precision can matter."""
    import torch
    g = torch.Generator().manual_seed(1000 * step + 10 * rank + k)
    return (torch.randint(-8, 9, shape, generator=g).float() * 2.0 ** -14).bfloat16()


def zero_parity_check(rank, world, device):
    """ZeRO-2 reduction + owner-only SR-AdamW + ZeRO-1 redistribution on this job's ranks, for the
    three ways the path can run (NCCL all-gather; fused peer push; fused peer push + fused gradient
    pull), 5 steps each.  Afterwards every rank's copy of every parameter is compared bit for bit
    with the CPU checker run on rank 0's host on the summed gradients (the reference's contract:
    owner's gradient = SUM over ranks, zero2.py:27-57; every rank ends with the owners' values,
    zero1.py:67-91).  The checker only checks: nothing here is timed."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from ramtorch_b200 import AdamW
    from ramtorch_b200._shard_plan import plan_for, release_plan
    from ramtorch_b200.zero1 import broadcast_zero_params, create_zero_param_groups
    from ramtorch_b200.zero2 import setup_grad_sharding_hooks
    modes = {"all-gather": ("0", "0"), "peer-push": ("1", "0"), "peer-push+grad-pull": ("1", "1")}
    saved = {k: os.environ.get(k) for k in ("RT_ZERO_FUSED_PUSH", "RT_ZERO2_FUSED_PULL")}
    report = {"ok": True, "world": world, "modes": [], "elements": 0, "steps": PARITY_STEPS, "mismatches": {}}
    init = torch.Generator().manual_seed(0)
    start = [(torch.randn(s, generator=init) * 0.02).bfloat16() for s in PARITY_SHAPES]
    try:
        for mode, (push, pull) in modes.items():
            os.environ["RT_ZERO_FUSED_PUSH"], os.environ["RT_ZERO2_FUSED_PULL"] = push, pull
            params = [torch.nn.Parameter(t.clone().to(device)) for t in start]
            groups = [{"params": [p for p in params if p.dim() == 1], "weight_decay": 0.0},
                      {"params": [p for p in params if p.dim() > 1]}]
            rpg = create_zero_param_groups(groups, world)
            setup_grad_sharding_hooks(rpg, rank)
            opt = AdamW(rpg[rank], dtype=torch.bfloat16, storage_device=device, seed=21, **PARITY_HP)
            for step in range(PARITY_STEPS):
                grads = [_parity_grad(step, rank, k, p.shape).to(device) for k, p in enumerate(params)]
                sum((p * g).sum() for p, g in zip(params, grads)).backward()
                opt.step()
                broadcast_zero_params(rpg)
                for p in params:
                    p.grad = None
            torch.cuda.synchronize()
            used = sorted({str(b.mode) for b in plan_for(rpg).buckets.values()})
            flat = torch.cat([p.detach().reshape(-1) for p in params])     # bf16: a type NCCL can move
            everyone = [torch.empty_like(flat) for _ in range(world)] if rank == 0 else None
            dist.gather(flat, everyone, dst=0)
            bad = 0
            if rank == 0:
                bad = _parity_against_checker(start, groups, params, everyone, world, np)
                report["elements"] += int(flat.numel()) * world
            verdict = torch.tensor([bad], device=device, dtype=torch.int64)
            dist.broadcast(verdict, src=0)
            report["modes"].append({"mode": mode, "redistribution": used, "mismatching_elements": int(verdict.item())})
            if int(verdict.item()):
                report["ok"] = False
                report["mismatches"][mode] = int(verdict.item())
            release_plan(rpg)
            del opt, rpg, params, groups
            gc.collect()
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    return report


def _parity_against_checker(start, groups, params, everyone, world, np):
    """Rank 0: replay the loop with the CPU checker and count the elements, over all ranks' copies,
    whose bits differ."""
    import oracle
    import torch
    ids = {}
    next_id = 0
    for gi, grp in enumerate(groups):               # global parameter ids as create_zero_param_groups numbers them
        for p in grp["params"]:
            ids[id(p)] = (next_id, gi)
            next_id += 1
    want = []
    for k, p in enumerate(params):
        tid, gi = ids[id(p)]
        n = p.numel()
        pb = start[k].reshape(-1).view(torch.int16).numpy().view(np.uint16).copy()
        m = np.zeros(n, np.uint16); v = np.zeros(n, np.uint16)
        for step in range(PARITY_STEPS):
            total = torch.zeros(p.shape, dtype=torch.float32)
            for r in range(world):                       # rank order, fp32: exact for these gradients
                total += _parity_grad(step, r, k, p.shape).float()
            gb = total.bfloat16().reshape(-1).view(torch.int16).numpy().view(np.uint16).copy()
            h = oracle.make_hyper(PARITY_HP["lr"], PARITY_HP["betas"], PARITY_HP["eps"],
                                  0.0 if gi == 0 else PARITY_HP["weight_decay"], step + 1, shared_draws=True)
            oracle.adamw_sr(pb, gb, m, v, oracle.BF16, oracle.BF16, oracle.BF16, h, seed=21, tensor_id=tid)
        want.append(pb)
    want = np.concatenate(want)
    bad = 0
    for copy in everyone:
        got = copy.cpu().view(torch.int16).numpy().view(np.uint16)
        bad += int((got != want).sum())
    return bad


# ---------------------------------------------------------------------------------------------
# resident step
# ---------------------------------------------------------------------------------------------
BYTES_PER_ELEM = {"c2": 22}       # every other workload has bf16 moments: 14


def measure_resident(wl, args, device, rank, world, *, steps, warmup, independent=False, reference_order=False,
                     elems=ELEMS_PER_GPU, list_count=64, grad_sync=False, fused_pull=False, sustain_s=0.0,
                     want_update_only=False, balance="count", measure_reduce_scatter=False):
    """Time `steps` optimizer steps of one workload with everything resident in HBM.  Returns a dict;
    frees what it allocated."""
    import torch
    import torch.distributed as dist
    from ramtorch_b200 import AdamW, _native as N
    from ramtorch_b200._shard_plan import plan_for, release_plan
    from ramtorch_b200.zero1 import broadcast_zero_params, create_zero_param_groups
    local = device.index
    state_dtype = torch.float32 if wl == "c2" else torch.bfloat16
    bytes_per_elem = BYTES_PER_ELEM.get(wl, 14)
    start_step = 10 if wl == "c1" else START_STEP

    # Every workload is a list of parameters in ONE group handed to create_zero_param_groups, so the
    # reference's round-robin (parameter k -> rank k % world) decides ownership.  A rank holds all
    # parameters (they are replicated) but gradients and moments only for the ones it owns.
    steppers, rpgs = [], []

    def make_set(shapes, seed):
        params = [torch.empty(s, dtype=torch.bfloat16, device=device).normal_(0, 0.02) for s in shapes]
        rpg = create_zero_param_groups([{"params": params}], world, balance=balance)
        owned = rpg[rank][0]["params"]
        opt = AdamW(rpg[rank], dtype=state_dtype, storage_device=device, seed=seed, sync=False,
                    reference_order=reference_order, shared_draws=not independent, **HP)
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
        owned_elems = make_set([(elems,)] * world, 0)     # one shard per rank: rank r owns tensor r
    elif wl == "c1":
        owned_elems = [make_set([(1 << 24,)] * world, k) for k in range(12)][0]
    elif wl == "c3":
        owned_elems = make_set(llama_shapes(), 0)
    elif wl == "list":
        owned_elems = make_set([(elems,)] * list_count, 0)
    else:
        owned_elems = make_set(ragged_shapes(), 0)
    torch.cuda.synchronize()

    grad_sync = world > 1 and (grad_sync or fused_pull)
    if grad_sync:
        from ramtorch_b200.zero2 import reduce_gradients_now, setup_grad_sharding_hooks
        saved_pull = os.environ.get("RT_ZERO2_FUSED_PULL")
        if fused_pull:
            os.environ["RT_ZERO2_FUSED_PULL"] = "1"
        for rpg in rpgs:
            for grp_list in rpg.values():
                for grp in grp_list:
                    for p in grp["params"]:
                        p.requires_grad_(True)
            setup_grad_sharding_hooks(rpg, rank)   # flat gradient buffer; every p.grad becomes a view of it
            for bk in plan_for(rpg).buckets.values():
                bk.gflat.normal_(0, 1e-3)          # every rank holds a gradient for every parameter
        if fused_pull:
            if saved_pull is None:
                os.environ.pop("RT_ZERO2_FUSED_PULL", None)
            else:
                os.environ["RT_ZERO2_FUSED_PULL"] = saved_pull

    rs_events = []

    def one_step(k):
        if grad_sync:
            reduce_gradients_now(rpgs[k % len(rpgs)])
            if len(rs_events) < 4096:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                rs_events.append(e)
        steppers[k % len(steppers)].step()

    def redistribute(k):
        if world > 1:
            broadcast_zero_params(rpgs[k % len(rpgs)])

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for k in range(max(warmup, len(steppers))):
        one_step(k); redistribute(k)
    fence()
    sampler = ClockSampler(local) if rank == 0 else None
    rs_events.clear()
    # Per-step events split a step into update and redistribution.  On one GPU there is nothing to
    # split, and for steps of tens of microseconds the two event records per step would themselves
    # be a tenth of what is measured: such loops are bracketed by one pair of events only.
    per_step = world > 1 or steps <= 64
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps + 1 if per_step else 2)]
    launches0 = N.stats()["kernel_launches"]
    t_wall0 = time.time()
    ev[0].record()
    if per_step:
        for k in range(steps):
            one_step(k)
            ev[2 * k + 1].record()
            redistribute(k)
            ev[2 * k + 2].record()
    else:
        for k in range(steps):
            steppers[k % len(steppers)].step()
        ev[1].record()
    host_ms = (time.time() - t_wall0) * 1e3 / steps
    fence()
    t_wall1 = time.time()
    launches = N.stats()["kernel_launches"] - launches0
    total_ms = ev[0].elapsed_time(ev[-1])
    if per_step:
        upd_ms = sum(ev[2 * k].elapsed_time(ev[2 * k + 1]) for k in range(steps)) / steps
        ag_ms = sum(ev[2 * k + 1].elapsed_time(ev[2 * k + 2]) for k in range(steps)) / steps
    else:
        upd_ms, ag_ms = total_ms / steps, 0.0
    clocks = sampler.window(t_wall0, t_wall1) if sampler else None
    sync_ms = None
    if grad_sync and len(rs_events) == steps:
        # part of t_update spent in the gradient reduction (NCCL reduce-scatter, or the barrier of the fused path)
        sync_ms = sum(ev[2 * k].elapsed_time(rs_events[k]) for k in range(steps)) / steps

    # the same loop for at least sustain_s seconds: the board reaches its power cap within ~0.5 s of
    # back-to-back launches, so the short figure above is a burst and this one is what a long job sees
    sustained = None
    if sustain_s > 0:
        n_sus = int(min(max(steps, math.ceil(sustain_s * 1e3 / max(total_ms / steps, 1e-3))), 100000))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tw0 = time.time()
        s0.record()
        for k in range(n_sus):
            one_step(k); redistribute(k)
        s1.record()
        fence()
        tw1 = time.time()
        sustained = {"steps": n_sus, "ms_per_step": s0.elapsed_time(s1) / n_sus, "seconds": tw1 - tw0,
                     "clocks": sampler.window(tw0, tw1) if sampler else None}

    # update alone (N > 1, fused redistribution): the same steps with the peer stores switched off
    upd_only_ms = None
    if want_update_only and world > 1:
        lib = N.lib()
        pushing = [pl for opt in steppers for pl in opt._plans.values() if pl.push_bucket is not None]
        for pl in pushing:
            N.check(lib.rt_plan_set_push(pl.handle, None), "rt_plan_set_push")
        fence()
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_u = max(3, min(steps, 10))
        u0.record()
        for k in range(n_u):
            steppers[k % len(steppers)].step()
        u1.record()
        fence()
        upd_only_ms = u0.elapsed_time(u1) / n_u
        # these steps changed the owners' parameters without redistributing them; nothing below reads
        # the replicas again, and the plans (whose push tables were cleared) are dropped with the set

    elems_t = torch.tensor([float(owned_elems)], device=device, dtype=torch.float64)
    if world > 1:
        vals = [total_ms, upd_ms, ag_ms, upd_only_ms or 0.0, sustained["ms_per_step"] if sustained else 0.0]
        t = torch.tensor(vals, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, upd_ms, ag_ms, uo, su = t.tolist()
        upd_only_ms = uo if upd_only_ms is not None else None
        if sustained:
            sustained["ms_per_step"] = su
        dist.all_reduce(elems_t, op=dist.ReduceOp.SUM)
    total_elems = int(elems_t.item())
    ms_per_step = total_ms / steps
    modes = None
    if world > 1:
        modes = sorted({str(bk.mode) for bk in plan_for(rpgs[0]).buckets.values()})
    out = dict(workload=wl, total_elems=total_elems, per_rank_elems=total_elems / world, ms_per_step=ms_per_step,
               value=total_elems / (ms_per_step * 1e-3), upd_ms=upd_ms, ag_ms=ag_ms, host_ms=host_ms,
               launches=int(launches), clocks=clocks, sync_ms=sync_ms, sustained=sustained, modes=modes,
               upd_only_ms=upd_only_ms, bytes_per_elem=bytes_per_elem, grad_sync=grad_sync, rs_ms=None)
    if sustained:
        sustained["value"] = total_elems / (sustained["ms_per_step"] * 1e-3)

    # ZeRO-2 reduce-scatter measured on its own (N > 1, when it is not already inside the step)
    if world > 1 and not grad_sync and measure_reduce_scatter and not want_update_only:
        from ramtorch_b200.zero2 import reduce_gradients_now, setup_grad_sharding_hooks
        for grp_list in rpgs[0].values():
            for grp in grp_list:
                for p in grp["params"]:
                    p.requires_grad_(True)
        setup_grad_sharding_hooks(rpgs[0], rank)   # flat gradient buffer, p.grad become views of it
        for _ in range(2):
            reduce_gradients_now(rpgs[0])
        fence()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(5):
            reduce_gradients_now(rpgs[0])
        r1.record(); torch.cuda.synchronize()
        t = torch.tensor([r0.elapsed_time(r1) / 5], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["rs_ms"] = t.item()

    if sampler:
        sampler.stop()
    for opt in steppers:
        for p in list(opt.state):
            p.grad = None
        for pl in list(opt._plans.values()):
            pl.close()
        opt._plans.clear()
        opt._fast = None
    for rpg in rpgs:
        release_plan(rpg)
    steppers.clear(); rpgs.clear()
    opt = rpg = None
    gc.collect()
    torch.cuda.empty_cache()
    return out


def hbm_roofline(res, peak, which):
    achieved = res["bytes_per_elem"] * res["per_rank_elems"] / (res["upd_ms"] * 1e-3) / 1e9
    traffic = NCU_DRAM_BYTES_PER_ELEM * res["per_rank_elems"] if (res["workload"] == "c2" and NCU_DRAM_BYTES_PER_ELEM) else None
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_source": which, "traffic": traffic, "algorithmic_bytes": res["bytes_per_elem"] * res["per_rank_elems"],
            "kernel_ms": res["upd_ms"], "frac_of_nominal_8TBs": achieved / 8000.0}


def variant_entry(name, res, peak):
    """One row of the `variants` block: the 20-step (burst) figure and the >= 1 s (sustained) one."""
    bpe, n = res["bytes_per_elem"], res["per_rank_elems"]
    row = {"name": name, "workload": WORKLOADS[res["workload"]], "elements": res["total_elems"],
           "bytes_per_element": bpe, "ms": res["ms_per_step"], "kernel_ms": res["upd_ms"],
           "params_per_s": res["value"], "gbs": bpe * n / (res["ms_per_step"] * 1e-3) / 1e9,
           "frac": bpe * n / (res["ms_per_step"] * 1e-3) / 1e9 / peak, "clocks": res["clocks"],
           "host_ms_per_step": res["host_ms"], "gpu_launches": res["launches"]}
    s = res["sustained"]
    if s:
        row["sustained"] = {"steps": s["steps"], "seconds": s["seconds"], "ms": s["ms_per_step"],
                            "gbs": bpe * n / (s["ms_per_step"] * 1e-3) / 1e9,
                            "frac": bpe * n / (s["ms_per_step"] * 1e-3) / 1e9 / peak, "clocks": s["clocks"]}
    return row


# ---------------------------------------------------------------------------------------------
# host-offloaded steps
# ---------------------------------------------------------------------------------------------
def measure_c4(args, device, rank, world, steps=3, chunk_elems=1 << 27, ring_depth=2, grads_in_hbm=False):
    """Config 4: parameters, moments (and gradients) in pinned CPU RAM, streamed through the GPU."""
    import torch
    import torch.distributed as dist
    from ramtorch_b200 import AdamW, _native as N
    n_tensors, n_each = 60, 1 << 27
    mine = [k for k in range(n_tensors) if k % world == rank]
    budget = host_mem_available_bytes() // max(world, 1)
    while len(mine) * n_each * 8 * 1.2 > budget and len(mine) > 1:
        mine = mine[:-1]
    params = [torch.empty(n_each, dtype=torch.bfloat16, pin_memory=True) for _ in mine]
    opt = AdamW(params, dtype=torch.bfloat16, storage_device="cpu", seed=0, offload_chunk_elems=chunk_elems,
                offload_ring_depth=ring_depth, reference_order=args.reference_order,
                shared_draws=not args.independent_draws, **HP)
    scratch = torch.empty(n_each, dtype=torch.float32, device=device)
    for p in params:
        st = opt.state[p]
        p.copy_(scratch.normal_(0, 0.02)); st["ema"].copy_(scratch.normal_(0, 1e-3))
        st["ema_squared"].copy_(scratch.normal_(0, 1e-6).abs_())
        st["step"] = START_STEP
        if grads_in_hbm:
            p.rt_device_grad = torch.empty(n_each, dtype=torch.bfloat16, device=device).normal_(0, 1e-3)
        else:
            p.grad = torch.empty(n_each, dtype=torch.bfloat16, pin_memory=True)
            p.grad.copy_(scratch.normal_(0, 1e-3))
    del scratch
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
    clocks = sampler.stop(t0, t1) if sampler else None
    for p in params:
        p.grad = None
        p.rt_device_grad = None
    del opt, params
    gc.collect()
    torch.cuda.empty_cache()
    h2d = (s1["h2d_bytes"] - s0["h2d_bytes"]) / steps
    d2h = (s1["d2h_bytes"] - s0["d2h_bytes"]) / steps
    ceiling = link_ceiling(device, world=world, mix=(int(h2d), int(d2h)))
    total = int(elems.item())
    link = {"h2d_gbs_per_gpu": h2d / (ms * 1e-3) / 1e9, "d2h_gbs_per_gpu": d2h / (ms * 1e-3) / 1e9,
            "ceiling": ceiling, "pcie_gen5_x16_nominal_gbs_per_direction": 63.0}
    link["frac_of_measured_bidirectional"], link["ceiling_total_gbs"] = link_frac(
        link["h2d_gbs_per_gpu"], link["d2h_gbs_per_gpu"], ceiling, world)
    return dict(ms=ms, total=total, steps=steps, h2d=h2d, d2h=d2h, link=link, clocks=clocks,
                launches=int(s1["kernel_launches"] - s0["kernel_launches"]), chunk_elems=chunk_elems,
                ring_depth=ring_depth, grads_in_hbm=grads_in_hbm)


def run_c4(args, device, rank, world):
    import torch.distributed as dist
    r = measure_c4(args, device, rank, world, steps=max(1, min(args.steps, 3)), grads_in_hbm=args.grads_in_hbm)
    if rank == 0:
        value = r["total"] / (r["ms"] * 1e-3)
        link = r["link"]
        e2e = {"value": value, "unit": UNIT, "h2d_bytes_per_step": int(r["h2d"]), "d2h_bytes_per_step": int(r["d2h"]),
               "ms_per_step": r["ms"]}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": r["steps"], "warmup": 1,
                "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": WORKLOADS["c4"] + ("; variant: gradients kept in HBM" if args.grads_in_hbm else ""),
                           "elements_per_step": r["total"], "chunk_elems": r["chunk_elems"], "ring_depth": r["ring_depth"],
                           "l2": "streamed chunks of 1 GiB per slot far exceed L2",
                           "parallelism": f"tensors round-robin over {world} ranks" if world > 1 else "single"},
                "roofline": {"bound": "host link", "achieved": link["h2d_gbs_per_gpu"] + link["d2h_gbs_per_gpu"],
                             "peak": link["ceiling_total_gbs"], "unit": "GB/s",
                             "frac": link["frac_of_measured_bidirectional"], "traffic": None,
                             "peak_source": "pinned cudaMemcpyAsync in both directions at once with this step's byte ratio, "
                                            "same run, every rank at once"},
                "link": link, "e2e": e2e, "cpu_baseline": None, "gpu_launches": r["launches"], "clocks": r["clocks"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_e2e(args, device, rank, world):
    """The headline workload end to end through the public API from pinned HOST memory: every step
    copies 12 B/element in and 10 B/element out inside the timed region."""
    import torch
    import torch.distributed as dist
    from ramtorch_b200 import AdamW, _native as N
    n_host = args.elems
    budget = host_mem_available_bytes() // max(world, 1)
    while n_host * 12 * 1.3 > budget and n_host > (1 << 24):
        n_host //= 2
    hp_, hg = (torch.empty(n_host, dtype=torch.bfloat16, pin_memory=True) for _ in range(2))
    # storage_device="cpu" (the reference default): moments in pinned host memory
    hopt = AdamW([hp_], dtype=torch.float32, storage_device="cpu", seed=0, **HP)
    hst = hopt.state[hp_]
    blk = 1 << 27
    scratch = torch.empty(min(blk, n_host), dtype=torch.float32, device=device)
    for lo in range(0, n_host, blk):
        hi = min(n_host, lo + blk)
        s = scratch[:hi - lo]
        hp_[lo:hi].copy_(s.normal_(0, 0.02)); hg[lo:hi].copy_(s.normal_(0, 1e-3))
        hst["ema"][lo:hi].copy_(s.normal_(0, 1e-3)); hst["ema_squared"][lo:hi].copy_(s.normal_(0, 1e-6).abs_())
    hst["step"] = START_STEP
    del scratch
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
    hp_.grad = None
    del hopt, hst, hp_, hg
    gc.collect()
    torch.cuda.empty_cache()
    # the ceiling every rank gets while all of them copy at once (they share the host)
    ceil = link_ceiling(device, world=world, mix=(int(h2d), int(d2h)))
    e2e["link_ceiling"] = ceil
    e2e["frac_of_measured_bidirectional_link"], e2e["link_ceiling_total_gbs"] = link_frac(e2e["h2d_gbs"], e2e["d2h_gbs"], ceil, world)
    return e2e


# ---------------------------------------------------------------------------------------------
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
    ap.add_argument("--reference-order", action="store_true",
                    help="denominator and quotient in the reference's operation order (two IEEE divisions per element)")
    ap.add_argument("--independent-draws", action="store_true",
                    help="three independent Philox blocks per eight elements instead of one shared block "
                         "(AdamW(shared_draws=False)); only matters for bf16 moments")
    ap.add_argument("--grads-in-hbm", action="store_true",
                    help="c4 only: gradients of the CPU parameters stay in HBM (p.rt_device_grad)")
    ap.add_argument("--with-grad-sync", action="store_true",
                    help="N > 1: include the ZeRO-2 gradient reduction in every timed step")
    ap.add_argument("--fused-grad-pull", action="store_true",
                    help="N > 1: no reduce-scatter; the optimizer kernel sums the ranks' gradients over NVLink")
    ap.add_argument("--balance", default="count", choices=["count", "bytes"],
                    help="ownership of whole tensors: the reference's round-robin by count, or greedy by bytes")
    ap.add_argument("--sustain", type=float, default=0.0, help="also time the loop for at least this many seconds")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-variants", action="store_true", help="N = 1, c2: skip the variants block")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the multi-GPU parity check")
    ap.add_argument("--no-c4-variant", action="store_true", help="skip config 4 in the variants block (64 GB pinned)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

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
    peak, which = measured_peak()

    if wl == "c4":
        return run_c4(args, device, rank, world)

    # ---------------------------------------------------------------- N > 1: parity first, then the link
    parity = None
    nvlink = None
    if world > 1:
        if not args.no_parity:
            parity = zero_parity_check(rank, world, device)
            if not parity["ok"]:
                if rank == 0:
                    print(json.dumps({"metric": METRIC, "error": "multi-GPU parity check failed", "parity_check": parity}),
                          flush=True)
                dist.destroy_process_group()
                raise SystemExit(3)
        try:
            nvlink = nvlink_ceiling(device, rank, world)
        except Exception as e:     # no peer mapping on this box: keep going with the recorded rate
            nvlink = {"gbs_per_direction_per_gpu": None, "error": repr(e)}

    # ---------------------------------------------------------------- resident step (value)
    fused = args.with_grad_sync or args.fused_grad_pull
    res = measure_resident(wl, args, device, rank, world, steps=args.steps, warmup=warmup,
                           independent=args.independent_draws, reference_order=args.reference_order,
                           elems=args.elems, list_count=args.list_count, grad_sync=args.with_grad_sync,
                           fused_pull=args.fused_grad_pull, sustain_s=args.sustain,
                           want_update_only=world > 1 and not fused, balance=args.balance)
    roofline = hbm_roofline(res, peak, which)
    per_rank = res["per_rank_elems"]
    bytes_per_elem = res["bytes_per_elem"]
    upd_ms = res["upd_ms"]
    if world > 1 and res["modes"] == ["push"]:
        # fused update + redistribution: the kernel also stores every updated bf16 parameter into the
        # other ranks' buffers, so its target time is the slower of the HBM time and the NVLink time
        # (bytes leaving this GPU / the peer-copy rate per direction measured above with every rank
        # copying to a neighbour at once)
        measured = nvlink and nvlink.get("gbs_per_direction_per_gpu")
        nvlink_peak = measured or NVLINK_FALLBACK_GBS
        # parameters pushed to the peers, plus (fused reduction) this rank's gradients read by the peers
        egress = 2.0 * per_rank * (world - 1) * (2 if args.fused_grad_pull else 1)
        t_hbm = bytes_per_elem * per_rank / (peak * 1e9)
        t_link = egress / (nvlink_peak * 1e9)
        target = max(t_hbm, t_link)
        link_bound = t_link > t_hbm
        roofline = {"bound": "nvlink" if link_bound else "hbm",
                    "achieved": egress / (upd_ms * 1e-3) / 1e9 if link_bound else roofline["achieved"],
                    "peak": nvlink_peak if link_bound else peak, "unit": "GB/s",
                    "frac": target / (upd_ms * 1e-3), "traffic": None, "kernel_ms": upd_ms,
                    "peak_source": (("peer copies around a ring of all ranks at once, measured in this run" if measured
                                     else "recorded peer-copy rate (not measurable in this run)") if link_bound else which),
                    "nvlink_egress_bytes": egress, "hbm_algorithmic_bytes": bytes_per_elem * per_rank,
                    "target_ms": target * 1e3}

    redistribution = None
    if world > 1:
        modes = res["modes"]
        redistribution = {"push": "fused peer stores from the optimizer kernel + barrier",
                          "gather": "NCCL all-gather"}.get(modes[0], modes[0]) if len(modes) == 1 else str(modes)

    # ZeRO-2 reduce-scatter on its own and the full ZeRO step (reduction + update + redistribution)
    rs = None
    full = None
    if world > 1 and wl in ("c2", "c3") and not fused:
        rs = measure_resident(wl, args, device, rank, world, steps=5, warmup=warmup, elems=args.elems,
                              measure_reduce_scatter=True, balance=args.balance)["rs_ms"]
        f1 = measure_resident(wl, args, device, rank, world, steps=max(5, args.steps // 2), warmup=warmup,
                              elems=args.elems, grad_sync=True, balance=args.balance)
        f2 = measure_resident(wl, args, device, rank, world, steps=max(5, args.steps // 2), warmup=warmup,
                              elems=args.elems, fused_pull=True, balance=args.balance)
        full = {"what": "gradient reduction + update + redistribution, every step, CUDA-event timed, max over ranks",
                "nccl_reduce_scatter_then_update_push_ms": f1["ms_per_step"],
                "of_which_reduce_scatter_ms": f1["sync_ms"],
                "fused_pull_update_push_ms": f2["ms_per_step"],
                "params_per_s_fused": f2["value"], "params_per_s_nccl": f1["value"]}

    # ---------------------------------------------------------------- end to end from host memory
    e2e = None
    if not args.no_e2e and wl == "c2":
        e2e = measure_e2e(args, device, rank, world)

    # ---------------------------------------------------------------- the other configurations (N = 1)
    variants = None
    if world == 1 and wl == "c2" and not args.no_variants and args.elems == ELEMS_PER_GPU:
        variants = []
        sus = max(args.sustain, 1.0)
        r = measure_resident("c2", args, device, rank, world, steps=args.steps, warmup=warmup, sustain_s=sus)
        variants.append(variant_entry("config 2 (headline workload)", r, peak))
        for name, kw in (("all bf16, default (shared draws, default order)", {}),
                         ("all bf16, independent draws", {"independent": True}),
                         ("all bf16, reference order", {"reference_order": True})):
            r = measure_resident("bf16", args, device, rank, world, steps=args.steps, warmup=warmup, sustain_s=sus, **kw)
            variants.append(variant_entry(name, r, peak))
        for w, steps in (("c1", 240), ("c3", args.steps), ("c5", args.steps)):
            r = measure_resident(w, args, device, rank, world, steps=steps, warmup=warmup, sustain_s=sus)
            variants.append(variant_entry("config " + w[1], r, peak))
        if not args.no_c4_variant and host_mem_available_bytes() > 110 * 2**30:
            try:
                c4 = measure_c4(args, device, rank, world, steps=2)
                variants.append({"name": "config 4 (host-offloaded, as specified: 256 MiB chunks)",
                                 "workload": WORKLOADS["c4"], "elements": c4["total"], "ms": c4["ms"],
                                 "params_per_s": c4["total"] / (c4["ms"] * 1e-3),
                                 "h2d_gbs": c4["link"]["h2d_gbs_per_gpu"], "d2h_gbs": c4["link"]["d2h_gbs_per_gpu"],
                                 "frac": c4["link"]["frac_of_measured_bidirectional"], "bound": "host link",
                                 "link_ceiling": c4["link"]["ceiling"], "clocks": c4["clocks"],
                                 "chunk_elems": c4["chunk_elems"], "ring_depth": c4["ring_depth"]})
            except Exception as e:
                variants.append({"name": "config 4", "error": repr(e)})
        else:
            variants.append({"name": "config 4", "skipped": "needs ~64 GB of pinned host memory plus headroom"})

    base = None
    if rank == 0 and world == 1 and not args.no_cpu and wl == "c2":
        base = cpu_baseline()

    if rank == 0:
        label = WORKLOADS[wl]
        if world > 1:
            label += "; ZeRO-1 redistribution of the updated parameters inside the step"
        l2 = ("rotating over 12 buffer sets of 128 MiB (1.5 GiB > L2)" if wl == "c1" else
              "per-GPU inputs far exceed L2; no flush needed")
        total_elems = res["total_elems"]
        line = {"metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                "scaling": "weak" if wl in ("c2", "bf16", "c1") else "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": label, "elements_per_step": total_elems, "l2": l2,
                           "math": ("reference order: sqrt(v)/bc + eps, p + (a*m)/den" if args.reference_order else
                                    "default order: fma(sqrt(v), 1/bc, eps), fma(a*m, 1/den, p)") + "; every operation IEEE-rounded",
                           "draws": "independent Philox blocks" if args.independent_draws else "one Philox block shared by p, m, v",
                           "ownership": args.balance,
                           "parallelism": f"zero1x{world}" if world > 1 else "single"},
                "roofline": roofline, "e2e": e2e, "cpu_baseline": base, "gpu_launches": res["launches"],
                "clocks": res["clocks"], "t_update_ms": upd_ms, "t_all_gather_ms": res["ag_ms"] if world > 1 else 0.0,
                "t_reduce_scatter_ms": rs, "t_grad_sync_inside_update_ms": res["sync_ms"],
                "zero1_redistribution": redistribution,
                "zero2_reduction": (None if world == 1 else
                                    "inside t_update: fused peer loads in the optimizer kernel" if args.fused_grad_pull else
                                    "inside t_update: NCCL reduce-scatter before the kernel" if res["grad_sync"] else
                                    "outside the timed step (t_reduce_scatter_ms measured separately)"),
                "host_ms_per_step": res["host_ms"]}
        if res["sustained"]:
            line["sustained"] = res["sustained"]
        if world > 1:
            line["parity_check"] = parity
            line["nvlink_ceiling"] = nvlink
            if full is not None:
                line["full_zero_step"] = full
            if res["upd_only_ms"] is not None:
                # the update without the redistribution (peer stores switched off): the part of the step
                # that can scale with N; the full step (value) also has to move (N-1)/N of all parameters
                # into every GPU
                line["t_update_only_ms"] = res["upd_only_ms"]
                line["update_only_params_per_s"] = total_elems / (res["upd_only_ms"] * 1e-3)
        if variants is not None:
            line["variants"] = variants
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
