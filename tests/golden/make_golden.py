"""Generate the golden fixtures in this directory by EXECUTING the reference on the CPU.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/RamTorch

Nothing of the reference is copied: ``ramtorch/stochastic_optimizers/adamw.py`` and
``ramtorch/zero1.py`` are loaded by file path and run unmodified.  Two host shims make the
optimizer runnable without a GPU (``step`` calls ``torch.cuda.current_device()`` and
``torch.cuda.synchronize()`` unconditionally, adamw.py:154/228/232), and the module-level name
``copy_stochastic_`` is wrapped so the fp32 values entering the rounding and the 16-bit draws of
``torch.randint`` can be recorded (adamw.py resolves the name at call time, :206-218).

Outputs (small, committed):
  sr_edge.npz, sr_random.npz     copy_stochastic_ : (fp32 bits, r16) -> bf16 bits
  step_<case>.npz                AdamW.step       : inputs, hyper-parameters, fp32 pre-rounding
                                 values, the draws used, and the tensors after the step
  zero1_ownership.json           create_zero_param_groups ownership maps
  MANIFEST.json                  torch version / CPU capability that produced them
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    torch.cuda.current_device = lambda: torch.device("cpu")
    torch.cuda.synchronize = lambda *a, **k: None
    mods = {}
    for name, rel in (("ref_adamw", "ramtorch/stochastic_optimizers/adamw.py"),
                      ("ref_zero1", "ramtorch/zero1.py")):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, rel))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods["ref_adamw"], mods["ref_zero1"]


class Recorder:
    """Wraps the reference's copy_stochastic_: records (seed, fp32 source, draws, target after)."""

    def __init__(self, ref, inject=None):
        self.ref, self.orig, self.calls, self.inject = ref, ref.copy_stochastic_, [], inject

    def __enter__(self):
        self.ref.copy_stochastic_ = self
        return self

    def __exit__(self, *exc):
        self.ref.copy_stochastic_ = self.orig

    def __call__(self, target, source, seed=0):
        real = torch.randint
        box = {}

        def randint(*a, **k):
            r = real(*a, **k)
            if self.inject is not None:
                r = self.inject.to(r.dtype).reshape(r.shape).clone()
            box["r"] = r.clone()
            return r

        torch.randint = randint
        try:
            self.orig(target, source, seed)
        finally:
            torch.randint = real
        self.calls.append((seed, source.detach().clone(), box["r"], target.detach().clone()))


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as numpy (bf16 -> uint16 bit patterns)."""
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy().ravel()
    return t.numpy().copy().ravel()


def gen_sr(ref):
    edge = np.array([0x00000000, 0x80000000, 0x00000001, 0x0000FFFF, 0x00010000, 0x007FFFFF,
                     0x00800000, 0x3F800000, 0x3F80FFFF, 0x3F808000, 0x3F807FFF, 0xBF808000,
                     0x7F7FFFFF, 0xFF7FFFFF, 0x7F7F0000, 0x7F800000, 0xFF800000, 0x7FC00000,
                     0x7FFFFFFF, 0xFFFFFFFF, 0x7F800001, 0x3A83126F, 0xBA83126F, 0x33D6BF95],
                    dtype=np.uint32)
    draws = np.array([0, 1, 0x7FFF, 0x8000, 0xFFFF, 0x1234, 0xFEDC], dtype=np.int64)
    src = np.repeat(edge, len(draws))
    r = np.tile(draws, len(edge))
    source = torch.from_numpy(src.view(np.float32).copy())
    target = torch.zeros(source.shape, dtype=torch.bfloat16)
    with Recorder(ref, inject=torch.from_numpy(r)) as rec:
        rec(target, source, 1)
    np.savez_compressed(os.path.join(HERE, "sr_edge.npz"), source_bits=src,
                        r16=r.astype(np.uint16), target_bits=bits(target))

    g = torch.Generator().manual_seed(1234)
    mag = torch.randint(-30, 8, (8192,), generator=g).float()
    source = torch.randn(8192, generator=g) * torch.pow(2.0, mag)
    target = torch.zeros(8192, dtype=torch.bfloat16)
    with Recorder(ref) as rec:
        rec(target, source, 77)
    np.savez_compressed(os.path.join(HERE, "sr_random.npz"), source_bits=bits(source).view(np.uint32),
                        r16=rec.calls[0][2].numpy().astype(np.uint16), target_bits=bits(target))


STEP_CASES = {
    # name: (shape, p dtype, g dtype, state dtype, optimizer kwargs, steps run, first step number)
    "bf16_all_fresh": ((4099,), "bf16", "bf16", "bf16",
                       dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01), 1, 1),
    "bf16_all_step11": ((4099,), "bf16", "bf16", "bf16",
                        dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01), 11, 1),
    "bf16_p_f32_state_t100": ((5000,), "bf16", "bf16", "f32",
                              dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01), 1, 100),
    "f32_all": ((3, 1001), "f32", "f32", "f32",
                dict(lr=3e-3, betas=(0.8, 0.95), eps=1e-6, weight_decay=0.1), 3, 1),
    "f16_all": ((2048 + 7,), "f16", "f16", "f16",
                dict(lr=1e-3, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01), 2, 1),
    "bf16_p_f32_grad_no_decay": ((37, 111), "bf16", "f32", "bf16",
                                 dict(lr=2e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0), 4, 1),
    "bf16_centralized_2d": ((37, 111), "bf16", "bf16", "bf16",
                            dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                                 centralization=0.5), 2, 1),
    "bf16_centralized_1d": ((1000,), "bf16", "bf16", "f32",
                            dict(lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                                 centralization=1.0), 2, 1),
}
DT = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}


def gen_step(ref, name, spec, seed):
    shape, pd, gd, sd, kw, nsteps, first = spec
    g = torch.Generator().manual_seed(seed)
    p = (torch.randn(shape, generator=g) * 0.02).to(DT[pd])
    if gd != pd:
        p.requires_grad_(True)
        p.grad_dtype = None  # torch >= 2.10 otherwise insists that grad dtype == param dtype
    opt = ref.AdamW([p], dtype=DT[sd], storage_device=torch.device("cpu"), **kw)
    st = opt.state[p]
    if first != 1:  # config-2 style: preset moments and the step counter
        st["step"] = first - 1
        st["ema"].copy_(torch.randn(shape, generator=g) * 1e-3)
        st["ema_squared"].copy_((torch.randn(shape, generator=g) * 1e-6).abs())
    rec_out = None
    for k in range(nsteps):
        p.grad = (torch.randn(shape, generator=g) * 1e-3).to(DT[gd])
        before = dict(p=bits(p), g=bits(p.grad), m=bits(st["ema"]), v=bits(st["ema_squared"]))
        with Recorder(ref) as rec:
            opt.step()
        if k == nsteps - 1:
            out = dict(before)
            out.update({"in_" + k2: v for k2, v in before.items()})
            for k2 in ("p", "g", "m", "v"):
                out.pop(k2)
            calls = {c[0] - st["step"]: c for c in rec.calls}  # seed offset 42 / 69 / 420
            for tag, off in (("p", 42), ("m", 69), ("v", 420)):
                if off in calls:
                    out["f32_" + tag] = calls[off][1].numpy().ravel().copy()
                    out["r16_" + tag] = calls[off][2].numpy().astype(np.uint16).ravel()
            out["out_p"], out["out_m"], out["out_v"] = bits(p), bits(st["ema"]), bits(st["ema_squared"])
            out["step"] = np.array(st["step"])
            rec_out = out
    meta = dict(shape=list(shape), p_dtype=pd, g_dtype=gd, state_dtype=sd, step=int(st["step"]),
                **{k: (list(v) if isinstance(v, tuple) else v) for k, v in kw.items()})
    np.savez_compressed(os.path.join(HERE, f"step_{name}.npz"), meta=json.dumps(meta), **rec_out)


def gen_zero1(zero1):
    cases = []
    for sizes, world in (([3, 2], 2), ([9], 8), ([1], 4), ([0, 5], 3), ([17, 4, 1], 8), ([291], 8)):
        groups, k = [], 0
        for gi, n in enumerate(sizes):
            params = [torch.zeros(1) for _ in range(n)]
            for t in params:
                t.tag = k
                k += 1
            groups.append({"params": params, "lr": 0.1 * (gi + 1), "foo": f"g{gi}"})
        rpg = zero1.create_zero_param_groups(groups, world)
        own = {str(r): [[p.tag for p in grp["params"]] for grp in gl] for r, gl in rpg.items()}
        extra = {str(r): [{k2: v for k2, v in grp.items() if k2 != "params"} for grp in gl]
                 for r, gl in rpg.items()}
        cases.append(dict(group_sizes=sizes, world_size=world, ownership=own, extra_keys=extra))
    with open(os.path.join(HERE, "zero1_ownership.json"), "w") as f:
        json.dump(cases, f, indent=1)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/RamTorch")
    root = sys.argv[1]
    ref, zero1 = load_reference(root)
    gen_sr(ref)
    for i, (name, spec) in enumerate(STEP_CASES.items()):
        gen_step(ref, name, spec, 100 + i)
    gen_zero1(zero1)
    with open(os.path.join(HERE, "MANIFEST.json"), "w") as f:
        json.dump(dict(torch=torch.__version__, cpu_capability=torch.backends.cpu.get_cpu_capability(),
                       reference_version="0.2.1", generator="tests/golden/make_golden.py"), f, indent=1)


if __name__ == "__main__":
    main()
