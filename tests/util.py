"""Shared helpers for the tests: golden loading, bf16 bit views, seeded inputs."""
import json
import os

import numpy as np
import torch

import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CODE = {"bf16": oracle.BF16, "f32": oracle.F32, "f16": oracle.F16}
TORCH_DT = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}
NP_DT = {"bf16": np.uint16, "f32": np.float32, "f16": np.float16}


def load_golden(name):
    d = np.load(os.path.join(GOLDEN, name))
    out = {k: d[k] for k in d.files}
    if "meta" in out:
        out["meta"] = json.loads(str(out["meta"]))
    return out


def step_cases():
    return sorted(f for f in os.listdir(GOLDEN) if f.startswith("step_") and f.endswith(".npz"))


def to_torch(arr: np.ndarray, kind: str, device="cpu") -> torch.Tensor:
    """numpy storage (bf16 as uint16 bits) -> torch tensor of dtype `kind`."""
    if kind == "bf16":
        t = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    else:
        t = torch.from_numpy(arr.copy())
    return t.to(device)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).ravel().copy()
    return t.numpy().ravel().copy()


def bits_equal(a: np.ndarray, b: np.ndarray) -> int:
    """Number of elements whose bit patterns differ."""
    ia = a.view(np.uint16 if a.itemsize == 2 else np.uint32)
    ib = b.view(np.uint16 if b.itemsize == 2 else np.uint32)
    return int((ia != ib).sum())


def synth(n, kind_p, kind_g, kind_s, seed, warm=True):
    """Seeded inputs with the value distributions of the benchmark configurations:
    p ~ N(0, 0.02), g ~ N(0, 1e-3), m ~ N(0, 1e-3), v = |N(0, 1e-6)|."""
    rng = np.random.default_rng(seed)

    def cast(x, kind):
        if kind == "bf16":
            return oracle.f32_to_bf16_bits_rn(x.astype(np.float32))
        return x.astype(NP_DT[kind])

    p = cast(rng.normal(0, 0.02, n), kind_p)
    g = cast(rng.normal(0, 1e-3, n), kind_g)
    if warm:
        m = cast(rng.normal(0, 1e-3, n), kind_s)
        v = cast(np.abs(rng.normal(0, 1e-6, n)), kind_s)
    else:
        m = cast(np.zeros(n), kind_s)
        v = cast(np.zeros(n), kind_s)
    return p, g, m, v
