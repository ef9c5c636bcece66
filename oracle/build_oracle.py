"""Compile the C checker into ``oracle/liboracle.so`` with gcc (TEST INFRASTRUCTURE).

``python -m oracle.build_oracle`` or ``build()``; rebuilds only when the source is newer.
The reference is pure Python, so there is nothing of it to compile: no ``oracle/_ref``.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sr_adamw_oracle.c")
OUT = os.path.join(HERE, "liboracle.so")
HDR = os.path.join(HERE, "..", "include", "rt_b200.h")


def build(force: bool = False) -> str:
    newest = max(os.path.getmtime(SRC), os.path.getmtime(HDR) if os.path.exists(HDR) else 0)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= newest:
        return OUT
    # -ffp-contract=off: only the explicit fmaf() calls may fuse; -fno-fast-math is the default.
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-mf16c", "-mfma", "-shared", "-fPIC",
           "-o", OUT + ".tmp", SRC, "-lm"]
    subprocess.run(cmd, check=True)
    os.replace(OUT + ".tmp", OUT)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
