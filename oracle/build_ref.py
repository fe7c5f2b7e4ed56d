"""Compile the reference's own inference kernels, from its sources where they lie, into oracle/_ref/.

TEST INFRASTRUCTURE ONLY. The reference builds kernels/qwen.cu to PTX with
`nvcc --ptx -O3 -arch=compute_86 -lineinfo -DQWEN_27B` (build.rs:5-21,36) and lets the driver JIT it; this recipe
runs the same command on the unmodified sources and writes oracle/_ref/qwen27b.ptx. No reference source is copied
into this repository; the PTX is a build output (git-ignored) that travels to the GPU box with the working tree.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "qwen27b.ptx")
# the same PTX assembled ahead of time for sm_100a (what the driver's JIT would do at load time on a B200)
CUBIN = os.path.join(HERE, "_ref", "qwen27b.cubin")


def build(reference: str | None = None, force: bool = False) -> str | None:
    # the reference checkout: $QWENNY_REFERENCE, else the directory `reference` beside this repository
    if reference is None:
        reference = os.environ.get("QWENNY_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    src = os.path.join(reference, "kernels", "qwen.cu")
    if not os.path.exists(src):
        return OUT if os.path.exists(OUT) else None
    if os.path.exists(OUT) and not force and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = ["nvcc", "--ptx", "-O3", "-arch=compute_86", "-lineinfo", "-DQWEN_27B", src, "-o", OUT]
    subprocess.run(cmd, check=True)
    subprocess.run(["ptxas", "-arch=sm_100a", "-O3", "-lineinfo", OUT, "-o", CUBIN], check=True)
    return OUT


if __name__ == "__main__":
    p = build(force="--force" in sys.argv)
    print(p or "reference sources not found and no prebuilt PTX")
