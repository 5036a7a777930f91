"""Builds the CPU oracle (test infrastructure) into oracle/libullis_oracle.so.

The reference crate is Rust and `rustc`/`cargo` are not available, so there is
no `oracle/_ref` build of the reference's own sources; the C restatement in
ullis_oracle.c is the only CPU arm.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ullis_oracle.c")
OUT = os.path.join(HERE, "libullis_oracle.so")


def build(force: bool = False) -> str:
    if (not force and os.path.exists(OUT)
            and os.path.getmtime(OUT) >= os.path.getmtime(SRC)):
        return OUT
    cmd = [
        "gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-fopenmp",
        # keep the reference's unfused multiply/add and IEEE semantics
        "-ffp-contract=off", "-fno-fast-math", "-mavx2", "-mno-fma",
        "-fvisibility=hidden", "-Wall", "-Wextra",
        SRC, "-o", OUT, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
