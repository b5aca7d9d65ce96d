"""Compile the C oracle (``come_oracle.c``) into ``libcome_oracle.so`` next to this file.

Test infrastructure: used by the CPU tests, the smoke check and the CPU-baseline leg of the benchmark.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "come_oracle.c")
LIB = os.path.join(HERE, "libcome_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", SRC, "-o", LIB, "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
