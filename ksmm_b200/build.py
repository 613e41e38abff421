"""Builds libksmm_cu.so in-tree with nvcc for sm_100a (`python -m ksmm_b200.build`)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")


def build_library(jobs=None, verbose=False):
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", CSRC, f"-j{jobs}"]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building libksmm_cu.so failed")
    lib = os.path.join(HERE, "libksmm_cu.so")
    if not os.path.exists(lib):
        raise RuntimeError(f"{lib} was not produced")
    return lib


if __name__ == "__main__":
    print(build_library(verbose=True))
