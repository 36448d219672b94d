"""Builds ``libwtconv_b200.so`` in-tree with nvcc for sm_100a (``python -m wtconv_b200.build``)."""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))


def build(jobs: int | None = None, verbose: bool = False) -> str:
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), f"-j{jobs}"]
    res = subprocess.run(cmd, capture_output=not verbose, text=True)
    if res.returncode != 0:
        sys.stderr.write((res.stdout or "") + (res.stderr or ""))
        raise RuntimeError("building libwtconv_b200.so failed")
    return os.path.join(_HERE, "libwtconv_b200.so")


if __name__ == "__main__":
    print(build(verbose=True))
