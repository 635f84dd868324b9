"""Build the CPU oracle (and oracle/_ref when the reference checkout exists).

Test infrastructure: called by the build entry point and by the test session
set-up, never by the product path.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DEFAULT = "/root/reference"


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_oracle(force: bool = False) -> str:
    """Compile tcab_oracle.c into oracle/liboracle.so and return its path."""
    so = os.path.join(HERE, "liboracle.so")
    src = os.path.join(HERE, "tcab_oracle.c")
    if force or not _newer(so, src, os.path.join(HERE, "Makefile")):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def build_ref(ref_root: str = REF_DEFAULT, force: bool = False) -> str | None:
    """Compile the reference's host-compilable pieces into oracle/_ref/.

    Returns the directory, or None when the reference checkout is absent (the
    prebuilt files, if any, are then used as they are).
    """
    out = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_root, "runtime", "tca")):
        return out if os.path.exists(os.path.join(out, "libtcaref.so")) else None
    so = os.path.join(out, "libtcaref.so")
    exe = os.path.join(out, "cpu_tests")
    if force or not (_newer(so, os.path.join(HERE, "ref_driver.cpp")) and os.path.exists(exe)):
        subprocess.run(["make", "-C", HERE, "ref", f"REF={ref_root}"], check=True,
                       stdout=subprocess.DEVNULL)
    return out


if __name__ == "__main__":
    print(build_oracle(force=True))
    print(build_ref(force=True))
