"""Puts the reference's own fake-quant implementation of the path where the CPU baseline can run it.

    python oracle/make_ref.py [/path/to/reference]

Copies the five Python files the path needs (args.py and utils/{quant_matmul, hadamard_matmul,
utils, plot}.py), unmodified, from the reference checkout into ``oracle/_ref/``.  That folder is
listed in .gitignore: the copies never enter this repository's history, they only sit beside the
built libraries so that a machine without the reference checkout (the GPU box) can time the
reference's CPU path on its own host cores.  ``oracle/reference_arm.py`` imports them from there.
TEST / BENCHMARK INFRASTRUCTURE ONLY: nothing under ``hot_b200/`` reads this folder.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
FILES = ["args.py", "utils/quant_matmul.py", "utils/hadamard_matmul.py", "utils/utils.py", "utils/plot.py"]


def make(ref_root: str = "/root/reference", out: str = OUT) -> bool:
    """Returns True when the copies are in place (False if the reference checkout is absent)."""
    if not os.path.isfile(os.path.join(ref_root, FILES[1])):
        return False
    lines = []
    for rel in FILES:
        src, dst = os.path.join(ref_root, rel), os.path.join(out, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
        with open(dst, "rb") as f:
            lines.append("%s  %s" % (hashlib.sha256(f.read()).hexdigest(), rel))
    with open(os.path.join(out, "MANIFEST.sha256"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return True


if __name__ == "__main__":
    ok = make(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    print("oracle/_ref ready" if ok else "reference checkout not found: nothing copied")
