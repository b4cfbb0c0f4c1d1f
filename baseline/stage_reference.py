"""Stages the reference's own scan modules (its `gqa25/*.py`, unmodified) into `baseline/_ref/gqa25/`, a directory
that git ignores, so that the reference's runtime-compiled CUDA scan (`slotkern_cuda.kv_scan_c`) can be timed on the
same GPU as this library (`baseline/time_reference_kernel.py`, called by `bench.py`).  The reference is a flat tree of
Python files with no package metadata, so `pip install --target` has nothing to install; a plain copy is what that
install would have produced.  Nothing under `baseline/_ref/` is imported by the product.

usage: python baseline/stage_reference.py [path of the reference checkout]
       (default: $SLOTSCAN_REFERENCE, else the directory `reference` beside this repository)"""
import glob
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "gqa25")


def reference_root(arg=None):
    cands = [arg, os.environ.get("SLOTSCAN_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "gqa25", "slotkern_cuda.py")):
            return c
    return None


def stage(arg=None):
    """Returns the number of files staged (0 when no reference checkout is reachable: nothing is changed then)."""
    root = reference_root(arg)
    if root is None:
        return 0
    os.makedirs(DEST, exist_ok=True)
    n = 0
    for src in sorted(glob.glob(os.path.join(root, "gqa25", "*.py"))):
        shutil.copyfile(src, os.path.join(DEST, os.path.basename(src)))
        n += 1
    return n


if __name__ == "__main__":
    print("staged %d files into %s" % (stage(sys.argv[1] if len(sys.argv) > 1 else None), DEST))
