"""Stages the reference's own CPU implementation of the bound pass under oracle/_ref/.

TEST AND BASELINE INFRASTRUCTURE ONLY.  Nothing in the faith_b200 package imports from here.

The reference (BoyuanFeng/Faith) is plain Python for this path, so "building" it means placing
the files it needs where the GPU box can see them: oracle/_ref/ is ignored by git (the reference's
sources never enter this repository's history) but travels with the working tree.  What is staged,
unchanged and under the same relative paths:

    Transformer_Verification_Code/Verifiers/*.py        Bounds, Verifier, VerifierForward, utils and
                                                         the modules the package __init__ imports
    HandTunedKernels/kernel_test/transformer_forward_test_bound.py   the kernel parity test

Usage:   python oracle/stage_reference.py [path of the reference checkout]
The checkout is taken from the argument, else from the environment variable FAITH_REFERENCE, else
from a directory named `reference` beside this repository.  Without a checkout the script does
nothing and returns 1; whatever was staged earlier stays in place.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
DEST = os.path.join(HERE, "_ref")

STAGED = [
    ("Transformer_Verification_Code/Verifiers", ".py"),
    ("HandTunedKernels/kernel_test/transformer_forward_test_bound.py", None),
]


def find_checkout(arg=None):
    for cand in (arg, os.environ.get("FAITH_REFERENCE"), os.path.join(os.path.dirname(REPO), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "Transformer_Verification_Code", "Verifiers", "Bounds.py")):
            return os.path.abspath(cand)
    return None


def staged_root():
    """Path of the staged copy if it is complete, else None."""
    ok = os.path.isfile(os.path.join(DEST, "Transformer_Verification_Code", "Verifiers", "Bounds.py")) and \
        os.path.isfile(os.path.join(DEST, "HandTunedKernels", "kernel_test", "transformer_forward_test_bound.py"))
    return DEST if ok else None


def stage(checkout=None):
    src_root = find_checkout(checkout)
    if src_root is None:
        return None
    if os.path.abspath(src_root) == os.path.abspath(DEST):
        return DEST
    for rel, ext in STAGED:
        src = os.path.join(src_root, rel)
        dst = os.path.join(DEST, rel)
        if os.path.isdir(src):
            os.makedirs(dst, exist_ok=True)
            for name in sorted(os.listdir(src)):
                if ext is None or name.endswith(ext):
                    shutil.copyfile(os.path.join(src, name), os.path.join(dst, name))
        else:
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            shutil.copyfile(src, dst)
    return DEST


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "no reference checkout found; nothing staged")
    sys.exit(0 if out else 1)
