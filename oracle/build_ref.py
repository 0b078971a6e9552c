"""Recipe that makes the reference's own CPU code for this path available to the checker.

    python oracle/build_ref.py [/path/to/reference/checkout]

The reference's executable weight spec is one plain Python file, paired_nvfp4_kernels/reference.py (prune,
quantize, pack, dequantize).  Nothing has to be compiled: the recipe places that file, unmodified, under
oracle/_ref/ (a git-ignored output folder, like a built library: it travels to the GPU box with the working tree
but never enters history), where bench.py's CPU baseline and reference arm load it by path for the weight
half of their work.  Without a checkout (the GPU box has none) the recipe does nothing and whatever an earlier
run placed stays in use.  The reference's GPU path cannot be built: it needs the CUTLASS v4.8.0 submodule, which
is empty in the checkout, and a GPU.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")


def build(reference_root="/root/reference", verbose=True):
    src = os.path.join(reference_root, "paired_nvfp4_kernels", "reference.py")
    if not os.path.exists(src):
        if verbose:
            print(f"oracle/_ref: no reference checkout at {reference_root}; nothing placed")
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    dst = os.path.join(OUT_DIR, "reference.py")
    shutil.copyfile(src, dst)
    if verbose:
        print(f"oracle/_ref: placed {dst}")
    return dst


if __name__ == "__main__":
    build(*(sys.argv[1:2]))
