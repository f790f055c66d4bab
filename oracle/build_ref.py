"""Recipe for oracle/_ref: the reference's own CPU implementation of the hot path.  TEST / BENCH INFRASTRUCTURE.

andylolu2/sparse-dropout's CPU path is three pure-Python files on top of PyTorch (paths inside that project):

    flash_dropout/functional/naive.py           blockwise_dropout_matmul_mask  (the masked-dense product)
    flash_dropout/functional/utils.py           blockwise_dropout_mask, mask_to_increment_table
    flash_dropout/functional/im2col_conv2d.py   im2col_conv2d

This script places unmodified copies of them, as package ``flash_dropout_reference.functional``, under the
git-ignored directory oracle/_ref/ (they are build outputs of this recipe, never part of the repository's history).
The package's own ``__init__`` files are empty stand-ins: the reference's import its CUDA and Triton front ends,
which are not part of the CPU path.  utils.py imports triton at module level; the image ships it.

    python oracle/build_ref.py /path/to/sparse-dropout

Used by oracle/cpu_path.py (timing the reference itself, ``kind: "reference"``) and by tests that compare the
restatement in oracle/masked_dense.py with the reference's functions.  Nothing in the product imports it.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = ("naive.py", "utils.py", "im2col_conv2d.py")


def build(ref_root: str) -> bool:
    """Returns True if oracle/_ref was (re)written, False if the reference checkout is not there."""
    src = os.path.join(ref_root, "flash_dropout", "functional")
    if not all(os.path.isfile(os.path.join(src, f)) for f in FILES):
        return False
    dst = os.path.join(REF_DIR, "flash_dropout_reference", "functional")
    os.makedirs(dst, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    for d in (os.path.dirname(dst), dst):
        with open(os.path.join(d, "__init__.py"), "w") as fh:
            fh.write("")
    return True


def load():
    """The reference's ``functional`` modules (naive, utils, im2col_conv2d) from oracle/_ref, or None if absent."""
    pkg = os.path.join(REF_DIR, "flash_dropout_reference", "functional")
    if not all(os.path.isfile(os.path.join(pkg, f)) for f in FILES):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import importlib
    return {name: importlib.import_module(f"flash_dropout_reference.functional.{name}")
            for name in ("naive", "utils", "im2col_conv2d")}


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/build_ref.py /path/to/sparse-dropout")
    print("oracle/_ref written" if build(sys.argv[1]) else "reference checkout not found: nothing written")
