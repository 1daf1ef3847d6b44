"""Places the reference's own CPU path under oracle/_ref/ (TEST INFRASTRUCTURE, not product).

The reference is plain Python: nothing to compile.  This recipe copies, byte for byte, the files of a reference
checkout that its CPU path and its callers consist of - torch_funcs/ (the four *_baseline functions), utils.py,
models/wrappers.py, layer.py, network.py, roofline.py, device.py and configs/ - into oracle/_ref/, which .gitignore
lists: the copy never enters the history, but it travels with the working tree to a machine that has no reference
checkout, where the tests and `bench.py --impl reference` import it.

    python oracle/make_ref.py /path/to/reference

Only tests/, bench.py's cpu_baseline / --impl reference legs and __graft_entry__ use what lands here.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
FILES = ["utils.py", "layer.py", "network.py", "roofline.py", "device.py", "models/__init__.py", "models/wrappers.py"]
DIRS = ["torch_funcs", "configs"]


def make(ref_root: str) -> str:
    if not os.path.isdir(os.path.join(ref_root, "torch_funcs")):
        raise SystemExit(f"{ref_root} is not a reference checkout (no torch_funcs/)")
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(DEST)
    for d in DIRS:
        shutil.copytree(os.path.join(ref_root, d), os.path.join(DEST, d), ignore=shutil.ignore_patterns("__pycache__"))
    for f in FILES:
        src = os.path.join(ref_root, f)
        if os.path.exists(src):
            dst = os.path.join(DEST, f)
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            shutil.copyfile(src, dst)
    return DEST


def available() -> bool:
    return os.path.isfile(os.path.join(DEST, "torch_funcs", "blast_funcs.py"))


def import_path() -> str:
    """Directory to put on sys.path so that `import torch_funcs`, `import utils`, `import models.wrappers` resolve to
    the reference's files."""
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(make(sys.argv[1]))
