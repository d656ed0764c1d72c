"""Installs the reference's CPU implementation of the hot path under ``baseline/_ref``.

The reference project has no installable package (no setup.py / pyproject); its CPU
route for this path is three pure-Python files that import each other as
``kernel.*``.  This script copies exactly those files, unmodified, from the
reference tree into ``baseline/_ref/kernel/`` (a git-ignored directory: the files
never enter this repository's history) and adds empty ``__init__.py`` files so
that ``sys.path.insert(0, 'baseline/_ref'); import kernel.tools.parity...`` works.
``bench.py --impl reference`` and the ``cpu_baseline`` leg then time the
reference's own functions (``kind: "reference"``); without the install they fall
back to the oracle's restatement (``kind: "port"``).

    python baseline/install_reference.py [/path/to/reference]
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = [
    "triton_kernel/pack_utils.py",
    "tools/parity/quant_reference.py",
    "tools/parity/fp16_reference.py",
]


def install(reference_root: str = "/root/reference") -> bool:
    """Returns True when the files are in place afterwards."""
    dst_root = os.path.join(HERE, "_ref", "kernel")
    if not os.path.isdir(reference_root):
        return all(os.path.exists(os.path.join(dst_root, f)) for f in FILES)
    for rel in FILES:
        src = os.path.join(reference_root, rel)
        dst = os.path.join(dst_root, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
    for d in ("", "triton_kernel", "tools", "tools/parity"):
        init = os.path.join(dst_root, d, "__init__.py")
        if not os.path.exists(init):
            open(init, "w").close()
    return True


if __name__ == "__main__":
    ok = install(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    print("installed" if ok else "reference tree not found; nothing installed")
