"""Place the unmodified reference package under oracle/_ref/ (test and benchmark infrastructure).

    python oracle/make_ref.py            # reads $BONGARD_REFERENCE, default: ../reference beside this repository

The reference is a pure-Python wheel whose only content is the `bongard` package
(`[tool.hatch.build.targets.wheel] packages = ["bongard"]` in its pyproject.toml).  Its build
backend (hatchling) is not available offline, so `pip install --target` cannot run; this script
produces the same installed tree by copying the package directory as it lies, byte for byte, plus
the licence.  oracle/_ref/ is listed in .gitignore: the copy never enters this repository's
history, it only travels with a working tree to the machine that runs the GPU tests, exactly as
the built shared library does.

What uses it: the drop-in tests (the reference's own JudgmentModel / forward_packed / Predictor
running over the substituted B200 modules) and the CPU arm of bench.py (the reference's
device="cpu" Predictor).  Nothing under bongard_b200/ imports it.
"""

import filecmp
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / '_ref'


def source():
    return Path(os.environ.get('BONGARD_REFERENCE', str(HERE.parents[1] / 'reference')))


def make(force=False):
    """Copy <reference>/bongard to oracle/_ref/bongard.  Returns the target, or None when no
    reference checkout is present (the prebuilt tree, if any, is left alone)."""
    src = source()
    package = src / 'bongard'
    if not (package / '__init__.py').exists():
        return TARGET if (TARGET / 'bongard' / '__init__.py').exists() else None
    dst = TARGET / 'bongard'
    if dst.exists() and not force:
        same = filecmp.dircmp(package, dst, ignore=['__pycache__'])
        if not (same.left_only or same.right_only or same.diff_files):
            return TARGET
    if dst.exists():
        shutil.rmtree(dst)
    TARGET.mkdir(parents=True, exist_ok=True)
    shutil.copytree(package, dst, ignore=shutil.ignore_patterns('__pycache__'))
    for extra in ('LICENSE', 'pyproject.toml'):
        if (src / extra).exists():
            shutil.copy2(src / extra, TARGET / extra)
    return TARGET


if __name__ == '__main__':
    out = make(force='--force' in sys.argv)
    print(out if out else 'no reference checkout found; nothing copied')
