"""Stage the reference's own Python package so that it can run where its checkout is absent.  TEST INFRASTRUCTURE.

The reference (w4096/mini-vllm) is pure Python.  Its package directory ``minivllm/`` is copied, file for
file and unmodified, into ``oracle/_ref/minivllm`` - a directory that is ignored by version control and
travels only with a working-tree snapshot.  ``oracle/reference_engine.py`` imports it from there to run
the reference's Scheduler, Executor, packing and model code as the checker of the token-identity test
and of the fixtures under ``tests/golden/``.

    python -m oracle.stage_reference [path/to/mini-vllm]

Without an argument the checkout is looked for next to this repository (a sibling directory called
``reference``).  Nothing happens, and ``None`` is returned, when there is no checkout.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


def staged_package() -> Path | None:
    """The staged ``minivllm`` package directory, if it has been staged."""
    p = DEST / "minivllm"
    return p if (p / "executor" / "executor.py").exists() else None


def stage(checkout: str | Path | None = None) -> Path | None:
    src = Path(checkout) if checkout else HERE.parent.parent / "reference"
    pkg = src / "minivllm"
    if not (pkg / "executor" / "executor.py").exists():
        return staged_package()
    DEST.mkdir(exist_ok=True)
    dst = DEST / "minivllm"
    if dst.exists():
        shutil.rmtree(dst)
    shutil.copytree(pkg, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return dst


if __name__ == "__main__":
    out = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "no reference checkout found; nothing staged")
