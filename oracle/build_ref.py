"""Recipe that brings the reference itself beside the oracle, as `oracle/_ref/mlops`.

TEST / BENCH INFRASTRUCTURE ONLY: nothing in `mlops_b200` imports it.

als244/mlops is pure Python (no compiled sources of its own), so "building" it is a copy of
its package tree `src/mlops` from a checkout of the reference into `oracle/_ref/`, which is
listed in `.gitignore` (it never enters this repository's history) and travels with the
working tree to a GPU machine. Importing it there needs torch only; its Triton kernels (the
builtin provider's CUDA path, `mlops.kernels.block_fp8.grouped_block_gemm`) compile on first
use when Triton is installed.

    python oracle/build_ref.py [path/to/reference]      # default: $MLOPS_REFERENCE or ../reference

`reference()` returns the imported `mlops` package from `oracle/_ref` (or from
`$MLOPS_REFERENCE_SRC` when set), or None where neither exists.
"""

from __future__ import annotations

import importlib
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def _default_checkout() -> Path | None:
    named = os.environ.get("MLOPS_REFERENCE")
    candidates = [Path(named)] if named else []
    candidates.append(HERE.parent.parent / "reference")
    for candidate in candidates:
        if (candidate / "src" / "mlops" / "__init__.py").exists():
            return candidate
    return None


def build(checkout: str | os.PathLike | None = None, force: bool = False) -> Path | None:
    """Copies `<checkout>/src/mlops` to `oracle/_ref/mlops`. Returns the target folder, the
    existing one when no checkout is at hand, or None when there is neither."""
    source = Path(checkout) if checkout is not None else _default_checkout()
    package = TARGET / "mlops"
    if source is None or not (source / "src" / "mlops").exists():
        return TARGET if package.exists() else None
    stamp = TARGET / "SOURCE"
    origin = str((source / "src" / "mlops").resolve())
    if package.exists() and not force and stamp.exists() and stamp.read_text() == origin:
        return TARGET
    if package.exists():
        shutil.rmtree(package)
    TARGET.mkdir(exist_ok=True)
    shutil.copytree(source / "src" / "mlops", package, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    stamp.write_text(origin)
    return TARGET


def reference():
    """The reference package, imported; None where it is not available."""
    if "mlops" in sys.modules:
        return sys.modules["mlops"]
    override = os.environ.get("MLOPS_REFERENCE_SRC")
    root = Path(override) if override else TARGET
    if not (root / "mlops" / "__init__.py").exists():
        return None
    sys.dont_write_bytecode = True
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    return importlib.import_module("mlops")


if __name__ == "__main__":
    where = build(sys.argv[1] if len(sys.argv) > 1 else None, force=True)
    print(where if where is not None else "no reference checkout found")
