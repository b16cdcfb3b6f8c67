"""Stages an importable copy of the reference package next to the oracle — TEST INFRASTRUCTURE.

    python oracle/make_ref.py <reference checkout>

The reference (ai-compiler-study/triton-kernels) is pure Python: its Triton kernels are compiled
by Triton at first call on the GPU.  Its setup.py lists only the top-level package
(setup.py:18-20), so a `pip install --target` of it leaves out `kernels/`, `modules/`, `flux/`,
`functional/` and cannot be imported.  This recipe copies the package directory as it lies in the
checkout into `oracle/_ref/triton_kernels/` (git-ignored: the copy never enters this
repository's history) so that machines without the checkout can still run the reference's own
kernels for head-to-head parity and timing.

Only tests/ and bench.py's reference arms import from `oracle/_ref`; nothing under
triton_kernels_b200/ does.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"


def stage(reference_checkout: str | Path) -> Path:
    src = Path(reference_checkout) / "triton_kernels"
    if not (src / "__init__.py").exists():
        raise FileNotFoundError(f"{src} is not the reference's package directory")
    dst = REF_DIR / "triton_kernels"
    if dst.exists():
        shutil.rmtree(dst)
    REF_DIR.mkdir(exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return dst


def import_reference():
    """The staged reference package (`triton_kernels`), or None when it has not been staged."""
    if not (REF_DIR / "triton_kernels" / "__init__.py").exists():
        return None
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import triton_kernels  # noqa: PLC0415

    return triton_kernels


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(stage(sys.argv[1]))
