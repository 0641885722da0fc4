"""Test infrastructure: puts a runnable copy of the reference's own Python modules for the quantization path under
``oracle/_ref/`` (ignored by git, never imported by the product), so that the CPU arm of the benchmark can time the
reference's classes themselves on a machine where the reference checkout is not mounted.

    python oracle/make_ref.py [/path/to/gptq_plus_mp_quant]

(default: ``REALQ_REFERENCE_ROOT``, else a checkout named ``reference`` beside this repository)

Copied as they are: ``utils/*.py``, ``utils/had_mat.pt`` and ``gptq_utils/*.py`` (the classes import each other
across these two packages).  Nothing is edited; ``oracle/ref_loader.py`` supplies the same accommodations as the
golden-fixture script (stub ``accelerate``, import ``transformers`` first)."""
from __future__ import annotations

import glob
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def build(ref_root: str | None = None) -> str | None:
    ref_root = ref_root or os.environ.get("REALQ_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(HERE)), "reference")
    if not os.path.isdir(os.path.join(ref_root, "gptq_utils")):
        return None
    for pkg in ("utils", "gptq_utils"):
        os.makedirs(os.path.join(DEST, pkg), exist_ok=True)
        for src in glob.glob(os.path.join(ref_root, pkg, "*.py")) + glob.glob(os.path.join(ref_root, pkg, "*.pt")):
            dst = os.path.join(DEST, pkg, os.path.basename(src))
            shutil.copyfile(src, dst)
            os.chmod(dst, 0o644)
    return DEST


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "reference checkout not found: nothing copied")
