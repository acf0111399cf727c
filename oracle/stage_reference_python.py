"""Stages the reference's Python package for runs on a GPU box.  TEST INFRASTRUCTURE ONLY.

    python oracle/stage_reference_python.py /path/to/electrock-infer
    ELECTROCK_REFERENCE=/path/to/electrock-infer python oracle/stage_reference_python.py

The reference source tree exists only where this repository was developed; the machines with GPUs
receive this repository alone.  This script copies, byte for byte, the reference's importable
package ``electrock_infer/`` (Python files only) into ``oracle/_ref/reference_python/``, which is
git-ignored like the compiled reference ops beside it: nothing of it enters the history, and
nothing in the product package knows about it.  Two consumers read the staged copy, both optional
and both skipped when it is absent:

  * ``oracle/gpu_reference.py``   the reference's own Triton MoE pipeline timed on the GPU
  * ``oracle/reference_engine.py``  the reference's engine generating with this library's layer
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref" / "reference_python"


def main() -> int:
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ELECTROCK_REFERENCE")
    if not where:
        print("give the path of the electrock-infer source tree as the first argument or in "
              "ELECTROCK_REFERENCE; nothing staged")
        return 2
    src = Path(where) / "electrock_infer"
    if not src.is_dir():
        print(f"{src} not found; nothing staged")
        return 0
    if OUT_DIR.exists():
        shutil.rmtree(OUT_DIR)
    count = 0
    for path in sorted(src.rglob("*.py")):
        dst = OUT_DIR / "electrock_infer" / path.relative_to(src)
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(path, dst)
        count += 1
    print(f"staged {count} files under {OUT_DIR}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
