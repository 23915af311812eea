"""Recipe for ``oracle/_ref/``: the reference's own arch-generic pieces, taken from the reference
checkout where it lies, for use as a checker on a GPU machine.  TEST INFRASTRUCTURE ONLY - the
product never imports anything under ``oracle/``.

Two files of the reference can run on an NVIDIA GPU unchanged:

* ``sageattention/triton_backend.py`` - its default back-end (``sageattn`` ``:488-530``,
  ``per_block_int8`` ``:248-298``); the ``else`` branch of its autotune list (``:64-73``) serves
  every non-AMD target.  It needs a GPU driver at import (``:13``), so it cannot run on a
  CPU-only machine.
* ``test_sageattn_rdna3.py`` - its 36 pytest cases, which import ``sageattn`` from whatever
  ``sageattention`` package is on the path.

``python oracle/make_ref.py [reference_dir]`` copies them into ``oracle/_ref/`` (git-ignored: the
reference's sources never enter this repository's history) and does nothing when the reference
checkout is absent.  Nothing is compiled: the native back-end of the reference is HIP/gfx11 only.
"""
from __future__ import annotations

import importlib.util
import os
import shutil
import sys
from pathlib import Path

ORACLE_DIR = Path(__file__).resolve().parent
REF_OUT = ORACLE_DIR / "_ref"
# where a checkout of the reference lies: SAGE_REFERENCE_DIR, else a sibling of this repository
DEFAULT_REFERENCE = Path(os.environ.get("SAGE_REFERENCE_DIR", str(ORACLE_DIR.parent.parent / "reference")))
FILES = {
    "sageattention/triton_backend.py": "ref_triton_backend.py",
    "test_sageattn_rdna3.py": "test_sageattn_rdna3.py",
}


def make_ref(reference_dir: Path = DEFAULT_REFERENCE) -> bool:
    """Returns True when ``oracle/_ref/`` holds the files afterwards."""
    reference_dir = Path(reference_dir)
    if not reference_dir.is_dir():
        return have_ref()
    REF_OUT.mkdir(exist_ok=True)
    for src, dst in FILES.items():
        shutil.copyfile(reference_dir / src, REF_OUT / dst)
    return True


def have_ref() -> bool:
    return all((REF_OUT / name).exists() for name in FILES.values())


def load_ref_triton():
    """Import the reference's Triton back-end from ``oracle/_ref`` under its own module name (the
    name ``sageattention`` belongs to the drop-in).  Needs a GPU driver."""
    path = REF_OUT / "ref_triton_backend.py"
    if not path.exists():
        raise FileNotFoundError(f"{path} is missing: run `python oracle/make_ref.py` where the reference checkout is")
    spec = importlib.util.spec_from_file_location("ref_triton_backend", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_triton_backend"] = mod
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ok = make_ref(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_REFERENCE)
    print(f"oracle/_ref {'ready' if ok else 'not made: no reference checkout'}")
