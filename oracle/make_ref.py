"""Mirror the reference's model sources, unmodified, into the git-ignored ``oracle/_ref/``.  TEST / BENCHMARK
INFRASTRUCTURE ONLY.

    python oracle/make_ref.py            (where the reference tree exists)

The benchmark's reference arm (``bench.py --impl reference``) and the live oracle pin time / check the
reference's OWN ``training_step``; the machine that runs the benchmark has no copy of the reference project,
so the handful of pure-Python files of its model package travel with the build outputs instead
(``oracle/_ref/`` is listed in ``.gitignore``: nothing of the reference enters the history).  The reference's
own packaging cannot be used offline (its build backend, hatchling, is not installed), hence this plain
byte-for-byte mirror of

    crosslayer_transcoder/model/*.py      crosslayer_transcoder/metrics/*.py
    crosslayer_transcoder/data/shared_memory.py   (the activation store whose consumer the ingestion tests
                                                   and the benchmark's ingestion comparison run against)

``oracle/ref_import.py`` imports them from the reference tree when it is present and from this mirror
otherwise.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

SRC = Path(os.environ.get("CLT_REFERENCE_ROOT", "/root/reference"))
DST = Path(__file__).resolve().parent / "_ref"
SUBDIRS = ("model", "metrics")
FILES = ("data/shared_memory.py",)


def make(verbose: bool = True) -> bool:
    """Returns True when the mirror exists afterwards."""
    base = SRC / "crosslayer_transcoder"
    if not (base / "model" / "clt.py").exists():
        if verbose:
            print(f"reference tree not found at {SRC}; keeping {DST} as it is")
        return (DST / "crosslayer_transcoder" / "model" / "clt.py").exists()
    for sub in SUBDIRS:
        out = DST / "crosslayer_transcoder" / sub
        out.mkdir(parents=True, exist_ok=True)
        for f in sorted((base / sub).glob("*.py")):
            shutil.copyfile(f, out / f.name)
    for rel in FILES:
        out = DST / "crosslayer_transcoder" / rel
        out.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(base / rel, out)
    if verbose:
        print(f"mirrored {', '.join(SUBDIRS + FILES)} of {base} into {DST}")
    return True


if __name__ == "__main__":
    sys.exit(0 if make() else 1)
